"""The attention block's host bookkeeping (tc_kv_session): a small multi-layer "engine"
driven the way GPUModel drives its attention block -- prefill, decode, a second session after
clear, chunked prefill, the window guard -- in all KV modes, against the oracle run on the
full history."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu

NH, NKV, HD, SLOTS, WINDOW = 8, 2, 128, 2, 256


class Engine:
    """A toy caller: every 'layer' gets its own seeded q/k/v rows per token."""

    def __init__(self, mode, seed, rope=False, scratch_rows=0, hd=HD):
        self.mode, self.seed, self.hd = mode, seed, hd
        self.tables = oracle.rope_tables(WINDOW, self.hd, 1e6) if rope else None
        rp = tuple(dev(t) for t in self.tables) if rope else None
        self.s = ops.KvSession(NH, NKV, self.hd, WINDOW, SLOTS, mode=mode, rope=rp, prefill_scratch_rows=scratch_rows)
        self.hist = [([], []) for _ in range(SLOTS)]     # what every slot's store should hold

    def rows(self, slot, pos, n):
        r = np.random.default_rng([self.seed, slot, pos])
        return (r.standard_normal((n, NH, self.hd), dtype=np.float32), r.standard_normal((n, NKV, self.hd), dtype=np.float32),
                r.standard_normal((n, NKV, self.hd), dtype=np.float32))

    def forward(self, n, graph_capture=False, dev_pos=False):
        pos = self.s.begin(n)
        outs, wants = [], []
        for slot in range(SLOTS):
            q, k, v = self.rows(slot, pos, n)
            dq = dev(q)
            out = torch.full((n, NH, self.hd), float("nan"), device="cuda")
            dp = torch.tensor([pos], dtype=torch.int32, device="cuda") if dev_pos else None
            self.s.attend(slot, dq, dev(k), dev(v), out, pos, dev_pos=dp, graph_capture=graph_capture)
            if self.tables is not None:
                q = oracle.rope_q(q, self.tables[0], self.tables[1], n, NH, self.hd, pos)
                kk = np.zeros((pos + n, NKV, self.hd), np.float32)
                vv = np.zeros_like(kk)
                oracle.kv_append(k, v, kk, vv, n, NKV, self.hd, pos, ropePos=pos, cosT=self.tables[0], sinT=self.tables[1])
                k = kk[pos:]
                assert np.array_equal(host(dq), q), "q is rotated in place"
            self.hist[slot][0].append(k)
            self.hist[slot][1].append(v)
            K = np.concatenate(self.hist[slot][0])
            V = np.concatenate(self.hist[slot][1])
            inv = 1.0 / math.sqrt(self.hd)
            if self.mode == "i8" or (self.mode == "f32+i8" and n == 1 and not graph_capture and not dev_pos):
                k8, v8, ks, vs = oracle.quant_kv8(K, V, NKV, self.hd)
                want = oracle.attention_i8(q, k8, v8, ks, vs, n, NH, NKV, self.hd, pos, inv)
            elif self.mode == "f16":
                want = oracle.attention_kv(q, K.astype(np.float16), V.astype(np.float16), n, NH, NKV, self.hd, pos, inv)
            else:
                want = oracle.attention_kv(q, K, V, n, NH, NKV, self.hd, pos, inv)
            outs.append(host(out))
            wants.append(want)
        self.s.commit(n)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        return outs, wants

    def clear(self):
        self.s.clear()
        self.hist = [([], []) for _ in range(SLOTS)]
        self.seed += 1000     # a new conversation: different rows


def _check(outs, wants, what, tol=None):
    for slot, (o, w) in enumerate(zip(outs, wants)):
        kw = dict(rtol=tol[0], atol=tol[1]) if tol else {}
        assert_close(o, w, what=f"{what}, slot {slot}", **kw)


@pytest.mark.parametrize("mode", ["f32", "f32+i8", "i8", "f16"])
def test_prefill_then_decode_then_a_second_conversation(mode):
    e = Engine(mode, seed=1)
    _check(*e.forward(37), f"{mode}: prompt")
    assert e.s.pos == 37
    if mode == "f32+i8":
        assert e.s.rows8(0) == 0 and e.s.rows8(1) == 0, "a prefill without scratch writes f32 rows only"
    for t in range(3):
        _check(*e.forward(1), f"{mode}: decode {t}")
    if mode in ("f32+i8", "i8"):
        assert e.s.rows8(0) == 40 and e.s.rows8(1) == 40, "every slot's pool is rebuilt by its own decode"
    # a second conversation must not see rows of the first one (pool rows are not zeroed, the
    # per-slot row counts keep them out)
    e.clear()
    assert e.s.pos == 0 and e.s.rows8(0) == 0 and e.s.rows8(1) == 0
    _check(*e.forward(9), f"{mode}: second prompt")
    _check(*e.forward(1), f"{mode}: second conversation decode")
    # a follow-up chunk after decoded tokens reads the whole history
    _check(*e.forward(5), f"{mode}: follow-up rows")
    _check(*e.forward(1), f"{mode}: decode after the follow-up")


@pytest.mark.parametrize("mode", ["f32+i8", "i8", "f32"])
def test_gated_model_shape_head_dim_256(mode):
    """The reference's own int8 shape: f32 store + int8 decode pool (or int8 store) at head_dim 256."""
    e = Engine(mode, seed=21, hd=256)
    _check(*e.forward(45), f"{mode} hd256: prompt")
    for t in range(2):
        _check(*e.forward(1), f"{mode} hd256: decode {t}")
    if mode != "f32":
        assert e.s.rows8(0) == 47 and e.s.rows8(1) == 47
    _check(*e.forward(3), f"{mode} hd256: follow-up rows")
    _check(*e.forward(1), f"{mode} hd256: decode after the follow-up")


@pytest.mark.parametrize("mode", ["f32", "i8"])
def test_chunked_prefill_carries_the_cache(mode):
    """ModelForward.cpp:104-127 feeds a long prompt in chunks; every chunk resumes where the
    previous one stopped, so the last row's attention equals a single prefill's."""
    a, b = Engine(mode, seed=7), Engine(mode, seed=7)
    whole, _ = a.forward(96)
    parts = []
    for n in (40, 40, 16):
        o, w = b.forward(n)
        _check(o, w, f"{mode}: chunk")
        parts.append(o)
    # the toy engine seeds rows by (slot, position of the call), so compare against the oracle
    # per chunk (above) and the positions
    assert a.s.pos == b.s.pos == 96 and whole[0].shape[0] == 96


def test_dense_rotation_in_the_store_and_tensor_core_prefill():
    e = Engine("f32", seed=3, rope=True, scratch_rows=160)
    outs, wants = e.forward(160)      # fresh prompt, scratch given: the fp16 tensor-core prefill
    _check(outs, wants, "rope + tcgen05 prefill", tol=(2e-2, 2e-3))
    _check(*e.forward(1), "rope decode")
    _check(*e.forward(4), "rope continued rows (tensor-core prefill over the existing cache)", tol=(2e-2, 2e-3))


@pytest.mark.parametrize("hd", [128, 64, 256])
def test_chunked_prompt_stays_on_the_tensor_core_prefill(hd):
    """With scratch for the whole window every chunk of a prompt -- not only the first, as in the
    reference (GPUComputeForward.cu:3828-3835) -- takes the fp16 tensor-core prefill."""
    e = Engine("f32", seed=13, scratch_rows=96, hd=hd)
    for n in (96, 70, 33):
        _check(*e.forward(n), f"tcgen05 prefill chunk of {n}", tol=(2e-2, 2e-3))
    _check(*e.forward(1), "decode after the chunks")


@pytest.mark.parametrize("mode", ["f16", "i8"])
def test_fp16_and_int8_stores_take_the_tensor_core_prefill_with_scratch(mode):
    e = Engine(mode, seed=31, scratch_rows=96)
    for n in (96, 41):
        _check(*e.forward(n), f"{mode} store: tcgen05 prefill chunk of {n}", tol=(2e-2, 2e-3))
    _check(*e.forward(1), f"{mode} store: decode after the chunks")


def test_mirror_stays_current_through_tensor_core_prefill_chunks():
    """f32 store + int8 decode pool, scratch given: the launch that makes the fp16 twins of a chunk
    also writes the chunk's pool rows, so the first decode step finds the pool complete."""
    e = Engine("f32+i8", seed=21, scratch_rows=96)
    pos = 0
    for n in (96, 50):
        _check(*e.forward(n), f"mirror: tcgen05 prefill chunk of {n}", tol=(2e-2, 2e-3))
        pos += n
        assert e.s.rows8(0) == pos and e.s.rows8(1) == pos
    _check(*e.forward(1), "mirror: decode over a pool written by the prefill launches")
    assert e.s.rows8(0) == pos + 1


def test_graph_capture_and_device_position_choose_host_free_paths():
    e = Engine("i8", seed=5)
    _check(*e.forward(20), "i8 prompt")
    _check(*e.forward(1, graph_capture=True, dev_pos=True), "i8 decode, captured form")
    e = Engine("f32+i8", seed=6)
    _check(*e.forward(20), "mirror prompt")
    _check(*e.forward(1, graph_capture=True, dev_pos=True), "mirror decode, captured form (f32 path)")
    _check(*e.forward(1), "mirror decode after it (pool rebuilt to the position)")
    assert e.s.rows8(0) == 22


def test_window_guard_is_a_state_not_a_fault():
    e = Engine("f32", seed=9)
    e.forward(WINDOW - 2)
    e.forward(1)
    with pytest.raises(capi.ContextFull):
        e.s.begin(2)
    assert e.s.context_full and e.s.pos == WINDOW - 1
    e.forward(1)                      # exactly fills the window
    with pytest.raises(capi.ContextFull):
        e.s.begin(1)
    e.clear()
    assert not e.s.context_full
    _check(*e.forward(3), "after clear")


def test_config_guards():
    with pytest.raises(capi.TcError):
        ops.KvSession(7, 2, 128, 64, 1)          # heads not a multiple of kv heads


def test_decode_sequence_replayed_from_a_cuda_graph():
    """The graph-safe decode sequence of the int8 store: quantise-append and attention read the
    position from device memory, so ONE captured step replays for every token (the reference
    cannot capture its int8 store path: the row counts live on the host)."""
    e = Engine("i8", seed=11)
    _check(*e.forward(33), "prompt before capture")
    s = e.s
    dq = torch.zeros((1, NH, HD), device="cuda")
    dk = torch.zeros((SLOTS, 1, NKV, HD), device="cuda")
    dv = torch.zeros_like(dk)
    douts = torch.zeros((SLOTS, 1, NH, HD), device="cuda")
    dpos = torch.tensor([s.pos], dtype=torch.int32, device="cuda")
    qs = torch.zeros((SLOTS, 1, NH, HD), device="cuda")

    def step():
        for slot in range(SLOTS):
            s.attend(slot, qs[slot], dk[slot], dv[slot], douts[slot], 0, dev_pos=dpos, graph_capture=True)
        dpos.add_(1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                      # warm-up outside capture (writes row 33 with zeros, position -> 34)
    torch.cuda.current_stream().wait_stream(side)
    dpos.fill_(s.pos)               # back to the real position; the zero row is overwritten below
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    dpos.fill_(s.pos)               # capture does not execute
    inv = 1.0 / math.sqrt(HD)
    for t in range(4):
        pos = s.begin(1)
        rows = [e.rows(slot, pos, 1) for slot in range(SLOTS)]
        for slot, (q, k, v) in enumerate(rows):
            qs[slot].copy_(dev(q))
            dk[slot].copy_(dev(k))
            dv[slot].copy_(dev(v))
        g.replay()
        torch.cuda.synchronize()
        assert int(dpos.item()) == pos + 1
        for slot, (q, k, v) in enumerate(rows):
            e.hist[slot][0].append(k)
            e.hist[slot][1].append(v)
            K, V = np.concatenate(e.hist[slot][0]), np.concatenate(e.hist[slot][1])
            k8, v8, ks, vs = oracle.quant_kv8(K, V, NKV, HD)
            want = oracle.attention_i8(q, k8, v8, ks, vs, 1, NH, NKV, HD, pos, inv)
            assert_close(host(douts[slot]), want, what=f"graph replay {t}, slot {slot}")
        s.commit(1)
    assert ops.device_status() == 0


@pytest.mark.parametrize("mode", ["f32", "f16", "f32+i8"])
def test_split_decode_replayed_at_a_growing_device_position(mode):
    """A decode step on the f32 / fp16 store (also the captured form of the mirror mode) captured
    once and replayed while the position -- which lives on the device -- grows well past the
    value it had at capture time: the launch has to be sized for the window, not for the
    capture-time position (the reference's *Pos decode launches its fixed chunk grid)."""
    e = Engine(mode, seed=31)
    _check(*e.forward(33), "prompt before capture")
    s = e.s
    dk = torch.zeros((SLOTS, 1, NKV, HD), device="cuda")
    dv = torch.zeros_like(dk)
    douts = torch.zeros((SLOTS, 1, NH, HD), device="cuda")
    dpos = torch.tensor([s.pos], dtype=torch.int32, device="cuda")
    qs = torch.zeros((SLOTS, 1, NH, HD), device="cuda")

    def step():
        for slot in range(SLOTS):
            s.attend(slot, qs[slot], dk[slot], dv[slot], douts[slot], s.pos, dev_pos=dpos, graph_capture=True)
        dpos.add_(1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                      # warm-up outside capture (its zero row is overwritten below)
    torch.cuda.current_stream().wait_stream(side)
    dpos.fill_(s.pos)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    dpos.fill_(s.pos)
    inv = 1.0 / math.sqrt(HD)
    for t in range(150):            # 33 -> 183: several times the capture-time length
        pos = s.begin(1)
        rows = [e.rows(slot, pos, 1) for slot in range(SLOTS)]
        for slot, (q, k, v) in enumerate(rows):
            qs[slot].copy_(dev(q))
            dk[slot].copy_(dev(k))
            dv[slot].copy_(dev(v))
        g.replay()
        for slot, (q, k, v) in enumerate(rows):
            e.hist[slot][0].append(k)
            e.hist[slot][1].append(v)
        s.commit(1)
        if t % 10 != 9 and t not in (0, 30, 31, 32, 94, 95):
            continue
        torch.cuda.synchronize()
        assert int(dpos.item()) == pos + 1
        for slot, (q, k, v) in enumerate(rows):
            K, V = np.concatenate(e.hist[slot][0]), np.concatenate(e.hist[slot][1])
            if mode == "f16":
                K, V = K.astype(np.float16), V.astype(np.float16)
            want = oracle.attention_kv(q, K, V, 1, NH, NKV, HD, pos, inv)
            assert_close(host(douts[slot]), want, what=f"{mode}: graph replay {t} (position {pos}), slot {slot}")
    assert ops.device_status() == 0
