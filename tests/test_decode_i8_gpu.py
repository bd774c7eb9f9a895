"""int8-KV decode attention on the GPU against the oracle (tolerance 1e-3
relative / 1e-4 absolute on f32 outputs) and against double precision."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import ops, synth
from tests.util import assert_close, dev, host, make_i8_store

pytestmark = pytest.mark.gpu


def _run_single(nH, nKV, hd, ctx, numChunks, seed, extra_rows=0, dev_pos=False):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(k, v, nKV, hd, extra_rows)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8[:ctx], v8[:ctx], ks[:ctx], vs[:ctx], 1, nH, nKV, hd, ctx - 1, inv)
    exact = oracle.attention_f64(q, k8[:ctx], v8[:ctx], ks[:ctx], vs[:ctx], 1, nH, nKV, hd, ctx - 1, inv)
    out = torch.full((1, nH, hd), float("nan"), device="cuda")
    ws = ops.workspace(1, nH, hd, numChunks)
    for w in ws:
        w.fill_(float("nan"))  # poison: a slot that is read without being written shows up
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda") if dev_pos else None
    bound = ctx - 1 + (extra_rows if dev_pos else 0)  # with a device position the host value is an upper bound
    ops.decode_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ws, nH, nKV, hd, bound, numChunks,
                  invSqrt=inv, dev_pos=pos)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    assert_close(got, want, what=f"decode_i8 nH={nH} nKV={nKV} ctx={ctx} vs oracle")
    assert_close(got, exact, what=f"decode_i8 nH={nH} nKV={nKV} ctx={ctx} vs f64")
    return got


@pytest.mark.parametrize("ctx", [1, 2, 15, 16, 17, 31, 32, 33, 127, 128, 129, 1000, 8192])
def test_7b_shape_context_edges(ctx):
    _run_single(28, 4, 128, ctx, numChunks=256, seed=ctx)


@pytest.mark.parametrize("nH,nKV", [(40, 8), (14, 2), (12, 2), (8, 8), (8, 1), (5, 1), (21, 3), (16, 4), (6, 6),
                                    (32, 2), (24, 2), (9, 1), (40, 1)])
def test_head_layouts(nH, nKV):
    _run_single(nH, nKV, 128, 777, numChunks=64, seed=nH * 10 + nKV)


@pytest.mark.parametrize("nH,nKV,ctx", [(8, 2, 700), (16, 4, 1), (16, 4, 17), (24, 4, 4097), (32, 8, 2500),
                                         (6, 1, 333), (16, 2, 20000)])
def test_head_dim_256(nH, nKV, ctx):
    """The reference's own int8 shape (its int8 kernels are fixed at head_dim 256)."""
    _run_single(nH, nKV, 256, ctx, numChunks=64, seed=nH + ctx)


def test_head_dim_256_device_position_and_slack_rows():
    _run_single(16, 4, 256, 1500, numChunks=32, seed=77, extra_rows=64, dev_pos=True)


@pytest.mark.parametrize("numChunks", [1, 2, 3, 512])
def test_chunk_slot_capacity(numChunks):
    _run_single(28, 4, 128, 5000, numChunks=numChunks, seed=numChunks)


def test_rows_past_the_length_are_ignored():
    # garbage int8 rows and NaN scales sit right behind the live rows
    _run_single(28, 4, 128, 1000, numChunks=128, seed=3, extra_rows=200)


def test_device_position():
    _run_single(28, 4, 128, 1234, numChunks=128, seed=4, extra_rows=300, dev_pos=True)


def test_32b_shape_long_context():
    _run_single(40, 8, 128, 40000, numChunks=512, seed=5)


def test_large_magnitudes_and_zero_rows():
    nH, nKV, hd, ctx = 28, 4, 128, 600
    rng = np.random.default_rng(9)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32) * 40.0
    q[0, 3] = 0.0
    k = rng.standard_normal((ctx, nKV, hd), dtype=np.float32) * 0.05
    v = rng.standard_normal((ctx, nKV, hd), dtype=np.float32) * 500.0
    v[10] = 0.0
    k[11] = 0.0
    v[12:20] *= 1e-4
    k8, v8, ks, vs = make_i8_store(k, v, nKV, hd)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, inv)
    out = torch.empty((1, nH, hd), device="cuda")
    ops.decode_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ops.workspace(1, nH, hd, 64), nH, nKV, hd,
                  ctx - 1, 64, invSqrt=inv)
    # outputs are O(500): the absolute floor scales with the data
    assert_close(host(out), want, rtol=1e-3, atol=1e-4 * 500, what="scaled magnitudes")


def test_batch_of_ragged_sequences_in_one_pool():
    nH, nKV, hd = 28, 4, 128
    lens = np.array([1, 33, 512, 700, 2048, 95, 1500, 31], np.uint32)
    B, rows_per_seq = len(lens), 2048 + 16
    rng = np.random.default_rng(21)
    q = rng.standard_normal((B, nH, hd), dtype=np.float32)
    k8 = rng.integers(-128, 128, (B, rows_per_seq, nKV, hd), dtype=np.int8)
    v8 = rng.integers(-128, 128, (B, rows_per_seq, nKV, hd), dtype=np.int8)
    ks = np.full((B, rows_per_seq, nKV), np.nan, np.float32)
    vs = np.full((B, rows_per_seq, nKV), np.nan, np.float32)
    inv = 1.0 / math.sqrt(hd)
    want = np.zeros((B, nH, hd), np.float32)
    for b, n in enumerate(lens):
        k = rng.standard_normal((n, nKV, hd), dtype=np.float32)
        v = rng.standard_normal((n, nKV, hd), dtype=np.float32)
        a, c, d, e = oracle.quant_kv8(k, v, nKV, hd)
        k8[b, :n], v8[b, :n], ks[b, :n], vs[b, :n] = a, c, d, e
        want[b] = oracle.attention_i8(q[b:b + 1], a, c, d, e, 1, nH, nKV, hd, int(n) - 1, inv)[0]
    out = torch.full((B, nH, hd), float("nan"), device="cuda")
    numChunks = 64
    ws = ops.workspace(B, nH, hd, numChunks)
    for w in ws:
        w.fill_(float("nan"))
    used = ops.decode_i8_batch(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ws, dev(lens), B, nH, nKV, hd,
                               int(lens.max()), numChunks, rows_per_seq=rows_per_seq, invSqrt=inv)
    torch.cuda.synchronize()
    assert 1 <= used <= numChunks and ops.device_status() == 0
    assert_close(host(out), want, what="ragged batch")
    # explicit row bases (sequences placed out of order in the pool) give the same answer
    order = np.array([3, 0, 7, 1, 6, 2, 5, 4])
    base = (order.astype(np.uint64) * rows_per_seq)
    k8p, v8p, ksp, vsp = (np.empty_like(x) for x in (k8, v8, ks, vs))
    for b in range(B):
        k8p[order[b]], v8p[order[b]], ksp[order[b]], vsp[order[b]] = k8[b], v8[b], ks[b], vs[b]
    out2 = torch.empty_like(out)
    ops.decode_i8_batch(dev(q), dev(k8p), dev(v8p), dev(ksp), dev(vsp), out2, ws, dev(lens), B, nH, nKV, hd,
                        int(lens.max()), numChunks, row_base=dev(base), invSqrt=inv)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


def test_partials_contract_and_merge_entry_point():
    """partialsOnly leaves (m, l, acc) in the reference's layout; the separate
    merge entry point (and the oracle's merge) turn them into the same output."""
    nH, nKV, hd, ctx, numChunks = 28, 4, 128, 3000, 32
    rng = np.random.default_rng(8)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
    ws = ops.workspace(1, nH, hd, numChunks)
    for w in ws:
        w.zero_()
    out = torch.zeros((1, nH, hd), device="cuda")
    lens = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    used = ops.decode_i8_batch(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ws, lens, 1, nH, nKV, hd, ctx,
                               numChunks, partials_only=True)
    assert used > 1
    acc, m, l = (host(w) for w in ws)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, 1.0 / math.sqrt(hd))
    merged = oracle.combine_partials(acc, m, l, 1, nH, numChunks, hd)   # unused slots hold l == 0
    assert_close(merged, want, what="oracle merge of GPU partials")
    out2 = torch.empty_like(out)
    ops.merge_partials(ws[0], ws[1], ws[2], out2, 1, nH, numChunks, hd)
    assert_close(host(out2), want, what="GPU merge of GPU partials")
    # determinism: the same call twice gives the same bits
    ws2 = ops.workspace(1, nH, hd, numChunks)
    for w in ws2:
        w.zero_()
    ops.decode_i8_batch(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ws2, lens, 1, nH, nKV, hd, ctx,
                        numChunks, partials_only=True)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(ws, ws2))


@pytest.mark.parametrize("hd,pdl,dev_lens", [(128, False, True), (128, True, False), (128, False, False), (256, False, True)])
def test_new_rows_quantised_by_the_decode_launch(hd, pdl, dev_lens):
    """appendK / appendV: the launch writes row len - 1 of every sequence itself -- the bytes and scales
    of tc_kv_quantize_i8_batch -- and attends over it; output and pool equal quantise-then-decode."""
    nH, nKV, B, numChunks = 16, 4, 3, 64
    lens = np.array([700, 129, 1], np.uint32) if dev_lens else np.array([513, 513, 513], np.uint32)
    rows_per_seq = 720 + 16
    rng = np.random.default_rng(hd + int(pdl))
    inv = 1.0 / math.sqrt(hd)
    q = rng.standard_normal((B, nH, hd), dtype=np.float32)
    newk = rng.standard_normal((B, nKV, hd), dtype=np.float32)
    newv = rng.standard_normal((B, nKV, hd), dtype=np.float32)
    newk[1, 2] = 0.0                                       # an all-zero row: scale 1
    k8 = np.zeros((B, rows_per_seq, nKV, hd), np.int8)
    v8 = np.zeros_like(k8)
    ks = np.full((B, rows_per_seq, nKV), np.nan, np.float32)
    vs = np.full_like(ks, np.nan)
    want = np.zeros((B, nH, hd), np.float32)
    for b, n in enumerate(lens):
        k = np.concatenate([rng.standard_normal((n - 1, nKV, hd), dtype=np.float32), newk[b:b + 1]])
        v = np.concatenate([rng.standard_normal((n - 1, nKV, hd), dtype=np.float32), newv[b:b + 1]])
        a, c, d, e = oracle.quant_kv8(k, v, nKV, hd)
        k8[b, :n - 1], v8[b, :n - 1], ks[b, :n - 1], vs[b, :n - 1] = a[:-1], c[:-1], d[:-1], e[:-1]   # the last row is missing
        want[b] = oracle.attention_i8(q[b:b + 1], a, c, d, e, 1, nH, nKV, hd, int(n) - 1, inv)[0]
    ws = ops.workspace(B, nH, hd, numChunks)
    dl = dev(lens) if dev_lens else None
    # reference arm: quantise launch, then decode
    p1 = [dev(x) for x in (k8, v8, ks, vs)]
    out1 = torch.full((B, nH, hd), float("nan"), device="cuda")
    ops.kv_quantize_i8_batch(dev(newk), dev(newv), *p1, B, nKV, hd, rows_per_seq=rows_per_seq,
                             **({"lens": dl, "len_add": -1} if dev_lens else {"pos": int(lens[0]) - 1}))
    ops.decode_i8_batch(dev(q), *p1, out1, ws, dl, B, nH, nKV, hd, int(lens.max()), numChunks,
                        rows_per_seq=rows_per_seq, invSqrt=inv)
    # fused arm
    p2 = [dev(x) for x in (k8, v8, ks, vs)]
    out2 = torch.full((B, nH, hd), float("nan"), device="cuda")
    ops.decode_i8_batch(dev(q), *p2, out2, ws, dl, B, nH, nKV, hd, int(lens.max()), numChunks,
                        rows_per_seq=rows_per_seq, invSqrt=inv, append=(dev(newk), dev(newv)), pdl=pdl,
                        prefetch_rows=int(lens.max()) - 1 if pdl else 0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out2), want, what="decode with the new rows appended by the launch")
    # (the dependent-launch form merges with another kernel: same rule, another summation order)
    assert torch.equal(out1, out2) if not pdl else torch.allclose(out1, out2, rtol=1e-5, atol=1e-6)
    for a, b_, name in zip(p1, p2, ("k8", "v8", "ks", "vs")):
        for s_ in range(B):
            n = int(lens[s_])
            assert torch.equal(a[s_, :n], b_[s_, :n]), f"{name}: pool rows of sequence {s_}"


def test_new_row_past_the_pool_is_skipped_and_flagged():
    """A device length that puts the appended row outside the pool: nothing is written there, the
    error word carries the row-bound bit, nothing faults (the canary rows behind the pool stay)."""
    nH, nKV, hd, rows = 8, 2, 128, 256
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    k8 = torch.randint(-128, 128, (rows + 8, nKV, hd), dtype=torch.int8, device="cuda", generator=g)
    v8 = torch.randint(-128, 128, (rows + 8, nKV, hd), dtype=torch.int8, device="cuda", generator=g)
    ks = torch.rand((rows + 8, nKV), device="cuda", generator=g)
    vs = torch.rand((rows + 8, nKV), device="cuda", generator=g)
    before = [x.clone() for x in (k8, v8, ks, vs)]
    q = torch.randn((1, nH, hd), device="cuda", generator=g)
    newk = torch.randn((1, nKV, hd), device="cuda", generator=g)
    out = torch.empty((1, nH, hd), device="cuda")
    ws = ops.workspace(1, nH, hd, 16)
    lens = torch.tensor([rows + 1], dtype=torch.int32, device="cuda")     # row `rows` is one past the pool
    # (the host bound covers the bad length, so the block of the last chunk gets to the append)
    ops.decode_i8_batch(q, k8[:rows], v8[:rows], ks[:rows], vs[:rows], out, ws, lens, 1, nH, nKV, hd, rows + 8, 16,
                        rows_per_seq=rows, append=(newk, newk))
    torch.cuda.synchronize()
    assert ops.device_status(raise_on_flags=False) == 32
    for a, b_ in zip(before, (k8, v8, ks, vs)):
        assert torch.equal(a, b_)


def test_seeded_random_batches():
    """Thirty seeded batches: 1 to 5 sequences of 1 to 6000 rows, 1 to 8 kv heads with 1 to 12 q heads
    each (more than 8 take a second launch), head_dim 128 and 256, device or host lengths, chunk
    slot counts from 1 up, the new rows appended by the launch or not -- each against the oracle."""
    rng = np.random.default_rng(77)
    for case in range(30):
        hd = int(rng.choice([128, 128, 128, 256]))
        nKV = int(rng.choice([1, 2, 4, 8]))
        group = int(rng.choice([1, 2, 4, 5, 7, 8, 12]))
        nH = nKV * group
        B = int(rng.integers(1, 6))
        dev_lens = bool(rng.integers(0, 2))
        top = int(rng.choice([40, 300, 1500, 6000]))
        lens = rng.integers(1, top + 1, B).astype(np.uint32) if dev_lens else np.full(B, int(rng.integers(1, top + 1)), np.uint32)
        append = bool(rng.integers(0, 2))
        numChunks = int(rng.choice([1, 3, 16, 64]))
        rows_per_seq = int(lens.max()) + 16
        inv = 1.0 / math.sqrt(hd)
        q = rng.standard_normal((B, nH, hd), dtype=np.float32)
        k8 = np.zeros((B, rows_per_seq, nKV, hd), np.int8)
        v8 = np.zeros_like(k8)
        ks = np.full((B, rows_per_seq, nKV), np.nan, np.float32)
        vs = np.full_like(ks, np.nan)
        newk = np.zeros((B, nKV, hd), np.float32)
        newv = np.zeros_like(newk)
        want = np.zeros((B, nH, hd), np.float32)
        for b, n in enumerate(lens):
            n = int(n)
            k = rng.standard_normal((n, nKV, hd), dtype=np.float32)
            v = rng.standard_normal((n, nKV, hd), dtype=np.float32)
            a, c, d, e = oracle.quant_kv8(k, v, nKV, hd)
            m = n - 1 if append else n                      # with append the last row is handed in as f32
            k8[b, :m], v8[b, :m], ks[b, :m], vs[b, :m] = a[:m], c[:m], d[:m], e[:m]
            newk[b], newv[b] = k[n - 1], v[n - 1]
            want[b] = oracle.attention_i8(q[b:b + 1], a, c, d, e, 1, nH, nKV, hd, n - 1, inv)[0]
        out = torch.full((B, nH, hd), float("nan"), device="cuda")
        ws = ops.workspace(B, nH, hd, numChunks)
        for w in ws:
            w.fill_(float("nan"))
        ops.decode_i8_batch(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ws, dev(lens) if dev_lens else None, B, nH,
                            nKV, hd, int(lens.max()), numChunks, rows_per_seq=rows_per_seq, invSqrt=inv,
                            append=(dev(newk), dev(newv)) if append else None)
        torch.cuda.synchronize()
        what = f"case {case}: lens={lens.tolist()} nH={nH} nKV={nKV} hd={hd} chunks={numChunks} append={append} dev_lens={dev_lens}"
        assert ops.device_status(raise_on_flags=False) == 0, what
        assert_close(host(out), want, what=what)


def test_dependent_launch_chain_and_host_lengths():
    """Three 'layers' back to back with programmatic dependent launch (KV rows of a
    layer stream in while the previous layer's kernels drain) give the same
    bits as plain stream order; lens=None means every sequence is maxLen long."""
    nH, nKV, hd, ctx, B, layers, numChunks = 28, 4, 128, 3000, 2, 3, 64
    rows = ctx + 16
    rng = np.random.default_rng(17)
    inv = 1.0 / math.sqrt(hd)
    q = rng.standard_normal((layers, B, nH, hd), dtype=np.float32)
    pools, want = [], np.zeros((layers, B, nH, hd), np.float32)
    for l in range(layers):
        k8 = np.zeros((B, rows, nKV, hd), np.int8)
        v8 = np.zeros_like(k8)
        ks = np.full((B, rows, nKV), np.nan, np.float32)
        vs = np.full_like(ks, np.nan)
        for b in range(B):
            a, c, d, e = oracle.quant_kv8(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                          rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
            k8[b, :ctx], v8[b, :ctx], ks[b, :ctx], vs[b, :ctx] = a, c, d, e
            want[l, b] = oracle.attention_i8(q[l, b:b + 1], a, c, d, e, 1, nH, nKV, hd, ctx - 1, inv)[0]
        pools.append(tuple(dev(x) for x in (k8, v8, ks, vs)))
    qd = dev(q)
    ws = ops.workspace(B, nH, hd, numChunks)
    outs = {}
    for pdl in (False, True):
        out = torch.full((layers, B, nH, hd), float("nan"), device="cuda")
        for rep in range(2):
            for l in range(layers):
                k8, v8, ks, vs = pools[l]
                ops.decode_i8_batch(qd[l], k8, v8, ks, vs, out[l], ws, None, B, nH, nKV, hd, ctx, numChunks,
                                    rows_per_seq=rows, invSqrt=inv, pdl=pdl, prefetch_rows=ctx - 1)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert_close(host(out), want, what=f"pdl={pdl}")
        outs[pdl] = out
    # the two launch forms use different merge kernels (block per head / 32-dim slices): same rule,
    # different summation order
    assert torch.allclose(outs[False], outs[True], rtol=1e-5, atol=1e-6)


def test_next_pool_hint_changes_nothing_but_timing():
    """nextK8 / nextV8 only ask for an L2 prefetch of another pool: same bits out."""
    nH, nKV, hd, ctx, C = 28, 4, 128, 9000, 160
    rng = np.random.default_rng(41)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
    other_k = torch.randint(-128, 127, (ctx, nKV, hd), dtype=torch.int8, device="cuda")
    other_v = torch.randint(-128, 127, (ctx, nKV, hd), dtype=torch.int8, device="cuda")
    dq, dk8, dv8, dks, dvs = dev(q), dev(k8), dev(v8), dev(ks), dev(vs)
    ws = ops.workspace(1, nH, hd, C)
    a = torch.empty((1, nH, hd), device="cuda")
    b = torch.empty_like(a)
    ops.decode_i8_batch(dq, dk8, dv8, dks, dvs, a, ws, None, 1, nH, nKV, hd, ctx, C)
    ops.decode_i8_batch(dq, dk8, dv8, dks, dvs, b, ws, None, 1, nH, nKV, hd, ctx, C, next_kv=(other_k, other_v))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(a, b)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, 1.0 / math.sqrt(hd))
    assert_close(host(b), want, what="decode with a next-pool hint")


def test_context_split_partials_merge_on_one_gpu():
    """The context-axis split as two 'ranks' on one device: each half of the rows yields
    partials-only output, the partials are concatenated as the all-gather would and merged."""
    nH, nKV, hd, ctx, C = 28, 4, 128, 5000, 16
    rng = np.random.default_rng(31)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, inv)
    from tinycoder_inference_b200 import sharding
    parts = []
    for lo, hi in sharding.plan_context_ranges(ctx, 2):
        acc, m, l = ops.workspace(1, nH, hd, C)
        acc.zero_()
        m.fill_(-1e30)
        l.zero_()
        out = torch.empty((1, nH, hd), device="cuda")
        ops.decode_i8_batch(dev(q), dev(k8[lo:hi]), dev(v8[lo:hi]), dev(ks[lo:hi]), dev(vs[lo:hi]), out, (acc, m, l),
                            None, 1, nH, nKV, hd, hi - lo, C, invSqrt=inv, partials_only=True)
        parts.append((acc.view(nH, C, hd), m.view(nH, C), l.view(nH, C)))
    gacc = torch.cat([p[0] for p in parts], dim=1).contiguous()
    gm = torch.cat([p[1] for p in parts], dim=1).contiguous()
    gl = torch.cat([p[2] for p in parts], dim=1).contiguous()
    out = torch.empty((1, nH, hd), device="cuda")
    ops.merge_partials(gacc, gm, gl, out, 1, nH, 2 * C, hd)
    assert_close(host(out), want, what="context split, two ranges")
    # the same partials as ONE all-gathered buffer of per-rank [acc | m | l] blocks
    gathered = torch.cat([torch.cat([a.reshape(-1), m.reshape(-1), l.reshape(-1)]) for a, m, l in parts]).contiguous()
    out2 = torch.full((1, nH, hd), float("nan"), device="cuda")
    ops.merge_gathered(gathered, out2, nH, 2, C, hd)
    assert np.array_equal(host(out2), host(out)), "rank-strided merge differs from the concatenated one"


@pytest.mark.gpu
def test_context_split_decoder_single_rank_matches_oracle():
    nH, nKV, hd, ctx = 16, 2, 128, 3000
    rng = np.random.default_rng(32)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, inv)
    from tinycoder_inference_b200 import sharding
    dec = sharding.ContextSplitDecoder(nH, nKV, hd, ctx, chunk_slots=32)
    out = torch.empty((1, nH, hd), device="cuda")
    for _ in range(2):     # second call reuses the buffers
        dec(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ctx, invSqrt=inv)
    assert_close(host(out), want, what="ContextSplitDecoder, world 1")


@pytest.mark.parametrize("pdl", [False, True])
def test_merge_inside_the_kernel_by_the_last_arriving_block(pdl):
    """With arrival counters the split-KV kernel merges its own partials: ragged batch (device
    lengths, some chunks inactive), several layers back to back on the same partial buffers and
    the same counters, NaN-poisoned partial slots.  The counters are zero again afterwards."""
    nH, nKV, hd, B, layers, numChunks = 28, 4, 128, 5, 3, 64
    lens = np.array([4000, 1, 129, 2600, 777], np.int64)
    base = np.zeros(B, np.int64)
    base[1:] = np.cumsum(lens[:-1] + 16)
    rows = int((lens + 16).sum())
    rng = np.random.default_rng(23)
    inv = 1.0 / math.sqrt(hd)
    q = rng.standard_normal((layers, B, nH, hd), dtype=np.float32)
    pools, want = [], np.zeros((layers, B, nH, hd), np.float32)
    for l in range(layers):
        k8 = rng.integers(-128, 128, (rows, nKV, hd), dtype=np.int8)      # stale bytes between the sequences
        v8 = rng.integers(-128, 128, (rows, nKV, hd), dtype=np.int8)
        ks = np.full((rows, nKV), np.nan, np.float32)
        vs = np.full_like(ks, np.nan)
        for b in range(B):
            n, r0 = int(lens[b]), int(base[b])
            a, c, d, e = oracle.quant_kv8(rng.standard_normal((n, nKV, hd), dtype=np.float32),
                                          rng.standard_normal((n, nKV, hd), dtype=np.float32), nKV, hd)
            k8[r0:r0 + n], v8[r0:r0 + n], ks[r0:r0 + n], vs[r0:r0 + n] = a, c, d, e
            want[l, b] = oracle.attention_i8(q[l, b:b + 1], a, c, d, e, 1, nH, nKV, hd, n - 1, inv)[0]
        pools.append(tuple(dev(x) for x in (k8, v8, ks, vs)))
    qd = dev(q)
    ws = ops.workspace(B, nH, hd, numChunks)
    for w in ws:
        w.fill_(float("nan"))
    tickets = torch.zeros(B * nKV, dtype=torch.int32, device="cuda")
    dlens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    dbase = torch.tensor(base, dtype=torch.int64, device="cuda")
    out = torch.full((layers, B, nH, hd), float("nan"), device="cuda")
    for rep in range(3):
        for l in range(layers):
            k8, v8, ks, vs = pools[l]
            ops.decode_i8_batch(qd[l], k8, v8, ks, vs, out[l], ws, dlens, B, nH, nKV, hd, int(lens.max()), numChunks,
                                row_base=dbase, invSqrt=inv, pdl=pdl, tickets=tickets)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert int(tickets.abs().sum().item()) == 0, "every counter is back at zero"
    assert_close(host(out), want, what=f"in-kernel merge, pdl={pdl}")


def test_merge_inside_the_kernel_equals_the_merge_launch():
    """Same partials, same rule: the fused form against the two-launch form at the 7B shape, 8192 rows
    (host length, one sequence), and a single-chunk call where nothing has to be merged."""
    nH, nKV, hd = 28, 4, 128
    rng = np.random.default_rng(29)
    for ctx in (8192, 100):
        k8, v8, ks, vs = oracle.quant_kv8(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                          rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
        q = rng.standard_normal((1, nH, hd), dtype=np.float32)
        d = [dev(x) for x in (q, k8, v8, ks, vs)]
        _, chunks = ops.split_geometry(ctx, nH, hd)
        ws = ops.workspace(1, nH, hd, chunks)
        tickets = torch.zeros(nKV, dtype=torch.int32, device="cuda")
        a = torch.full((1, nH, hd), float("nan"), device="cuda")
        b = torch.full_like(a, float("nan"))
        ops.decode_i8_batch(*d, a, ws, None, 1, nH, nKV, hd, ctx, chunks, tickets=tickets)
        ops.decode_i8_batch(*d, b, ws, None, 1, nH, nKV, hd, ctx, chunks)
        torch.cuda.synchronize()
        want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, 1.0 / math.sqrt(hd))
        assert_close(host(a), want, what=f"fused, ctx {ctx}")
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
        assert int(tickets.abs().sum().item()) == 0
    assert ops.device_status() == 0
