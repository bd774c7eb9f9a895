"""KV writers on the GPU against the oracle: int8 quantise+append (bit-exact),
f32/fp16 append with and without the fused rotation (bit-exact)."""
import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tinycoder_inference_b200 import synth
from tests.util import dev, host

pytestmark = pytest.mark.gpu


def _quant_case(tokens, nKV, hd, dst_base, src_base, seed, special=False):
    rng = np.random.default_rng(seed)
    rows = src_base + tokens
    k = rng.standard_normal((rows, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((rows, nKV, hd), dtype=np.float32) * 3.0
    if special and tokens >= 4:
        k[src_base + 0] = 0.0                      # amax == 0 -> scale 1
        v[src_base + 1] = 0.0
        k[src_base + 2, :, 0] = 1e-30               # tiny amax
        v[src_base + 3, 0, :] = np.float32(127.5)   # ties at the clamp edge
        k[src_base + 3, 0, ::2] = 0.5
        k[src_base + 3, 0, 1::2] = np.float32(63.5)  # x/s lands on .5 -> round half even
    want = oracle.quant_kv8(k, v, nKV, hd, dst_base=dst_base, src_base=src_base, tokens=tokens)
    total = dst_base + tokens + 3
    k8 = torch.full((total, nKV, hd), 77, dtype=torch.int8, device="cuda")
    v8 = torch.full((total, nKV, hd), 77, dtype=torch.int8, device="cuda")
    ks = torch.full((total, nKV), -5.0, device="cuda")
    vs = torch.full((total, nKV), -5.0, device="cuda")
    ops.kv_quantize_i8(dev(k), dev(v), k8, v8, ks, vs, tokens, nKV, hd, dst_base, src_base)
    torch.cuda.synchronize()
    sl = slice(dst_base, dst_base + tokens)
    for got, ref in zip((k8, v8, ks, vs), want):
        assert np.array_equal(host(got)[sl], ref[sl])
    # rows outside [dst_base, dst_base + tokens) are untouched
    assert (host(k8)[dst_base + tokens:] == 77).all() and (host(ks)[:dst_base] == -5.0).all()


@pytest.mark.parametrize("tokens,nKV,hd,dst,src", [
    (8192, 4, 128, 0, 0),      # the 7B-shaped store of the decode configs
    (4096, 4, 128, 0, 0),      # the prefill mirror
    (1, 4, 128, 777, 0),       # one decode token appended at pos
    (37, 8, 128, 100, 5),      # mirror rebuild from row 5 of the f32 cache into row 100
    (129, 2, 64, 3, 0),
    (65, 4, 256, 0, 2),        # the reference's own head_dim
    (5, 1, 32, 0, 0),
    (3, 3, 96, 1, 1),
])
def test_quantize_bit_exact(tokens, nKV, hd, dst, src):
    _quant_case(tokens, nKV, hd, dst, src, seed=tokens + hd, special=True)


def test_quantize_zero_tokens_and_device_base():
    nKV, hd = 4, 128
    k = torch.randn(4, nKV, hd, device="cuda")
    k8 = torch.zeros(16, nKV, hd, dtype=torch.int8, device="cuda")
    s = torch.zeros(16, nKV, device="cuda")
    ops.kv_quantize_i8(k, k, k8, k8.clone(), s, s.clone(), 0, nKV, hd)
    base = torch.tensor([9], dtype=torch.int32, device="cuda")
    v8 = torch.zeros_like(k8)
    vs = torch.zeros_like(s)
    ops.kv_quantize_i8(k, k, k8, v8, s, vs, 4, nKV, hd, dst_base=0, dev_dst_base=base)
    torch.cuda.synchronize()
    want = oracle.quant_kv8(host(k), host(k), nKV, hd, dst_base=9)
    assert np.array_equal(host(k8)[9:13], want[0][9:13]) and (host(k8)[:9] == 0).all()
    assert np.array_equal(host(vs)[9:13], want[3][9:13])


def test_quantize_past_the_pool_is_refused():
    nKV, hd = 4, 128
    k = torch.randn(4, nKV, hd, device="cuda")
    k8 = torch.zeros(8, nKV, hd, dtype=torch.int8, device="cuda")
    s = torch.zeros(8, nKV, device="cuda")
    with pytest.raises(capi.ContextFull):
        ops.kv_quantize_i8(k, k, k8, k8, s, s, 4, nKV, hd, dst_base=6)


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("rope", [False, True])
@pytest.mark.parametrize("seqLen,nH,nKV,hd,cachePos", [(1, 14, 2, 64, 2047), (512, 28, 4, 128, 0), (7, 40, 8, 128, 33),
                                                      (3, 4, 4, 256, 5)])
def test_append_bit_exact(half, rope, seqLen, nH, nKV, hd, cachePos):
    rng = np.random.default_rng(seqLen * 31 + hd)
    rows = cachePos + seqLen + 2
    kSrc = rng.standard_normal((seqLen, nKV, hd), dtype=np.float32)
    vSrc = rng.standard_normal((seqLen, nKV, hd), dtype=np.float32)
    q = rng.standard_normal((seqLen, nH, hd), dtype=np.float32)
    dt = np.float16 if half else np.float32
    kRef = np.full((rows, nKV, hd), 9, dt)
    vRef = np.full((rows, nKV, hd), 9, dt)
    kDst, vDst = dev(kRef), dev(vRef)
    if rope:
        cosT, sinT = oracle.rope_tables(rows, hd, 1e6)
        oracle.kv_append(kSrc, vSrc, kRef, vRef, seqLen, nKV, hd, cachePos, cachePos, cosT, sinT)
        qRef = oracle.rope_q(q, cosT, sinT, seqLen, nH, hd, cachePos)
        qd = dev(q)
        ops.kv_append_rope(qd, dev(kSrc), dev(vSrc), kDst, vDst, seqLen, nH, nKV, hd, cachePos, cachePos,
                           dev(cosT), dev(sinT))
        assert np.array_equal(host(qd), qRef)
        q2 = dev(q)
        ops.rope_q(q2, dev(cosT), dev(sinT), seqLen, nH, hd, cachePos)
        assert np.array_equal(host(q2), qRef)
    else:
        oracle.kv_append(kSrc, vSrc, kRef, vRef, seqLen, nKV, hd, cachePos)
        ops.kv_append(dev(kSrc), dev(vSrc), kDst, vDst, seqLen, nKV, hd, cachePos)
    torch.cuda.synchronize()
    assert np.array_equal(host(kDst).view(np.uint8), kRef.view(np.uint8))
    assert np.array_equal(host(vDst).view(np.uint8), vRef.view(np.uint8))


def test_append_device_position_and_window_guard():
    nKV, hd = 4, 128
    kSrc = torch.randn(1, nKV, hd, device="cuda")
    kDst = torch.zeros(16, nKV, hd, device="cuda")
    vDst = torch.zeros(16, nKV, hd, device="cuda")
    pos = torch.tensor([11], dtype=torch.int32, device="cuda")
    ops.kv_append(kSrc, kSrc, kDst, vDst, 1, nKV, hd, 0, dev_pos=pos)
    torch.cuda.synchronize()
    assert torch.equal(kDst[11], kSrc[0]) and float(kDst[:11].abs().sum()) == 0.0
    with pytest.raises(capi.ContextFull):
        ops.kv_append(kSrc, kSrc, kDst, vDst, 1, nKV, hd, 16)


def test_cpu_engine_append_is_within_tolerance_of_gpu_form():
    # Model::storeKVWithRoPE rounds the two products separately; the GPU form fuses one.
    seqLen, nKV, hd = 5, 4, 128
    rng = np.random.default_rng(3)
    kSrc = rng.standard_normal((seqLen, nKV, hd), dtype=np.float32)
    cosT, sinT = oracle.rope_tables(16, hd, 1e6)
    a = np.zeros((16, nKV, hd), np.float32)
    b = np.zeros_like(a)
    oracle.kv_append(kSrc, kSrc, a, np.zeros_like(a), seqLen, nKV, hd, 3, 3, cosT, sinT)
    oracle.kv_append_cpu(kSrc, kSrc, b, np.zeros_like(b), seqLen, 3, nKV, hd, cosT, sinT)
    assert np.allclose(a, b, rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
def test_batched_quantise_appends_one_row_per_sequence():
    """tc_kv_quantize_i8_batch: the new token of every sequence lands behind that sequence's rows,
    with host position, device lengths and explicit row bases; bytes equal the oracle's."""
    import oracle
    B, nKV, hd, rps = 5, 4, 128, 40
    rng = np.random.default_rng(77)
    k = rng.standard_normal((B, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((B, nKV, hd), dtype=np.float32) * 2
    want = oracle.quant_kv8(k, v, nKV, hd)

    def fresh():
        return (torch.zeros((B * rps, nKV, hd), dtype=torch.int8, device="cuda"),
                torch.zeros((B * rps, nKV, hd), dtype=torch.int8, device="cuda"),
                torch.zeros((B * rps, nKV), device="cuda"), torch.zeros((B * rps, nKV), device="cuda"))

    def check_rows(pool, rows):
        k8, v8, ks, vs = (host(t) for t in pool)
        for b, r in enumerate(rows):
            assert np.array_equal(k8[r], want[0][b]) and np.array_equal(v8[r], want[1][b])
            assert np.array_equal(ks[r], want[2][b]) and np.array_equal(vs[r], want[3][b])
        mask = np.ones(B * rps, bool)
        mask[list(rows)] = False
        assert not k8[mask].any() and not vs[mask].any(), "only the new rows are written"

    pool = fresh()
    ops.kv_quantize_i8_batch(dev(k), dev(v), *pool, B, nKV, hd, rows_per_seq=rps, pos=7)
    check_rows(pool, [b * rps + 7 for b in range(B)])
    lens = np.array([1, 40, 13, 2, 30], np.uint32)          # lengths that already count the new token
    pool = fresh()
    ops.kv_quantize_i8_batch(dev(k), dev(v), *pool, B, nKV, hd, rows_per_seq=rps, lens=dev(lens), len_add=-1)
    check_rows(pool, [b * rps + int(lens[b]) - 1 for b in range(B)])
    base = np.array([120, 0, 41, 81, 160], np.uint64)
    pool = fresh()
    ops.kv_quantize_i8_batch(dev(k), dev(v), *pool, B, nKV, hd, row_base=dev(base), lens=dev(lens), len_add=-1)
    check_rows(pool, [int(base[b]) + int(lens[b]) - 1 for b in range(B)])
    from tinycoder_inference_b200 import capi
    with pytest.raises(capi.ContextFull):
        ops.kv_quantize_i8_batch(dev(k), dev(v), *pool, B, nKV, hd, rows_per_seq=rps, pos=rps * 2)


def test_device_position_outside_the_pool_is_skipped_and_reported():
    """A position read from device memory cannot be checked on the host.  The writers check it
    where it is known: a row that would land outside the pool is not stored (rows behind the
    pool keep their canary bytes) and bit 32 of the device error word says so.  Nothing faults."""
    nKV, hd, rows, canary = 2, 128, 8, 4
    r = np.random.default_rng(3)
    k = dev(r.standard_normal((1, nKV, hd), dtype=np.float32))
    v = dev(r.standard_normal((1, nKV, hd), dtype=np.float32))
    # int8 quantiser, single-sequence form with the destination row on the device
    k8 = torch.full((rows + canary, nKV, hd), 91, dtype=torch.int8, device="cuda")
    v8 = torch.full_like(k8, -37)
    ks = torch.full((rows + canary, nKV), 7.0, device="cuda")
    vs = torch.full_like(ks, 9.0)
    assert ops.device_status() == 0
    for bad in (rows, rows + 2):
        ops.kv_quantize_i8(k, v, k8, v8, ks, vs, 1, nKV, hd, dev_dst_base=torch.tensor([bad], dtype=torch.int32, device="cuda"),
                           max_rows=rows)
        torch.cuda.synchronize()
        assert ops.device_status(raise_on_flags=False) == 32
        assert (k8 == 91).all() and (v8 == -37).all() and (ks == 7.0).all() and (vs == 9.0).all()
    ops.kv_quantize_i8(k, v, k8, v8, ks, vs, 1, nKV, hd, dev_dst_base=torch.tensor([rows - 1], dtype=torch.int32, device="cuda"),
                       max_rows=rows)      # the last row of the pool is fine
    assert ops.device_status() == 0 and not (k8[rows - 1] == 91).all() and (k8[rows:] == 91).all()
    # batched form: one sequence's length points past the pool
    k8.fill_(91)
    kb = dev(r.standard_normal((2, nKV, hd), dtype=np.float32))
    lens = torch.tensor([3, rows + 1], dtype=torch.int32, device="cuda")     # rows per sequence: 4
    ops.kv_quantize_i8_batch(kb, kb, k8, v8, ks, vs, 2, nKV, hd, rows_per_seq=4, lens=lens, len_add=0, total_rows=rows)
    assert ops.device_status(raise_on_flags=False) == 32
    assert not (k8[3] == 91).all() and (k8[rows:] == 91).all(), "the good sequence is stored, the bad one is not"
    # f32 append with a device position
    kd = torch.full((rows + canary, nKV, hd), 5.0, device="cuda")
    vd = torch.full_like(kd, 6.0)
    two = dev(r.standard_normal((2, nKV, hd), dtype=np.float32))
    ops.kv_append(two, two, kd, vd, 2, nKV, hd, 0, dev_pos=torch.tensor([rows - 1], dtype=torch.int32, device="cuda"),
                  max_rows=rows)           # first row fits, second does not
    assert ops.device_status(raise_on_flags=False) == 32
    assert torch.equal(kd[rows - 1], two[0]) and (kd[rows:] == 5.0).all() and (vd[rows:] == 6.0).all()
    assert ops.device_status() == 0
