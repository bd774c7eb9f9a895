"""Parity at the benchmark configurations' OWN sizes (the small cases elsewhere pick other
tilings: 16-token warp tiles, several waves, fewer kv heads per block):

  C2  7B shape (28 q / 4 kv heads, head_dim 128), int8 KV, context 8192, batch 8
  C3  7B-shaped causal fp16 prefill, 4096 rows, plus the int8 mirror of all 4096 rows
  C4  32B shape (40 q / 8 kv heads), int8 KV, context 131072, one layer
  C5  64 ragged sequences in [512, 32768] (the bench's own seeded lengths), 7B shape, int8 KV

Inputs are drawn on the device (seeded), the int8 stores are built by the library's quantiser
(bit-exact with the oracle's, checked on a sample here and everywhere in test_kv_write_gpu.py)
and every output is compared with the CPU restatement of the reference kernels."""
import math
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import ops
from tests.util import assert_close, host

pytestmark = pytest.mark.gpu


def _randn(shape, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device="cuda")


def _build_store(rows, nKV, hd, seed, pad=16):
    """f32 rows drawn on the device in blocks, quantised by the library into one pool."""
    k8 = torch.empty((rows + pad, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.empty_like(k8)
    ks = torch.full((rows + pad, nKV), float("nan"), device="cuda")
    vs = torch.full_like(ks, float("nan"))
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    blk = 32768
    first = None
    for r0 in range(0, rows, blk):
        n = min(blk, rows - r0)
        kf = torch.randn((n, nKV, hd), generator=g, device="cuda")
        vf = torch.randn((n, nKV, hd), generator=g, device="cuda")
        ops.kv_quantize_i8(kf, vf, k8, v8, ks, vs, n, nKV, hd, dst_base=r0)
        if first is None:
            first = (host(kf[:64]), host(vf[:64]))
    # the library's bytes are the oracle's bytes (sample: the first 64 rows)
    want = oracle.quant_kv8(first[0], first[1], nKV, hd)
    assert np.array_equal(host(k8[:64]), want[0]) and np.array_equal(host(v8[:64]), want[1])
    assert np.array_equal(host(ks[:64]), want[2]) and np.array_equal(host(vs[:64]), want[3])
    return k8, v8, ks, vs


@pytest.mark.parametrize("device_lengths", [False, True])
def test_c2_batch8_context_8192(device_lengths):
    nH, nKV, hd, ctx, B = 28, 4, 128, 8192, 8
    inv = 1.0 / math.sqrt(hd)
    rows_per_seq = ctx + 16
    k8, v8, ks, vs = _build_store(B * rows_per_seq - 16, nKV, hd, seed=0xC2)
    q = _randn((B, nH, hd), 0xC2 + 1)
    out = torch.full((B, nH, hd), float("nan"), device="cuda")
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(B, nH, hd, chunks)
    lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda") if device_lengths else None
    ops.decode_i8_batch(q, k8, v8, ks, vs, out, ws, lens, B, nH, nKV, hd, ctx, chunks, rows_per_seq=rows_per_seq,
                        invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    hk8, hv8, hks, hvs, hq, got = host(k8), host(v8), host(ks), host(vs), host(q), host(out)
    for b in range(B):
        r0 = b * rows_per_seq
        want = oracle.attention_i8(hq[b:b + 1], hk8[r0:r0 + ctx], hv8[r0:r0 + ctx], hks[r0:r0 + ctx], hvs[r0:r0 + ctx],
                                   1, nH, nKV, hd, ctx - 1, inv)
        assert_close(got[b:b + 1], want, what=f"C2 batch 8, sequence {b}")


def test_c4_32b_shape_context_131072():
    nH, nKV, hd, ctx = 40, 8, 128, 131072
    inv = 1.0 / math.sqrt(hd)
    k8, v8, ks, vs = _build_store(ctx, nKV, hd, seed=0xC4)
    q = _randn((1, nH, hd), 0xC4 + 1)
    out = torch.full((1, nH, hd), float("nan"), device="cuda")
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(1, nH, hd, chunks)
    ops.decode_i8(q, k8, v8, ks, vs, out, ws, nH, nKV, hd, ctx - 1, chunks, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    hk8, hv8, hks, hvs = host(k8[:ctx]), host(v8[:ctx]), host(ks[:ctx]), host(vs[:ctx])
    want = oracle.attention_i8(host(q), hk8, hv8, hks, hvs, 1, nH, nKV, hd, ctx - 1, inv)
    assert_close(host(out), want, what="C4 40/8/128 at 131072 rows")
    exact = oracle.attention_f64(host(q), hk8, hv8, hks, hvs, 1, nH, nKV, hd, ctx - 1, inv)
    assert_close(host(out), exact, what="C4 against double precision")


def test_c5_64_ragged_sequences():
    nH, nKV, hd, nseq = 28, 4, 128, 64
    inv = 1.0 / math.sqrt(hd)
    # the bench's own lengths: 512 + (u64 mod 32257) from its seed
    rng = np.random.Generator(np.random.Philox(key=[0x7C0DE005, 0]))
    lens = (512 + rng.integers(0, 32257, nseq, dtype=np.uint64)).astype(np.int64)
    base = np.zeros(nseq, dtype=np.int64)
    base[1:] = np.cumsum(lens[:-1] + 16)
    rows = int((lens + 16).sum())
    k8, v8, ks, vs = _build_store(rows - 16, nKV, hd, seed=0xC5)
    q = _randn((nseq, nH, hd), 0xC5 + 1)
    out = torch.full((nseq, nH, hd), float("nan"), device="cuda")
    maxlen = int(lens.max())
    _, chunks = ops.split_geometry(maxlen, nH, hd)
    chunks = min(chunks, 64)
    ws = ops.workspace(nseq, nH, hd, chunks)
    dlens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    dbase = torch.tensor(base, dtype=torch.int64, device="cuda")
    ops.decode_i8_batch(q, k8, v8, ks, vs, out, ws, dlens, nseq, nH, nKV, hd, maxlen, chunks, row_base=dbase,
                        invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    hk8, hv8, hks, hvs, hq, got = host(k8), host(v8), host(ks), host(vs), host(q), host(out)

    def one(b):
        r0, n = int(base[b]), int(lens[b])
        return oracle.attention_i8(hq[b:b + 1], hk8[r0:r0 + n], hv8[r0:r0 + n], hks[r0:r0 + n], hvs[r0:r0 + n], 1, nH,
                                   nKV, hd, n - 1, inv)

    with ThreadPoolExecutor(8) as ex:          # the C checker runs outside the interpreter lock
        wants = list(ex.map(one, range(nseq)))
    for b in range(nseq):
        assert_close(got[b:b + 1], wants[b], what=f"C5 sequence {b} ({int(lens[b])} rows)")


def test_c3_prefill_4096_rows_and_the_int8_mirror():
    nH, nKV, hd, S = 28, 4, 128, 4096
    inv = 1.0 / math.sqrt(hd)
    q, k, v = _randn((S, nH, hd), 0xC3), _randn((S, nKV, hd), 0xC3 + 1), _randn((S, nKV, hd), 0xC3 + 2)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    n = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 1024
    # the int8 mirror of all 4096 positions, as the configuration asks: written by the launch that
    # makes the fp16 twins
    k8 = torch.zeros((S + 16, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.zeros_like(k8)
    ks = torch.zeros((S + 16, nKV), device="cuda")
    vs = torch.zeros_like(ks)
    ops.prefill_f16(q, k, v, out, buf[off:off + n], S, nH, nKV, hd, invSqrt=inv, kv8=(k8, v8, ks, vs))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    hq, hk, hv, got = host(q), host(k), host(v), host(out)
    assert np.isfinite(got).all()
    w8 = oracle.quant_kv8(hk, hv, nKV, hd)
    assert np.array_equal(host(k8[:S]), w8[0]) and np.array_equal(host(v8[:S]), w8[1]), "mirror bytes"
    assert np.array_equal(host(ks[:S]), w8[2]) and np.array_equal(host(vs[:S]), w8[3]), "mirror scales"
    # a sample of rows against the materialised-path restatement: every 64th row, the tile
    # edges, the last 256 rows (the CPU needs only those rows' scores)
    rows = sorted(set(range(0, S, 64)) | {127, 128, 129, 255, 256, 257, 2047, 2048, 2049} | set(range(S - 256, S)))
    parts = np.array_split(np.array(rows, np.uint32), 8)

    def some(r):
        return oracle.prefill_f16_rows(hq, hk, hv, r, S, nH, nKV, hd, inv)

    with ThreadPoolExecutor(8) as ex:
        want = np.concatenate(list(ex.map(some, parts)))
    assert_close(got[rows], want, rtol=2e-2, atol=2e-3, what="C3 prefill, 4096 rows (row sample)")
