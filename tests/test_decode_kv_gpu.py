"""f32-cache attention on the GPU against the oracle: split-KV decode (with the
Q8_1 epilogue), and the unsplit causal kernel for several query rows."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu


def _case(nH, nKV, hd, ctx, seed, pad=0, poison=True):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k = rng.standard_normal((ctx + pad, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((ctx + pad, nKV, hd), dtype=np.float32)
    if pad and poison:
        k[ctx:] = np.nan   # rows past the position hold whatever was there before
        v[ctx:] = np.nan
    return q, k, v


def _decode(nH, nKV, hd, ctx, numChunks, seed, pad=0, dev_pos=False, q81=False):
    q, k, v = _case(nH, nKV, hd, ctx, seed, pad)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_kv(q, k[:ctx], v[:ctx], 1, nH, nKV, hd, ctx - 1, inv)
    exact = oracle.attention_f64(q, k[:ctx], v[:ctx], None, None, 1, nH, nKV, hd, ctx - 1, inv)
    out = torch.full((1, nH, hd), float("nan"), device="cuda")
    ws = ops.workspace(1, nH, hd, numChunks)
    for w in ws:
        w.fill_(float("nan"))
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda") if dev_pos else None
    blocks = torch.zeros(nH * (hd // 32) * 40, dtype=torch.uint8, device="cuda") if q81 else None
    ops.decode_kv(dev(q), dev(k), dev(v), out, ws, 1, nH, nKV, hd, ctx - 1 + (pad if dev_pos else 0), numChunks,
                  invSqrt=inv, dev_pos=pos, q81=blocks)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert_close(got, want, what=f"decode_kv {nH}/{nKV}/{hd} ctx {ctx} vs oracle")
    assert_close(got, exact, what=f"decode_kv {nH}/{nKV}/{hd} ctx {ctx} vs f64")
    if q81:
        assert np.array_equal(host(blocks), oracle.q8_1_blocks(got))
    return got, want


@pytest.mark.parametrize("ctx", [1, 2, 15, 16, 17, 63, 64, 65, 500, 2048])
def test_qwen05b_shape(ctx):
    # 14 q heads, 2 kv heads, head_dim 64: the f32 decode configuration
    _decode(14, 2, 64, ctx, numChunks=64, seed=ctx)


@pytest.mark.parametrize("nH,nKV,hd,ctx", [(28, 4, 128, 1000), (40, 8, 128, 777), (12, 2, 128, 300), (8, 8, 64, 200),
                                          (7, 1, 64, 90), (9, 3, 128, 33), (16, 4, 64, 4096),
                                          (32, 2, 64, 400), (18, 2, 128, 200), (9, 1, 64, 150),
                                          (16, 2, 256, 700), (8, 8, 256, 100), (24, 4, 256, 3000), (7, 1, 256, 33)])
def test_shapes(nH, nKV, hd, ctx):
    _decode(nH, nKV, hd, ctx, numChunks=128, seed=nH + ctx)


def test_stale_rows_device_position_and_q81():
    _decode(14, 2, 64, 1500, numChunks=64, seed=1, pad=100)
    _decode(14, 2, 64, 1500, numChunks=64, seed=2, pad=300, dev_pos=True)
    _decode(28, 4, 128, 900, numChunks=32, seed=3, q81=True)
    _decode(14, 2, 64, 20, numChunks=32, seed=4, q81=True)   # one chunk, still merged for the blocks


def test_cpu_engine_path_agrees():
    # Model::attentionFused (block-32 online softmax, -inf start) and the GPU rule give the same numbers
    q, k, v = _case(14, 2, 64, 700, 11)
    got, want = _decode(14, 2, 64, 700, 64, 11)
    cpu = oracle.attention_fused_cpu(q, k, v, 1, 699, 14, 2, 64)
    assert_close(got, cpu, what="GPU kernel vs CPU engine restatement")
    if oracle.ref_available() and oracle.ref().has_avx512():
        ref = oracle.ref().attention_fused(q, k, v, 699, 1, 14, 2, 64)[0]
        assert_close(got, ref, what="GPU kernel vs reference leaves + pool")


@pytest.mark.parametrize("nH,nKV,hd,ctx,numChunks", [(14, 2, 64, 2048, 64), (14, 2, 64, 1, 64), (14, 2, 64, 17, 64),
                                                    (28, 4, 128, 1000, 128), (40, 8, 128, 5000, 32),
                                                    (12, 2, 128, 129, 1), (7, 1, 64, 300, 16), (8, 8, 64, 63, 8),
                                                    (24, 2, 64, 500, 16), (20, 2, 128, 260, 32)])
def test_fp16_cache_decode(nH, nKV, hd, ctx, numChunks):
    """The dense models' optional fp16 cache (KVT = __half in the reference): same rule, the
    products see float(k), float(v).  Rows behind the position hold NaN."""
    rng = np.random.default_rng(ctx * 3 + nH)
    pad = 40
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k = rng.standard_normal((ctx + pad, nKV, hd), dtype=np.float32).astype(np.float16)
    v = (rng.standard_normal((ctx + pad, nKV, hd), dtype=np.float32) * 3).astype(np.float16)
    k[ctx:] = np.nan
    v[ctx:] = np.nan
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_kv(q, k[:ctx], v[:ctx], 1, nH, nKV, hd, ctx - 1, inv)
    out = torch.full((1, nH, hd), float("nan"), device="cuda")
    ws = ops.workspace(1, nH, hd, numChunks)
    for w in ws:
        w.fill_(float("nan"))
    ops.decode_kv(dev(q), dev(k), dev(v), out, ws, 1, nH, nKV, hd, ctx - 1, numChunks, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), want, what=f"fp16 cache decode {nH}/{nKV}/{hd} ctx {ctx}")
    # device position (host value = upper bound) and the Q8_1 epilogue
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    blocks = torch.zeros(nH * (hd // 32) * 40, dtype=torch.uint8, device="cuda")
    out2 = torch.full((1, nH, hd), float("nan"), device="cuda")
    ops.decode_kv(dev(q), dev(k), dev(v), out2, ws, 1, nH, nKV, hd, ctx - 1 + pad, numChunks, invSqrt=inv, dev_pos=pos,
                  q81=blocks)
    torch.cuda.synchronize()
    assert_close(host(out2), want, what="fp16 cache decode, device position")
    assert np.array_equal(host(blocks), oracle.q8_1_blocks(host(out2)))


@pytest.mark.parametrize("S,nH,nKV,hd,cachePos", [(37, 14, 2, 64, 0), (8, 28, 4, 128, 100), (129, 12, 2, 128, 17)])
def test_fp16_cache_causal_rows(S, nH, nKV, hd, cachePos):
    rng = np.random.default_rng(S + cachePos + 1)
    rows = cachePos + S
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((rows + 5, nKV, hd), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((rows + 5, nKV, hd), dtype=np.float32).astype(np.float16)
    k[rows:] = np.nan
    v[rows:] = np.nan
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_kv(q, k, v, S, nH, nKV, hd, cachePos, inv)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_kv(dev(q), dev(k), dev(v), out, S, nH, nKV, hd, cachePos, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), want, what="fp16 cache causal rows")


def test_append_then_attend_fp16_cache():
    """tc_kv_append into an fp16 cache, then decode over it: the pair the dense engine runs per token."""
    nH, nKV, hd, ctx = 14, 2, 64, 300
    rng = np.random.default_rng(8)
    kf = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
    vf = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    kc = torch.zeros((ctx + 8, nKV, hd), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.kv_append(dev(kf), dev(vf), kc, vc, ctx, nKV, hd, 0)
    assert np.array_equal(host(kc)[:ctx], kf.astype(np.float16))     # round-to-nearest-even, as __float2half_rn
    out = torch.empty((1, nH, hd), device="cuda")
    ops.decode_kv(dev(q), kc, vc, out, ops.workspace(1, nH, hd, 32), 1, nH, nKV, hd, ctx - 1, 32)
    want = oracle.attention_kv(q, kf.astype(np.float16), vf.astype(np.float16), 1, nH, nKV, hd, ctx - 1, 1.0 / math.sqrt(hd))
    assert_close(host(out), want, what="append + decode, fp16 cache")


@pytest.mark.parametrize("S,nH,nKV,hd,cachePos", [(37, 14, 2, 64, 0), (8, 28, 4, 128, 100), (1, 14, 2, 64, 55),
                                                 (129, 12, 2, 128, 17), (64, 8, 8, 64, 0), (21, 8, 2, 256, 40),
                                                 (70, 16, 4, 256, 0)])
def test_causal_rows(S, nH, nKV, hd, cachePos):
    rng = np.random.default_rng(S + cachePos)
    rows = cachePos + S
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((rows + 5, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((rows + 5, nKV, hd), dtype=np.float32)
    k[rows:] = np.nan
    v[rows:] = np.nan
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_kv(q, k, v, S, nH, nKV, hd, cachePos, inv)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_kv(dev(q), dev(k), dev(v), out, S, nH, nKV, hd, cachePos, invSqrt=inv)
    torch.cuda.synchronize()
    assert_close(host(out), want, what="causal rows f32")
    pos = torch.tensor([cachePos], dtype=torch.int32, device="cuda")
    out2 = torch.empty_like(out)
    ops.prefill_kv(dev(q), dev(k), dev(v), out2, S, nH, nKV, hd, 0, invSqrt=inv, dev_pos=pos)
    assert torch.equal(out, out2)
    if S > 1:  # the decode entry point with several rows takes the same kernel
        out3 = torch.empty_like(out)
        ops.decode_kv(dev(q), dev(k), dev(v), out3, ops.workspace(1, nH, hd, 4), S, nH, nKV, hd, cachePos, 4,
                      invSqrt=inv)
        assert torch.equal(out, out3)


def test_window_guard():
    q = torch.zeros((4, 14, 64), device="cuda")
    k = torch.zeros((8, 2, 64), device="cuda")
    with pytest.raises(capi.ContextFull):
        ops.prefill_kv(q, k, k, q.clone(), 4, 14, 2, 64, 6)
    with pytest.raises(capi.ContextFull):
        ops.decode_kv(q[:1], k, k, q[:1].clone(), ops.workspace(1, 14, 64, 4), 1, 14, 2, 64, 8, 4)
