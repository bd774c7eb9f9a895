"""Causal fp16 prefill on tcgen05 against the oracle's restatement of the
reference's materialised path (fp16 operands, f32 accumulation, fp16
probabilities).  Tolerance for this path: 2e-2 (relative), as the reference's own
fp16-vs-f32 comparison allows (max abs diff 0.0146 on its outputs)."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu

RTOL16, ATOL16 = 2e-2, 2e-3


def _run(S, nH, nKV, seed, scale=1.0):
    hd = 128
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((S, nH, hd), dtype=np.float32) * scale
    k = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    inv = 1.0 / math.sqrt(hd)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    nbytes = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd)
    scratch = torch.empty(nbytes + 1024, dtype=torch.uint8, device="cuda")
    off = (-scratch.data_ptr()) % 1024
    ops.prefill_f16(dev(q), dev(k), dev(v), out, scratch[off:off + nbytes], S, nH, nKV, hd, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    return q, k, v, got, inv


@pytest.mark.parametrize("S,nH,nKV", [(128, 1, 1), (256, 4, 2), (300, 8, 2), (1, 4, 4), (129, 7, 1), (512, 28, 4)])
def test_against_materialised_reference_path(S, nH, nKV):
    q, k, v, got, inv = _run(S, nH, nKV, seed=S + nH)
    want = oracle.prefill_f16(q, k, v, S, nH, nKV, 128, inv)
    assert_close(got, want, rtol=RTOL16, atol=ATOL16, what=f"prefill_f16 S={S} nH={nH}")
    # and close to exact attention on the fp16-rounded operands (shows where both sit)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, S, nH, nKV, 128, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="vs f64 on fp16 operands")


def test_long_rows_and_peaked_scores():
    # 1536 rows: 12 query tiles, lazy rescale exercised by scores with a wide range
    q, k, v, got, inv = _run(1536, 4, 2, seed=5, scale=6.0)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, 1536, 4, 2, 128, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="peaked scores")


def test_matches_f32_causal_kernel_within_fp16_tolerance():
    q, k, v, got, inv = _run(384, 8, 4, seed=9)
    out = torch.empty((384, 8, 128), device="cuda")
    ops.prefill_kv(dev(q), dev(k), dev(v), out, 384, 8, 4, 128, 0, invSqrt=inv)
    assert_close(got, host(out), rtol=RTOL16, atol=2e-2, what="fp16 tcgen05 vs f32 kernel")


def test_scratch_too_small_is_refused():
    q = torch.zeros((128, 4, 128), device="cuda")
    k = torch.zeros((128, 2, 128), device="cuda")
    s = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.TcError) as e:
        ops.prefill_f16(q, k, k, q.clone(), s, 128, 4, 2, 128)
    assert e.value.code == capi.TC_EWORKSPACE
