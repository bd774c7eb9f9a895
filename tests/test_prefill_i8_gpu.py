"""Causal attention of several query rows over the int8 store against the oracle."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import assert_close, dev, host, make_i8_store

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,nH,nKV,cachePos,hd", [(37, 28, 4, 0, 128), (8, 28, 4, 100, 128), (1, 28, 4, 55, 128),
                                                 (300, 12, 2, 17, 128), (64, 40, 8, 0, 128), (9, 8, 8, 1000, 128),
                                                 (5, 4, 2, 40, 256), (70, 16, 4, 0, 256), (13, 8, 2, 600, 256)])
def test_causal_rows_over_int8_store(S, nH, nKV, cachePos, hd):
    rng = np.random.default_rng(S * 7 + cachePos)
    rows = cachePos + S
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((rows, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((rows, nKV, hd), dtype=np.float32), nKV, hd, extra_rows=9)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8[:rows], v8[:rows], ks[:rows], vs[:rows], S, nH, nKV, hd, cachePos, inv)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, S, nH, nKV, hd, cachePos, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), want, what="causal rows int8")
    pos = torch.tensor([cachePos], dtype=torch.int32, device="cuda")
    out2 = torch.empty_like(out)
    ops.prefill_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out2, S, nH, nKV, hd, 0, invSqrt=inv, dev_pos=pos)
    assert torch.equal(out, out2)


def test_chunked_prefill_carry_matches_single_prefill():
    """Two 48-row calls carrying the store equal one 96-row call (the reference's
    split-prefill check, unit_tests/ModelTest.cpp:279-325, at kernel level)."""
    nH, nKV, hd, S = 28, 4, 128, 96
    rng = np.random.default_rng(2)
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    kd, vd, qd = dev(k), dev(v), dev(q)
    k8 = torch.zeros((S + 16, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.zeros_like(k8)
    ks = torch.zeros((S + 16, nKV), device="cuda")
    vs = torch.zeros_like(ks)
    whole = torch.empty((S, nH, hd), device="cuda")
    ops.kv_quantize_i8(kd, vd, k8, v8, ks, vs, S, nKV, hd)
    ops.prefill_i8(qd, k8, v8, ks, vs, whole, S, nH, nKV, hd, 0)
    k8b, v8b, ksb, vsb = torch.zeros_like(k8), torch.zeros_like(v8), torch.zeros_like(ks), torch.zeros_like(vs)
    parts = torch.empty_like(whole)
    for c in range(2):
        ops.kv_quantize_i8(kd, vd, k8b, v8b, ksb, vsb, 48, nKV, hd, dst_base=48 * c, src_base=48 * c)
        ops.prefill_i8(qd[48 * c:48 * c + 48], k8b, v8b, ksb, vsb, parts[48 * c:48 * c + 48], 48, nH, nKV, hd, 48 * c)
    torch.cuda.synchronize()
    assert torch.equal(whole, parts)


def test_guard():
    q = torch.zeros((4, 28, 128), device="cuda")
    k8 = torch.zeros((8, 4, 128), dtype=torch.int8, device="cuda")
    s = torch.zeros((8, 4), device="cuda")
    with pytest.raises(capi.ContextFull):
        ops.prefill_i8(q, k8, k8, s, s, q.clone(), 4, 28, 4, 128, 6)
