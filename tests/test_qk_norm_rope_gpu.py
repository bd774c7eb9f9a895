"""Q/K RMSNorm + partial rotation (the gated models' step in front of attention) and the
rotation tables: against the oracle, and bit for bit against outputs recorded from the
reference's own kernels on a B200 (tests/golden/ref_gpu_golden_f2.npz)."""
import os

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.golden import ref_gpu_cases as cases
from tests.util import assert_close, dev, host

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_golden_f2.npz")


def test_tables_equal_the_oracle_bitwise():
    for rows, hd, theta in ((40, 64, 1e6), (17, 128, 1e4), (9, 256, 1e7)):
        c, s = ops.rope_tables(rows, hd, theta)
        oc, os_ = oracle.rope_tables(rows, hd, theta)
        assert np.array_equal(c, oc) and np.array_equal(s, os_)
    for rows, nd, theta in ((33, 64, 1e7), (12, 128, 1e6), (5, 32, 1e4)):
        c, s = ops.mrope_tables(rows, nd, theta)
        oc, os_ = oracle.mrope_tables(rows, nd, theta)
        assert np.array_equal(c, oc) and np.array_equal(s, os_)
        assert c[0].tolist() == [1.0] * (nd // 2) and not s[0].any()


def _run(c, case_id, dev_pos=False):
    qg, k, wq, wk = cases.norm_rope_case(case_id, c)
    cosT, sinT = oracle.mrope_tables(c["rows"], c["nDims"], c["theta"])
    qOut = torch.full((c["S"], c["nH"], c["hd"]), float("nan"), device="cuda")
    dk = dev(k)
    pos = torch.tensor([c["pos"]], dtype=torch.int32, device="cuda") if dev_pos else None
    ops.qk_norm_rope(dev(qg), qOut, dk, dev(wq), dev(wk), c["hd"], c["nDims"], c["nH"], c["nKV"], c["S"],
                     0 if dev_pos else c["pos"], dev(cosT), dev(sinT), dev_pos=pos)
    torch.cuda.synchronize()
    return qg, k, wq, wk, cosT, sinT, host(qOut), host(dk)


@pytest.mark.gpu
@pytest.mark.parametrize("i,name", list(enumerate(cases.CASES_F2)))
def test_norm_rope_against_oracle_and_reference_kernels(i, name):
    c = cases.CASES_F2[name]
    qg, k, wq, wk, cosT, sinT, gq, gk = _run(c, 20 + i)
    wq_ = oracle.norm_rope(qg, wq, c["hd"], c["nDims"], c["nH"], c["S"], c["pos"], cosT, sinT, in_stride=2 * c["hd"])
    wk_ = oracle.norm_rope(k, wk, c["hd"], c["nDims"], c["nKV"], c["S"], c["pos"], cosT, sinT)
    # the oracle's 1/sqrtf differs from the device rsqrtf in the last bits
    assert_close(gq, wq_, rtol=2e-6, atol=1e-7, what="q norm+rope vs oracle")
    assert_close(gk, wk_, rtol=2e-6, atol=1e-7, what="k norm+rope vs oracle")
    # a device position gives the same bits as the host position
    _, _, _, _, _, _, gq2, gk2 = _run(c, 20 + i, dev_pos=True)
    assert np.array_equal(gq, gq2) and np.array_equal(gk, gk2)
    G = np.load(GOLD)
    assert np.array_equal(gq, G[f"{name}.q"]), "q differs from kQ35QNormRoPE"
    assert np.array_equal(gk, G[f"{name}.k"]), "k differs from kQ35KNormRoPE"


@pytest.mark.parametrize("i,name", list(enumerate(cases.CASES_F2)))
def test_oracle_against_reference_kernels(i, name):
    """CPU: the restatement reproduces the recorded kernel outputs (to the rsqrt difference)."""
    c = cases.CASES_F2[name]
    qg, k, wq, wk = cases.norm_rope_case(20 + i, c)
    cosT, sinT = oracle.mrope_tables(c["rows"], c["nDims"], c["theta"])
    G = np.load(GOLD)
    q_ = oracle.norm_rope(qg, wq, c["hd"], c["nDims"], c["nH"], c["S"], c["pos"], cosT, sinT, in_stride=2 * c["hd"])
    k_ = oracle.norm_rope(k, wk, c["hd"], c["nDims"], c["nKV"], c["S"], c["pos"], cosT, sinT)
    assert_close(q_, G[f"{name}.q"], rtol=2e-6, atol=1e-7, what="oracle q vs reference kernel")
    assert_close(k_, G[f"{name}.k"], rtol=2e-6, atol=1e-7, what="oracle k vs reference kernel")


@pytest.mark.gpu
def test_either_side_alone_and_guards():
    c = cases.CASES_F2["qk_norm_rope_128"]
    qg, k, wq, wk = cases.norm_rope_case(21, c)
    cosT, sinT = oracle.mrope_tables(c["rows"], c["nDims"], c["theta"])
    dc, ds = dev(cosT), dev(sinT)
    dk = dev(k)
    ops.qk_norm_rope(None, None, dk, None, dev(wk), c["hd"], c["nDims"], c["nH"], c["nKV"], c["S"], c["pos"], dc, ds)
    want = oracle.norm_rope(k, wk, c["hd"], c["nDims"], c["nKV"], c["S"], c["pos"], cosT, sinT)
    assert_close(host(dk), want, rtol=2e-6, atol=1e-7, what="k alone")
    qOut = torch.empty((c["S"], c["nH"], c["hd"]), device="cuda")
    ops.qk_norm_rope(dev(qg), qOut, None, dev(wq), None, c["hd"], c["nDims"], c["nH"], c["nKV"], c["S"], c["pos"], dc, ds)
    want = oracle.norm_rope(qg, wq, c["hd"], c["nDims"], c["nH"], c["S"], c["pos"], cosT, sinT, in_stride=2 * c["hd"])
    assert_close(host(qOut), want, rtol=2e-6, atol=1e-7, what="q alone")
    with pytest.raises(capi.ContextFull):      # position past the table
        ops.qk_norm_rope(None, None, dk, None, dev(wk), c["hd"], c["nDims"], c["nH"], c["nKV"], c["S"], c["rows"], dc, ds)
    with pytest.raises(capi.TcError):          # odd number of rotated dims
        ops.qk_norm_rope(None, None, dk, None, dev(wk), c["hd"], 7, c["nH"], c["nKV"], c["S"], 0, dc, ds)
