"""Pins the CPU restatement (oracle/tc_oracle.c) against outputs of the reference
project's OWN CUDA kernels, recorded on a B200 by tests/golden/make_ref_gpu_golden.py
(tests/golden/ref_gpu_golden.npz).  Integer / byte outputs must match exactly; float
outputs differ only by the device's exp2f / __expf versus libm (a few ulp)."""
import math
import os

import numpy as np
import pytest

import oracle
from tests.golden import ref_gpu_cases as cases

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_golden.npz"))
C = cases.CASES
FTOL = dict(rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("name,case_id", [("quant_hd128", 1), ("quant_hd256", 2)])
def test_quantiser_is_bit_exact(name, case_id):
    c = C[name]
    k, v = cases.quant_case(case_id, c["tokens"], c["nKV"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    assert np.array_equal(k8, G[f"{name}.k8"]) and np.array_equal(v8, G[f"{name}.v8"])
    assert np.array_equal(ks, G[f"{name}.ks"]) and np.array_equal(vs, G[f"{name}.vs"])


def test_int8_decode_split_eager_and_partials():
    c = C["decode_i8"]
    k, v = cases.store_case(3, c["ctx"], c["nKV"], c["hd"])
    q = cases.q_case(3, 1, c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    inv = 1.0 / math.sqrt(c["hd"])
    acc, m, l = oracle.decode_i8_split(q, k8, v8, ks, vs, c["nH"], c["nKV"], c["hd"], c["ctx"] - 1, c["chunks"],
                                       c["chunk"], inv)
    np.testing.assert_allclose(m, G["decode_i8.partM"], **FTOL)
    np.testing.assert_allclose(l, G["decode_i8.partL"], rtol=2e-5, atol=1e-6)
    out = oracle.combine_partials(acc, m, l, 1, c["nH"], c["chunks"], c["hd"])
    np.testing.assert_allclose(out, G["decode_i8.split_out"], **FTOL)
    eager = oracle.attention_i8(q, k8, v8, ks, vs, 1, c["nH"], c["nKV"], c["hd"], c["ctx"] - 1, inv)
    np.testing.assert_allclose(eager, G["decode_i8.eager_out"], **FTOL)


def test_int8_prefill():
    c = C["prefill_i8"]
    k, v = cases.store_case(4, c["cachePos"] + c["S"], c["nKV"], c["hd"])
    q = cases.q_case(4, c["S"], c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    out = oracle.attention_i8(q, k8, v8, ks, vs, c["S"], c["nH"], c["nKV"], c["hd"], c["cachePos"],
                              1.0 / math.sqrt(c["hd"]))
    np.testing.assert_allclose(out, G["prefill_i8.out"], **FTOL)


@pytest.mark.parametrize("name,case_id", [("decode_f32_c1", 5), ("decode_f32_7b", 6)])
def test_f32_split_decode_and_q81_blocks(name, case_id):
    c = C[name]
    k, v = cases.store_case(case_id, c["ctx"], c["nKV"], c["hd"])
    q = cases.q_case(case_id, 1, c["nH"], c["hd"])
    inv = 1.0 / math.sqrt(c["hd"])
    # the reference launcher regroups the same online softmax (sub-warps, 8-warp merge): tolerance, not bits
    acc, m, l = oracle.decode_kv_split(q, k, v, 1, c["nH"], c["nKV"], c["hd"], c["ctx"] - 1, c["chunks"], c["chunk"],
                                       inv)
    out = oracle.combine_partials(acc, m, l, 1, c["nH"], c["chunks"], c["hd"])
    np.testing.assert_allclose(out, G[f"{name}.out"], **FTOL)
    # the Q8_1 fold is a byte format: exact on the values the reference itself produced
    assert np.array_equal(oracle.q8_1_blocks(G[f"{name}.out"]), G[f"{name}.q81"])


def test_unsplit_causal_f32():
    c = C["attention_f32"]
    k, v = cases.store_case(7, c["cachePos"] + c["S"], c["nKV"], c["hd"])
    q = cases.q_case(7, c["S"], c["nH"], c["hd"])
    out = oracle.attention_kv(q, k, v, c["S"], c["nH"], c["nKV"], c["hd"], c["cachePos"], 1.0 / math.sqrt(c["hd"]))
    np.testing.assert_allclose(out, G["attention_f32.out"], **FTOL)


def test_rope_and_append_are_bit_exact():
    c = C["rope_store"]
    cosT, sinT = oracle.rope_tables(c["rows"], c["hd"], c["theta"])
    kS, vS = cases.store_case(8, c["S"], c["nKV"], c["hd"])
    q = cases.q_case(8, c["S"], c["nH"], c["hd"])
    assert np.array_equal(oracle.rope_q(q, cosT, sinT, c["S"], c["nH"], c["hd"], c["cachePos"]), G["rope_store.q"])
    kD = np.zeros((c["rows"], c["nKV"], c["hd"]), np.float32)
    vD = np.zeros_like(kD)
    oracle.kv_append(kS, vS, kD, vD, c["S"], c["nKV"], c["hd"], c["cachePos"], c["cachePos"], cosT, sinT)
    assert np.array_equal(kD, G["rope_store.k"]) and np.array_equal(vD, G["rope_store.v"])


def test_merge_and_q81_fold():
    c = C["combine_q81"]
    acc, m, l = cases.partials_case(9, c["nH"], c["chunks"], c["hd"])
    out = oracle.combine_partials(acc, m, l, 1, c["nH"], c["chunks"], c["hd"])
    np.testing.assert_allclose(out, G["combine_q81.out"], **FTOL)     # 8-warp regrouping: tolerance
    assert np.array_equal(oracle.q8_1_blocks(G["combine_q81.out"]), G["combine_q81.q81"])


def test_sigmoid_gate():
    c = C["sigmoid_gate"]
    o = cases.q_case(10, c["S"], c["nH"], c["hd"])
    g = cases.q_case(11, c["S"], c["nH"], 2 * c["hd"]) * 4
    np.testing.assert_allclose(oracle.sigmoid_gate(o, g, c["S"], c["nH"], c["hd"]), G["sigmoid_gate.out"],
                               rtol=1e-5, atol=1e-6)


def test_causal_softmax_rows_of_the_materialised_prefill():
    """kAttnSoftmaxCausal: mx = max(score)*scale, p = exp2((s*scale - mx)*log2e)/sum as fp16, zeros past the row."""
    c = C["softmax_causal"]
    sc = cases.q_case(12, c["nH"], c["S"], c["S"]) * 20
    want = G["softmax_causal.p"].astype(np.float32)
    got = np.zeros_like(want)
    for h in range(c["nH"]):
        for r in range(c["S"]):
            s = sc[h, r, :r + 1].astype(np.float64) * c["scale"]
            e = np.exp(s - s.max())
            got[h, r, :r + 1] = (e / e.sum()).astype(np.float16).astype(np.float32)
    assert (want[:, np.triu_indices(c["S"], 1)[0], np.triu_indices(c["S"], 1)[1]] == 0).all()
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=1e-6)     # one fp16 ulp


A8 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_golden_a8.npz")


@pytest.mark.parametrize("idx,name", list(enumerate(cases.A8_CASES)))
def test_materialised_prefill(idx, name):
    """The fp16 prefill restatement against the reference's whole materialised path run on a
    B200 (its kF32ToF16 and kAttnSoftmaxCausal kernels around the two cuBLAS products it
    issues).  The order of the f32 accumulation inside the library products is not defined, so
    an fp16 probability can land on the neighbouring value: tolerance 1e-3 relative, twenty
    times tighter than the 2e-2 bar of the fp16 prefill itself."""
    g = np.load(A8)
    c = cases.A8_CASES[name]
    q, k, v = cases.a8_case(40 + idx, c)
    rows = cases.a8_rows(c["S"])
    got = oracle.prefill_f16_rows(q, k, v, rows, c["S"], c["nH"], c["nKV"], c["hd"], 1.0 / math.sqrt(c["hd"]))
    want = g[f"{name}.out_rows"]
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)
