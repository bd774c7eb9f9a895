"""The library's kernels against outputs recorded from the reference project's own
CUDA kernels on a B200 (tests/golden/ref_gpu_golden.npz): same seeded inputs, the
reference's result on one side, ours on the other -- no oracle in between."""
import math
import os

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import ops
from tests.golden import ref_gpu_cases as cases
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_golden.npz"))
C = cases.CASES


@pytest.mark.parametrize("name,case_id", [("quant_hd128", 1), ("quant_hd256", 2)])
def test_quantiser_equals_reference_kernel_bytes(name, case_id):
    c = C[name]
    k, v = cases.quant_case(case_id, c["tokens"], c["nKV"], c["hd"])
    k8 = torch.zeros((c["tokens"], c["nKV"], c["hd"]), dtype=torch.int8, device="cuda")
    v8 = torch.zeros_like(k8)
    ks = torch.zeros((c["tokens"], c["nKV"]), device="cuda")
    vs = torch.zeros_like(ks)
    ops.kv_quantize_i8(dev(k), dev(v), k8, v8, ks, vs, c["tokens"], c["nKV"], c["hd"])
    for key, t in (("k8", k8), ("v8", v8), ("ks", ks), ("vs", vs)):
        assert np.array_equal(host(t), G[f"{name}.{key}"]), key


@pytest.mark.parametrize("name,case_id", [("decode_f32_c1", 5), ("decode_f32_7b", 6)])
def test_f32_decode_equals_reference_launcher(name, case_id):
    c = C[name]
    k, v = cases.store_case(case_id, c["ctx"], c["nKV"], c["hd"])
    q = cases.q_case(case_id, 1, c["nH"], c["hd"])
    out = torch.empty((1, c["nH"], c["hd"]), device="cuda")
    q81 = torch.zeros(c["nH"] * (c["hd"] // 32) * 40, dtype=torch.uint8, device="cuda")
    ops.decode_kv(dev(q), dev(k), dev(v), out, ops.workspace(1, c["nH"], c["hd"], c["chunks"]), 1, c["nH"], c["nKV"],
                  c["hd"], c["ctx"] - 1, c["chunks"], c["chunk"], 1.0 / math.sqrt(c["hd"]), q81=q81)
    assert_close(host(out), G[f"{name}.out"], what=name)
    # the Q8_1 bytes follow our own f32 output exactly; against the reference's bytes allow the
    # last-digit differences that a 1e-3 output tolerance implies: quantised values within one step
    ours = host(q81).reshape(-1, 40)[:, 4:].view(np.int8).astype(np.int32)
    theirs = G[f"{name}.q81"].reshape(-1, 40)[:, 4:].view(np.int8).astype(np.int32)
    assert np.abs(ours - theirs).max() <= 1


def test_int8_decode_equals_reference_kernels():
    """kQ35WarpAttention8Split + kAttnCombinePartial and the eager kQ35WarpAttention8 at the
    reference's own shape (head_dim 256), store built by the pinned quantiser."""
    c = C["decode_i8"]
    k, v = cases.store_case(3, c["ctx"], c["nKV"], c["hd"])
    q = cases.q_case(3, 1, c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    out = torch.empty((1, c["nH"], c["hd"]), device="cuda")
    ops.decode_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, ops.workspace(1, c["nH"], c["hd"], c["chunks"]),
                  c["nH"], c["nKV"], c["hd"], c["ctx"] - 1, c["chunks"], c["chunk"], 1.0 / math.sqrt(c["hd"]))
    assert_close(host(out), G["decode_i8.split_out"], what="int8 split decode")
    assert_close(host(out), G["decode_i8.eager_out"], what="int8 eager decode")


def test_int8_prefill_equals_reference_kernel():
    c = C["prefill_i8"]
    rows = c["cachePos"] + c["S"]
    k, v = cases.store_case(4, rows, c["nKV"], c["hd"])
    q = cases.q_case(4, c["S"], c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    out = torch.empty((c["S"], c["nH"], c["hd"]), device="cuda")
    ops.prefill_i8(dev(q), dev(k8), dev(v8), dev(ks), dev(vs), out, c["S"], c["nH"], c["nKV"], c["hd"], c["cachePos"],
                   invSqrt=1.0 / math.sqrt(c["hd"]))
    assert_close(host(out), G["prefill_i8.out"], what="kQ35WarpAttention8Prefill")


def test_causal_rows_equal_reference_kernel():
    c = C["attention_f32"]
    k, v = cases.store_case(7, c["cachePos"] + c["S"], c["nKV"], c["hd"])
    q = cases.q_case(7, c["S"], c["nH"], c["hd"])
    out = torch.empty((c["S"], c["nH"], c["hd"]), device="cuda")
    ops.prefill_kv(dev(q), dev(k), dev(v), out, c["S"], c["nH"], c["nKV"], c["hd"], c["cachePos"])
    assert_close(host(out), G["attention_f32.out"], what="kWarpAttention")


def test_rope_and_append_equal_reference_kernels_bitwise():
    c = C["rope_store"]
    cosT, sinT = oracle.rope_tables(c["rows"], c["hd"], c["theta"])
    kS, vS = cases.store_case(8, c["S"], c["nKV"], c["hd"])
    q = dev(cases.q_case(8, c["S"], c["nH"], c["hd"]))
    kD = torch.zeros((c["rows"], c["nKV"], c["hd"]), device="cuda")
    vD = torch.zeros_like(kD)
    ops.kv_append_rope(q, dev(kS), dev(vS), kD, vD, c["S"], c["nH"], c["nKV"], c["hd"], c["cachePos"], c["cachePos"],
                       dev(cosT), dev(sinT))
    assert np.array_equal(host(q), G["rope_store.q"])
    assert np.array_equal(host(kD), G["rope_store.k"]) and np.array_equal(host(vD), G["rope_store.v"])


def test_merge_and_gate_equal_reference_kernels():
    c = C["combine_q81"]
    acc, m, l = cases.partials_case(9, c["nH"], c["chunks"], c["hd"])
    out = torch.empty((1, c["nH"], c["hd"]), device="cuda")
    ops.merge_partials(dev(acc), dev(m), dev(l), out, 1, c["nH"], c["chunks"], c["hd"])
    assert_close(host(out), G["combine_q81.out"], rtol=1e-5, atol=1e-6, what="merge")
    c = C["sigmoid_gate"]
    o = dev(cases.q_case(10, c["S"], c["nH"], c["hd"]))
    ops.sigmoid_gate(o, dev(cases.q_case(11, c["S"], c["nH"], 2 * c["hd"]) * 4), c["S"], c["nH"], c["hd"])
    assert_close(host(o), G["sigmoid_gate.out"], rtol=1e-5, atol=1e-6, what="gate")


A8 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_golden_a8.npz")


@pytest.mark.parametrize("idx,name", [(i, n) for i, n in enumerate(cases.A8_CASES)])
def test_prefill_f16_equals_reference_materialised_path(idx, name):
    """tc_attn_prefill_f16 (flash, tcgen05) against what the reference's materialised prefill --
    its conversion and softmax kernels around the cuBLAS products -- produced on a B200 for the
    same seeded rows; tolerance of the fp16 prefill (2e-2 relative)."""
    g = np.load(A8)
    c = cases.A8_CASES[name]
    q, k, v = cases.a8_case(40 + idx, c)
    S, nH, nKV, hd = c["S"], c["nH"], c["nKV"], c["hd"]
    n = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 1024
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_f16(dev(q), dev(k), dev(v), out, buf[off:off + n], S, nH, nKV, hd)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out)[cases.a8_rows(S)], g[f"{name}.out_rows"], rtol=2e-2, atol=2e-3, what=name)
