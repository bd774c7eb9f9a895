"""Records the outputs of the reference project's OWN CUDA kernels on seeded inputs.

Needs a GPU and oracle/_ref/libtc_ref_gpu.so (built by `make -C oracle refgpu` where
the reference checkout is mounted; the built library travels with the tree):

    python tests/golden/make_ref_gpu_golden.py [out.npz]
    python tests/golden/make_ref_gpu_golden.py f2 [out_f2.npz]      (ref_gpu_golden_f2.npz)
    python tests/golden/make_ref_gpu_golden.py a8 [out_a8.npz]      (ref_gpu_golden_a8.npz)

The result is committed as tests/golden/ref_gpu_golden.npz; inputs are regenerated
from seeds (tests/golden/ref_gpu_cases.py), only outputs are stored."""
import ctypes as C
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from tests.golden import ref_gpu_cases as cases  # noqa: E402

lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libtc_ref_gpu.so"))


_KEEP = []  # device copies must outlive the launches that read them


def d(a):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _KEEP.append(t)
    return t


def p(t):
    return C.c_void_p(t.data_ptr())


def call(fn, *args):
    rc = fn(*args)
    if rc != 0:
        raise RuntimeError(f"{fn.__name__} returned CUDA error {rc}")


def main(out_path):
    G = {}
    u32, f32 = C.c_uint32, C.c_float

    for name in ("quant_hd128", "quant_hd256"):
        c = cases.CASES[name]
        k, v = cases.quant_case(1 if name.endswith("128") else 2, c["tokens"], c["nKV"], c["hd"])
        k8 = torch.zeros((c["tokens"], c["nKV"], c["hd"]), dtype=torch.int8, device="cuda")
        v8 = torch.zeros_like(k8)
        ks = torch.zeros((c["tokens"], c["nKV"]), device="cuda")
        vs = torch.zeros_like(ks)
        call(lib.ref_gpu_quant_kv8, p(d(k)), p(d(v)), p(k8), p(v8), p(ks), p(vs), u32(c["tokens"]), u32(c["nKV"]),
             u32(c["hd"]), u32(0), u32(0))
        for key, t in (("k8", k8), ("v8", v8), ("ks", ks), ("vs", vs)):
            G[f"{name}.{key}"] = t.cpu().numpy()

    c = cases.CASES["decode_i8"]
    k, v = cases.store_case(3, c["ctx"], c["nKV"], c["hd"])
    q = cases.q_case(3, 1, c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])     # store built by the (pinned) quantiser
    inv = 1.0 / math.sqrt(c["hd"])
    dk8, dv8, dks, dvs, dq = d(k8), d(v8), d(ks), d(vs), d(q)
    out = torch.zeros((1, c["nH"], c["hd"]), device="cuda")
    pa = torch.zeros((c["nH"], c["chunks"], c["hd"]), device="cuda")
    pm = torch.zeros((c["nH"], c["chunks"]), device="cuda")
    pl = torch.zeros_like(pm)
    call(lib.ref_gpu_decode_i8_split, p(dq), p(dk8), p(dv8), p(dks), p(dvs), p(pa), p(pm), p(pl), p(out),
         u32(c["nH"]), u32(c["nKV"]), u32(c["ctx"] - 1), u32(c["chunks"]), u32(c["chunk"]), f32(inv))
    G["decode_i8.split_out"] = out.cpu().numpy()
    G["decode_i8.partM"] = pm.cpu().numpy()
    G["decode_i8.partL"] = pl.cpu().numpy()
    out2 = torch.zeros_like(out)
    call(lib.ref_gpu_decode_i8_eager, p(dq), p(dk8), p(dv8), p(dks), p(dvs), p(out2), u32(c["nH"]), u32(c["nKV"]),
         u32(c["ctx"] - 1), f32(inv))
    G["decode_i8.eager_out"] = out2.cpu().numpy()

    c = cases.CASES["prefill_i8"]
    rows = c["cachePos"] + c["S"]
    k, v = cases.store_case(4, rows, c["nKV"], c["hd"])
    q = cases.q_case(4, c["S"], c["nH"], c["hd"])
    k8, v8, ks, vs = oracle.quant_kv8(k, v, c["nKV"], c["hd"])
    out = torch.zeros((c["S"], c["nH"], c["hd"]), device="cuda")
    call(lib.ref_gpu_prefill_i8, p(d(q)), p(d(k8)), p(d(v8)), p(d(ks)), p(d(vs)), p(out), u32(c["S"]), u32(c["nH"]),
         u32(c["nKV"]), u32(c["cachePos"]), f32(1.0 / math.sqrt(c["hd"])))
    G["prefill_i8.out"] = out.cpu().numpy()

    for case_id, name in ((5, "decode_f32_c1"), (6, "decode_f32_7b")):
        c = cases.CASES[name]
        k, v = cases.store_case(case_id, c["ctx"], c["nKV"], c["hd"])
        q = cases.q_case(case_id, 1, c["nH"], c["hd"])
        out = torch.zeros((1, c["nH"], c["hd"]), device="cuda")
        pa = torch.zeros((c["nH"], c["chunks"], c["hd"]), device="cuda")
        pm = torch.zeros((c["nH"], c["chunks"]), device="cuda")
        pl = torch.zeros_like(pm)
        q81 = torch.zeros(c["nH"] * (c["hd"] // 32) * 40, dtype=torch.uint8, device="cuda")
        call(lib.ref_gpu_decode_f32, p(d(q)), p(d(k)), p(d(v)), p(out), p(pa), p(pm), p(pl), u32(c["nH"]),
             u32(c["nKV"]), u32(c["hd"]), u32(c["ctx"] - 1), u32(c["chunks"]), u32(c["chunk"]),
             f32(1.0 / math.sqrt(c["hd"])), p(q81))
        G[f"{name}.out"] = out.cpu().numpy()
        G[f"{name}.q81"] = q81.cpu().numpy()

    c = cases.CASES["attention_f32"]
    rows = c["cachePos"] + c["S"]
    k, v = cases.store_case(7, rows, c["nKV"], c["hd"])
    q = cases.q_case(7, c["S"], c["nH"], c["hd"])
    out = torch.zeros((c["S"], c["nH"], c["hd"]), device="cuda")
    call(lib.ref_gpu_attention_f32, p(d(q)), p(d(k)), p(d(v)), p(out), u32(c["S"]), u32(c["nH"]), u32(c["nKV"]),
         u32(c["hd"]), u32(c["cachePos"]), f32(1.0 / math.sqrt(c["hd"])))
    G["attention_f32.out"] = out.cpu().numpy()

    c = cases.CASES["rope_store"]
    cosT, sinT = oracle.rope_tables(c["rows"], c["hd"], c["theta"])
    kS, vS = cases.store_case(8, c["S"], c["nKV"], c["hd"])
    q = cases.q_case(8, c["S"], c["nH"], c["hd"])
    dq = d(q)
    kD = torch.zeros((c["rows"], c["nKV"], c["hd"]), device="cuda")
    vD = torch.zeros_like(kD)
    call(lib.ref_gpu_rope_store, p(dq), p(d(kS)), p(d(vS)), p(kD), p(vD), u32(c["S"]), u32(c["nH"]), u32(c["nKV"]),
         u32(c["hd"]), u32(c["cachePos"]), u32(c["cachePos"]), p(d(cosT)), p(d(sinT)))
    G["rope_store.q"] = dq.cpu().numpy()
    G["rope_store.k"] = kD.cpu().numpy()
    G["rope_store.v"] = vD.cpu().numpy()

    c = cases.CASES["combine_q81"]
    acc, m, l = cases.partials_case(9, c["nH"], c["chunks"], c["hd"])
    out = torch.zeros((1, c["nH"], c["hd"]), device="cuda")
    q81 = torch.zeros(c["nH"] * (c["hd"] // 32) * 40, dtype=torch.uint8, device="cuda")
    call(lib.ref_gpu_combine_w8_q81, p(d(acc)), p(d(m)), p(d(l)), p(out), u32(c["nH"]), u32(c["chunks"]), p(q81))
    G["combine_q81.out"] = out.cpu().numpy()
    G["combine_q81.q81"] = q81.cpu().numpy()

    c = cases.CASES["sigmoid_gate"]
    o = cases.q_case(10, c["S"], c["nH"], c["hd"])
    gq = cases.q_case(11, c["S"], c["nH"], 2 * c["hd"]) * 4
    do = d(o)
    call(lib.ref_gpu_sigmoid_gate, p(do), p(d(gq)), u32(c["S"]), u32(c["nH"]), u32(c["hd"]))
    G["sigmoid_gate.out"] = do.cpu().numpy()

    c = cases.CASES["softmax_causal"]
    sc = cases.q_case(12, c["nH"], c["S"], c["S"]) * 20      # [head][row][key] raw scores
    pout = torch.zeros((c["nH"], c["S"], c["S"]), dtype=torch.float16, device="cuda")
    call(lib.ref_gpu_softmax_causal, p(d(sc)), p(pout), u32(c["S"]), u32(c["nH"]), f32(c["scale"]))
    G["softmax_causal.p"] = pout.cpu().numpy()

    np.savez_compressed(out_path, **G)
    print(f"wrote {len(G)} arrays, {os.path.getsize(out_path)} bytes -> {out_path}")


def main_f2(out_path):
    """kQ35QNormRoPE + kQ35KNormRoPE -> ref_gpu_golden_f2.npz (python ... f2 [out.npz])."""
    G = {}
    u32 = C.c_uint32
    for i, (name, c) in enumerate(cases.CASES_F2.items()):
        qg, k, wq, wk = cases.norm_rope_case(20 + i, c)
        cosT, sinT = oracle.mrope_tables(c["rows"], c["nDims"], c["theta"])
        qOut = torch.zeros((c["S"], c["nH"], c["hd"]), device="cuda")
        dk = d(k)
        call(lib.ref_gpu_qk_norm_rope, p(d(qg)), p(qOut), p(dk), p(d(wq)), p(d(wk)), u32(c["hd"]), u32(c["nDims"]),
             u32(c["nH"]), u32(c["nKV"]), u32(c["S"]), u32(c["pos"]), p(d(cosT)), p(d(sinT)))
        G[f"{name}.q"] = qOut.cpu().numpy()
        G[f"{name}.k"] = dk.cpu().numpy()
    np.savez_compressed(out_path, **G)
    print(f"wrote {len(G)} arrays, {os.path.getsize(out_path)} bytes -> {out_path}")


def main_a8(out_path):
    """The reference's materialised fp16 prefill, cuBLAS products included -> ref_gpu_golden_a8.npz."""
    G = {}
    u32, f32 = C.c_uint32, C.c_float
    for i, (name, c) in enumerate(cases.A8_CASES.items()):
        q, k, v = cases.a8_case(40 + i, c)
        out = torch.zeros((c["S"], c["nH"], c["hd"]), device="cuda")
        call(lib.ref_gpu_prefill_f16_gemm, p(d(q)), p(d(k)), p(d(v)), p(out), u32(c["S"]), u32(c["nH"]), u32(c["nKV"]),
             u32(c["hd"]), f32(1.0 / math.sqrt(c["hd"])))
        G[f"{name}.out_rows"] = out.cpu().numpy()[cases.a8_rows(c["S"])]
    np.savez_compressed(out_path, **G)
    print(f"wrote {len(G)} arrays, {os.path.getsize(out_path)} bytes -> {out_path}")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "a8":
        main_a8(sys.argv[2] if len(sys.argv) > 2 else os.path.join(HERE, "ref_gpu_golden_a8.npz"))
    elif len(sys.argv) > 1 and sys.argv[1] == "f2":
        main_f2(sys.argv[2] if len(sys.argv) > 2 else os.path.join(HERE, "ref_gpu_golden_f2.npz"))
    else:
        main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_gpu_golden.npz"))
