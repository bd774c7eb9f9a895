"""Seeded inputs of the golden cases recorded from the reference's own CUDA kernels.

Used by tests/golden/make_ref_gpu_golden.py (which runs the reference kernels on a
GPU and stores their OUTPUTS in ref_gpu_golden.npz) and by
tests/test_oracle_ref_gpu_golden.py (which regenerates the same inputs and checks
the CPU restatement, and the library's kernels, against the stored outputs)."""
import math

import numpy as np

SEED = 0x7C0DE100


def _rng(case):
    return np.random.Generator(np.random.Philox(key=[SEED, case]))


def quant_case(case, tokens, nKV, hd):
    r = _rng(case)
    k = r.standard_normal((tokens, nKV, hd), dtype=np.float32)
    v = r.standard_normal((tokens, nKV, hd), dtype=np.float32) * 3.0
    k[0] = 0.0                                  # amax == 0 -> scale 1
    v[1] = 0.0
    k[2, :, 0] = 1e-30
    v[3, 0, :] = np.float32(127.5)
    k[3, 0, ::2] = 0.5
    k[3, 0, 1::2] = np.float32(63.5)            # x / s lands on .5: round half to even
    return k, v


def store_case(case, ctx, nKV, hd):
    r = _rng(case)
    return (r.standard_normal((ctx, nKV, hd), dtype=np.float32),
            r.standard_normal((ctx, nKV, hd), dtype=np.float32))


def q_case(case, rows, nH, hd):
    return _rng(case + 1000).standard_normal((rows, nH, hd), dtype=np.float32)


def partials_case(case, nH, chunks, hd):
    r = _rng(case)
    acc = r.standard_normal((1, nH, chunks, hd), dtype=np.float32) * 4
    m = r.standard_normal((1, nH, chunks), dtype=np.float32) * 3
    l = r.uniform(0.5, 30.0, (1, nH, chunks)).astype(np.float32)
    dead = r.uniform(size=l.shape) < 0.25
    dead[..., 0] = False
    l[dead] = 0.0
    m[dead] = -1e30
    return acc, m, l


# name -> parameters; kept small so the fixture stays a few hundred KB
CASES = {
    "quant_hd128": dict(tokens=48, nKV=4, hd=128),
    "quant_hd256": dict(tokens=16, nKV=2, hd=256),
    "decode_i8": dict(nH=8, nKV=2, hd=256, ctx=700, chunks=22, chunk=32),
    "prefill_i8": dict(nH=4, nKV=2, hd=256, S=5, cachePos=40),
    "decode_f32_c1": dict(nH=14, nKV=2, hd=64, ctx=2048, chunks=64, chunk=32),      # the f32 benchmark shape
    "decode_f32_7b": dict(nH=28, nKV=4, hd=128, ctx=1000, chunks=32, chunk=32),
    "attention_f32": dict(nH=14, nKV=2, hd=64, S=6, cachePos=50),
    "rope_store": dict(nH=14, nKV=2, hd=64, S=3, cachePos=7, theta=1e6, rows=16),
    "combine_q81": dict(nH=28, chunks=20, hd=128),
    "sigmoid_gate": dict(S=2, nH=4, hd=256),
    "softmax_causal": dict(S=8, nH=2, scale=1.0 / math.sqrt(128.0)),
}

# recorded later into ref_gpu_golden_f2.npz (the step in front of attention in the gated models)
CASES_F2 = {
    "qk_norm_rope_256": dict(S=3, nH=4, nKV=2, hd=256, nDims=64, pos=5, rows=16, theta=1e7),
    "qk_norm_rope_128": dict(S=2, nH=6, nKV=3, hd=128, nDims=128, pos=0, rows=8, theta=1e6),
    "qk_norm_rope_64": dict(S=4, nH=2, nKV=1, hd=64, nDims=32, pos=9, rows=16, theta=1e4),
}


def norm_rope_case(case, c):
    r = _rng(case)
    qg = r.standard_normal((c["S"], c["nH"], 2 * c["hd"]), dtype=np.float32) * 2
    k = r.standard_normal((c["S"], c["nKV"], c["hd"]), dtype=np.float32) * 0.5
    wq = (1 + 0.1 * r.standard_normal(c["hd"])).astype(np.float32)
    wk = (1 + 0.1 * r.standard_normal(c["hd"])).astype(np.float32)
    return qg, k, wq, wk


# recorded into ref_gpu_golden_a8.npz: the reference's whole materialised prefill (kF32ToF16,
# cuBLAS score and P.V products, kAttnSoftmaxCausal) -- the stored outputs are a sample of rows
A8_CASES = {
    "prefill_f16_s200": dict(nH=4, nKV=2, hd=128, S=200),
    "prefill_f16_s512": dict(nH=7, nKV=1, hd=128, S=512),      # the reference's row cap, one full GQA group
    "prefill_f16_hd64": dict(nH=4, nKV=2, hd=64, S=96),
}


def a8_rows(S):
    """Rows whose outputs are stored: every 16th, the tile edges, the last 8."""
    rows = set(range(0, S, 16)) | {1, 63, 64, 65, 127, 128, 129, 255, 256, 257} | set(range(S - 8, S))
    return np.array(sorted(r for r in rows if r < S), np.uint32)


def a8_case(case, c):
    r = _rng(case)
    return (r.standard_normal((c["S"], c["nH"], c["hd"]), dtype=np.float32),
            r.standard_normal((c["S"], c["nKV"], c["hd"]), dtype=np.float32),
            r.standard_normal((c["S"], c["nKV"], c["hd"]), dtype=np.float32))
