/*
 * tc_oracle.c -- CPU restatement of the reference engine's attention / KV-cache
 * arithmetic.  TEST INFRASTRUCTURE ONLY: this file is the checker that the CUDA
 * path is compared against.  Nothing that ships (the package, the C-ABI library)
 * may link, import or call it; only tests/, the smoke check and the bench's
 * cpu_baseline / reference arm do.
 *
 * Every function names the reference source (path inside the reference project
 * and line range) whose arithmetic it follows.  The reference kernels are CUDA
 * "one warp per (token, q-head)" kernels; where summation order matters the
 * warp is emulated lane by lane (lane owns elements lane + 32*i; the dot product
 * is folded with the shfl_down 16,8,4,2,1 tree of kWarpReduceSum,
 * include/gpu/GpuAttentionKernels.hpp:39-44).
 *
 * Pinning status:
 *   - context planner: PINNED against the reference's own known answers
 *     (unit_tests/ContextPlanTest.cpp) and against the reference's compiled
 *     ContextPlan.cpp (oracle/_ref/libtc_ref.so, tests/golden/planner_golden.json).
 *   - int8 quantiser, int8 / f32 decode and causal attention, merge, Q8_1 fold,
 *     RoPE / append, sigmoid gate, causal softmax rows: PINNED against outputs of the
 *     reference's OWN CUDA kernels run on a B200 (oracle/ref_gpu_shim.cu ->
 *     tests/golden/ref_gpu_golden.npz; tests/test_oracle_ref_gpu_golden.py):
 *     bit-exact for bytes / integers / rotated values, a few ulp for softmax outputs
 *     (device exp2f versus libm).  The reference has no checkpoint-free test of its
 *     own for these, so the recorded kernel outputs are the anchor.
 *   - the QK^T / PV products of the materialised fp16 prefill live in cuBLAS (not
 *     part of the reference): orc_prefill_f16 states the contract (fp16 products,
 *     f32 accumulation, fp16 probabilities) and is unpinned at kernel level.
 *
 * Build: see oracle/Makefile (gcc -O2 -mfma -ffp-contract=off; contraction is
 * switched off so that every fused multiply-add below is an explicit fmaf, as in
 * the CUDA source).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>

#define ORC_LOG2E 1.4426950408889634f /* include/gpu/GpuCommon.hpp:77 */

/* ------------------------------------------------------------------------- */
/* helpers                                                                    */
/* ------------------------------------------------------------------------- */

/* kWarpReduceSum (include/gpu/GpuAttentionKernels.hpp:39-44): lane 0's value
 * after v += shfl_down(v, off) for off = 16..1.  Only lane 0 is broadcast, so
 * only the lanes that feed lane 0 need to be right: at each level lanes
 * [0, off) add lanes [off, 2*off). */
static float warp_reduce_sum(float v[32]) {
    for (int off = 16; off; off >>= 1)
        for (int l = 0; l < off; ++l) v[l] += v[l + off];
    return v[0];
}

static float half_round(float x) { /* f32 -> fp16 -> f32, round to nearest even */
    _Float16 h = (_Float16) x;
    return (float) h;
}

/* ------------------------------------------------------------------------- */
/* int8 KV quantiser                                                          */
/* ------------------------------------------------------------------------- */

/* kQ35QuantKV8 (include/gpu/GpuQwen35Kernels.hpp:586-637).
 * k, v: f32 [srcTokenBase + t][nKV][hd]; k8, v8: int8 [dstTokenBase + t][nKV][hd];
 * ks, vs: f32 [dstTokenBase + t][nKV].  scale = amax/127 (1.0 when amax == 0),
 * q = clamp(lrintf(x / scale), -128, 127): IEEE division, round-half-even. */
void orc_quant_kv8(const float *k, const float *v, int8_t *k8, int8_t *v8,
                   float *ks, float *vs, uint32_t tokens, uint32_t nKV,
                   uint32_t hd, uint64_t dstTokenBase, uint64_t srcTokenBase) {
    for (uint32_t t = 0; t < tokens; ++t) {
        for (uint32_t h = 0; h < nKV; ++h) {
            const uint64_t base = ((srcTokenBase + t) * nKV + h) * (uint64_t) hd;
            const uint64_t dbase = (dstTokenBase + t) * nKV + h;
            float mk = 0.0f, mv = 0.0f;
            for (uint32_t i = 0; i < hd; ++i) {
                mk = fmaxf(mk, fabsf(k[base + i]));
                mv = fmaxf(mv, fabsf(v[base + i]));
            }
            const float sk = mk > 0.0f ? mk / 127.0f : 1.0f;
            const float sv = mv > 0.0f ? mv / 127.0f : 1.0f;
            ks[dbase] = sk;
            vs[dbase] = sv;
            const uint64_t ob = dbase * (uint64_t) hd;
            for (uint32_t i = 0; i < hd; ++i) {
                long qk = lrintf(k[base + i] / sk);
                long qv = lrintf(v[base + i] / sv);
                k8[ob + i] = (int8_t) (qk < -128 ? -128 : (qk > 127 ? 127 : qk));
                v8[ob + i] = (int8_t) (qv < -128 ? -128 : (qv > 127 ? 127 : qv));
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* warp-emulated online softmax over a row range                              */
/* ------------------------------------------------------------------------- */

typedef struct {
    float m, l;
    float acc[32][8]; /* [lane][i], element index lane + 32*i; hd <= 256 */
} warp_state;

static void ws_init(warp_state *w) {
    w->m = -1e30f;
    w->l = 0.0f;
    memset(w->acc, 0, sizeof(w->acc));
}

/* One cache row folded into (m, l, acc): the loop body shared by
 * kQ35WarpAttention8Split (GpuQwen35Kernels.hpp:544-573), kQ35WarpAttention8
 * (:661-687), kQ35WarpAttention8Prefill (:2409-2430) for int8 rows, and by
 * kWarpAttention / kWarpAttentionSplit (GpuAttentionKernels.hpp:236-265,
 * 698-724) for f32 / fp16 rows.  kd / vd hold the row already converted to
 * float exactly as the kernel does it (float(k8)*sk, __half2float, or the f32
 * value itself). */
static void ws_fold_row(warp_state *w, const float *q, const float *kd,
                        const float *vd, uint32_t nv, float invSqrt) {
    float part[32];
    for (int lane = 0; lane < 32; ++lane) {
        float sc = 0.0f;
        for (uint32_t i = 0; i < nv; ++i)
            sc = fmaf(q[lane + 32 * i], kd[lane + 32 * i], sc);
        part[lane] = sc;
    }
    const float sc = warp_reduce_sum(part) * invSqrt;
    if (sc > w->m) {
        const float alpha = exp2f((w->m - sc) * ORC_LOG2E);
        for (int lane = 0; lane < 32; ++lane)
            for (uint32_t i = 0; i < nv; ++i) w->acc[lane][i] *= alpha;
        w->l *= alpha;
        w->m = sc;
    }
    const float p = exp2f((sc - w->m) * ORC_LOG2E);
    w->l += p;
    for (int lane = 0; lane < 32; ++lane)
        for (uint32_t i = 0; i < nv; ++i)
            w->acc[lane][i] = fmaf(p, vd[lane + 32 * i], w->acc[lane][i]);
}

static void dequant_row(const int8_t *r, float s, uint32_t hd, float *out) {
    /* static_cast<float>(k8) * sk, one rounding (GpuQwen35Kernels.hpp:555). */
    for (uint32_t i = 0; i < hd; ++i) out[i] = (float) r[i] * s;
}

/* ------------------------------------------------------------------------- */
/* int8 decode: split partials, eager, and the partial merge                  */
/* ------------------------------------------------------------------------- */

/* kQ35WarpAttention8Split (include/gpu/GpuQwen35Kernels.hpp:519-581) with the
 * lane count generalised from 256/32 to hd/32.  One sequence; attends rows
 * [0, cachePos].  partAcc [nHeads][numChunks][hd], partM/partL [nHeads][numChunks]. */
void orc_decode_i8_split(const float *q, const int8_t *k8, const int8_t *v8,
                         const float *ks, const float *vs, float *partAcc,
                         float *partM, float *partL, uint32_t nHeads,
                         uint32_t nKV, uint32_t cachePos, uint32_t numChunks,
                         uint32_t chunkSize, uint32_t hd, float invSqrt) {
    const uint32_t nv = hd / 32;
    float kd[256], vd[256];
    for (uint32_t qHead = 0; qHead < nHeads; ++qHead) {
        const uint32_t kvHead = qHead / (nHeads / nKV);
        for (uint32_t chunk = 0; chunk < numChunks; ++chunk) {
            warp_state w;
            ws_init(&w);
            const uint64_t lo = (uint64_t) chunk * chunkSize;
            if (lo <= cachePos) {
                uint64_t hi = lo + chunkSize - 1;
                if (hi > cachePos) hi = cachePos;
                for (uint64_t cs = lo; cs <= hi; ++cs) {
                    const uint64_t row = cs * nKV + kvHead;
                    dequant_row(k8 + row * hd, ks[row], hd, kd);
                    dequant_row(v8 + row * hd, vs[row], hd, vd);
                    ws_fold_row(&w, q + (uint64_t) qHead * hd, kd, vd, nv, invSqrt);
                }
            }
            const uint64_t pidx = (uint64_t) qHead * numChunks + chunk;
            for (int lane = 0; lane < 32; ++lane)
                for (uint32_t i = 0; i < nv; ++i)
                    partAcc[pidx * hd + lane + 32 * i] = w.acc[lane][i];
            partM[pidx] = w.m;
            partL[pidx] = w.l;
        }
    }
}

/* Causal attention over an int8 store for `seqLen` query rows:
 * kQ35WarpAttention8 (GpuQwen35Kernels.hpp:641-692) when seqLen == 1 and
 * kQ35WarpAttention8Prefill (:2380-2435) otherwise -- both serial over
 * cs in [0, cachePos + s], output acc * (1/l).  q, out: [seqLen][nHeads][hd]. */
void orc_attention_i8(const float *q, const int8_t *k8, const int8_t *v8,
                      const float *ks, const float *vs, float *out,
                      uint32_t seqLen, uint32_t nHeads, uint32_t nKV,
                      uint32_t cachePos, uint32_t hd, float invSqrt) {
    const uint32_t nv = hd / 32;
    float kd[256], vd[256];
    for (uint32_t s = 0; s < seqLen; ++s) {
        for (uint32_t qHead = 0; qHead < nHeads; ++qHead) {
            const uint32_t kvHead = qHead / (nHeads / nKV);
            const float *qp = q + ((uint64_t) s * nHeads + qHead) * hd;
            warp_state w;
            ws_init(&w);
            for (uint64_t cs = 0; cs <= (uint64_t) cachePos + s; ++cs) {
                const uint64_t row = cs * nKV + kvHead;
                dequant_row(k8 + row * hd, ks[row], hd, kd);
                dequant_row(v8 + row * hd, vs[row], hd, vd);
                ws_fold_row(&w, qp, kd, vd, nv, invSqrt);
            }
            const float invL = 1.0f / w.l;
            float *op = out + ((uint64_t) s * nHeads + qHead) * hd;
            for (int lane = 0; lane < 32; ++lane)
                for (uint32_t i = 0; i < nv; ++i)
                    op[lane + 32 * i] = w.acc[lane][i] * invL;
        }
    }
}

/* kAttnCombinePartial (include/gpu/GpuAttentionKernels.hpp:909-946).
 * partAcc [seqLen][nHeads][numChunks][hd]; chunks with l <= 0 are skipped. */
void orc_combine_partials(const float *partAcc, const float *partM,
                          const float *partL, float *out, uint32_t seqLen,
                          uint32_t nHeads, uint32_t numChunks, uint32_t hd) {
    for (uint32_t s = 0; s < seqLen; ++s) {
        for (uint32_t qHead = 0; qHead < nHeads; ++qHead) {
            const uint64_t base = ((uint64_t) s * nHeads + qHead) * numChunks;
            float M = -1e30f;
            for (uint32_t c = 0; c < numChunks; ++c) M = fmaxf(M, partM[base + c]);
            float *op = out + ((uint64_t) s * nHeads + qHead) * hd;
            float acc[256];
            for (uint32_t d = 0; d < hd; ++d) acc[d] = 0.0f;
            float lsum = 0.0f;
            for (uint32_t c = 0; c < numChunks; ++c) {
                if (partL[base + c] <= 0.0f) continue;
                const float w = exp2f((partM[base + c] - M) * ORC_LOG2E);
                lsum += w * partL[base + c];
                const float *pac = partAcc + (base + c) * hd;
                for (uint32_t d = 0; d < hd; ++d) acc[d] = fmaf(w, pac[d], acc[d]);
            }
            const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
            for (uint32_t d = 0; d < hd; ++d) op[d] = acc[d] * inv;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* f32 / fp16 KV: split partials and the unsplit causal kernel                */
/* ------------------------------------------------------------------------- */

static void load_row_kvt(const void *cache, uint64_t row, uint32_t hd, int kvHalf,
                         float *out) {
    /* kvLoad (include/gpu/GpuElementwiseKernels.hpp:69-74): f32 verbatim or
     * __half2float. */
    if (kvHalf) {
        const _Float16 *p = (const _Float16 *) cache + row * hd;
        for (uint32_t i = 0; i < hd; ++i) out[i] = (float) p[i];
    } else {
        memcpy(out, (const float *) cache + row * hd, hd * sizeof(float));
    }
}

/* kWarpAttentionSplit<HD, KVT, 1> (include/gpu/GpuAttentionKernels.hpp:625-766;
 * the WSUB == 1 layout -- sub-warps only regroup the same online softmax and
 * stay inside the f32 tolerance).  q [seqLen][nHeads][hd]; attends rows
 * [0, cachePos + s]. */
void orc_decode_kv_split(const float *q, const void *kCache, const void *vCache,
                         int kvHalf, float *partAcc, float *partM, float *partL,
                         uint32_t seqLen, uint32_t nHeads, uint32_t nKV,
                         uint32_t cachePos, uint32_t numChunks,
                         uint32_t chunkSize, uint32_t hd, float invSqrt) {
    const uint32_t nv = hd / 32;
    float kd[256], vd[256];
    for (uint32_t s = 0; s < seqLen; ++s)
        for (uint32_t qHead = 0; qHead < nHeads; ++qHead) {
            const uint32_t kvHead = qHead / (nHeads / nKV);
            const uint64_t csEnd = (uint64_t) cachePos + s;
            for (uint32_t chunk = 0; chunk < numChunks; ++chunk) {
                warp_state w;
                ws_init(&w);
                const uint64_t lo = (uint64_t) chunk * chunkSize;
                if (lo <= csEnd) {
                    uint64_t hi = lo + chunkSize - 1;
                    if (hi > csEnd) hi = csEnd;
                    for (uint64_t cs = lo; cs <= hi; ++cs) {
                        const uint64_t row = cs * nKV + kvHead;
                        load_row_kvt(kCache, row, hd, kvHalf, kd);
                        load_row_kvt(vCache, row, hd, kvHalf, vd);
                        ws_fold_row(&w, q + ((uint64_t) s * nHeads + qHead) * hd,
                                    kd, vd, nv, invSqrt);
                    }
                }
                const uint64_t pidx =
                        ((uint64_t) s * nHeads + qHead) * numChunks + chunk;
                for (int lane = 0; lane < 32; ++lane)
                    for (uint32_t i = 0; i < nv; ++i)
                        partAcc[pidx * hd + lane + 32 * i] = w.acc[lane][i];
                partM[pidx] = w.m;
                partL[pidx] = w.l;
            }
        }
}

/* kWarpAttention<HD, KVT> (include/gpu/GpuAttentionKernels.hpp:211-272): the
 * unsplit causal kernel (eager decode, and prefill beyond the cuBLAS window). */
void orc_attention_kv(const float *q, const void *kCache, const void *vCache,
                      int kvHalf, float *out, uint32_t seqLen, uint32_t nHeads,
                      uint32_t nKV, uint32_t cachePos, uint32_t hd,
                      float invSqrt) {
    const uint32_t nv = hd / 32;
    float kd[256], vd[256];
    for (uint32_t s = 0; s < seqLen; ++s)
        for (uint32_t qHead = 0; qHead < nHeads; ++qHead) {
            const uint32_t kvHead = qHead / (nHeads / nKV);
            const float *qp = q + ((uint64_t) s * nHeads + qHead) * hd;
            warp_state w;
            ws_init(&w);
            for (uint64_t cs = 0; cs <= (uint64_t) cachePos + s; ++cs) {
                const uint64_t row = cs * nKV + kvHead;
                load_row_kvt(kCache, row, hd, kvHalf, kd);
                load_row_kvt(vCache, row, hd, kvHalf, vd);
                ws_fold_row(&w, qp, kd, vd, nv, invSqrt);
            }
            const float invL = 1.0f / w.l;
            float *op = out + ((uint64_t) s * nHeads + qHead) * hd;
            for (int lane = 0; lane < 32; ++lane)
                for (uint32_t i = 0; i < nv; ++i)
                    op[lane + 32 * i] = w.acc[lane][i] * invL;
        }
}

/* ------------------------------------------------------------------------- */
/* CPU engine path: Model::attentionFused                                     */
/* ------------------------------------------------------------------------- */

/* dotProductFMA_AVX512 (src/cpp/core/SIMDMatMulVecAVX512.cpp:61-75): 16 lanes of
 * fused multiply-add over j, then _mm512_reduce_add_ps (pairwise halves
 * 8+8, 4+4, 2+2, 1+1), then a scalar tail. */
static float dot_fma16(const float *a, const float *b, uint32_t n) {
    float s[16];
    for (int i = 0; i < 16; ++i) s[i] = 0.0f;
    uint32_t j = 0;
    for (; j + 16 <= n; j += 16)
        for (int i = 0; i < 16; ++i) s[i] = fmaf(a[j + i], b[j + i], s[i]);
    for (int w = 8; w; w >>= 1)
        for (int i = 0; i < w; ++i) s[i] += s[i + w];
    float r = s[0];
    for (; j < n; ++j) r += a[j] * b[j];
    return r;
}

/* accumulateFMA_AVX512 (src/cpp/core/SIMDMatMulVecAVX512.cpp:46-59). */
static void axpy_fma(float *local, const float *x, float alpha, uint32_t n) {
    for (uint32_t j = 0; j < n; ++j) local[j] = fmaf(alpha, x[j], local[j]);
}

/* Model::attentionFused (src/cpp/core/ModelPrimitives.cpp:221-344) for the
 * (s, g) task range [task0, task1) of the seqLen x nKVHeads task grid (the
 * engine's parallelFor2D hands out exactly these tasks).  32-position blocks
 * with a block max, m starts at -inf, o rescaled as o += (alpha-1)*o. */
void orc_attention_fused_cpu_tasks(const float *q, const float *kCache,
                                   const float *vCache, float *output,
                                   uint32_t seqLen, uint32_t cachePos,
                                   uint32_t nHeads, uint32_t nKVHeads,
                                   uint32_t headDim, uint32_t task0,
                                   uint32_t task1) {
    const uint32_t nGroups = nHeads / nKVHeads;
    const float invSqrt = 1.0f / sqrtf((float) headDim);
    enum { BLOCK = 32 };
    (void) seqLen;
    for (uint32_t task = task0; task < task1; ++task) {
        const uint32_t s = task / nKVHeads, g = task % nKVHeads;
        const uint64_t csEnd = (uint64_t) cachePos + s;
        for (uint32_t h = 0; h < nGroups; ++h) {
            const uint32_t qHead = g * nGroups + h;
            const float *qPtr = q + ((uint64_t) s * nHeads + qHead) * headDim;
            float o[256];
            for (uint32_t d = 0; d < headDim; ++d) o[d] = 0.0f;
            float m = -INFINITY, l = 0.0f;
            uint64_t cs = 0;
            for (; cs + BLOCK <= csEnd + 1; cs += BLOCK) {
                float scores[BLOCK];
                for (uint32_t b = 0; b < BLOCK; ++b)
                    scores[b] = dot_fma16(qPtr,
                                          kCache + ((cs + b) * nKVHeads + g) * headDim,
                                          headDim) *
                                invSqrt;
                float blockMax = scores[0];
                for (uint32_t b = 1; b < BLOCK; ++b)
                    blockMax = scores[b] > blockMax ? scores[b] : blockMax;
                const float mNew = m > blockMax ? m : blockMax;
                const float alpha = exp2f((m - mNew) * ORC_LOG2E);
                if (alpha != 1.0f) axpy_fma(o, o, alpha - 1.0f, headDim);
                l *= alpha;
                for (uint32_t b = 0; b < BLOCK; ++b) {
                    const float p = exp2f((scores[b] - mNew) * ORC_LOG2E);
                    l += p;
                    axpy_fma(o, vCache + ((cs + b) * nKVHeads + g) * headDim, p,
                             headDim);
                }
                m = mNew;
            }
            for (; cs <= csEnd; ++cs) {
                const float score =
                        dot_fma16(qPtr, kCache + (cs * nKVHeads + g) * headDim,
                                  headDim) *
                        invSqrt;
                if (score > m) {
                    const float alpha = exp2f((m - score) * ORC_LOG2E);
                    if (alpha != 1.0f) axpy_fma(o, o, alpha - 1.0f, headDim);
                    l *= alpha;
                    m = score;
                }
                const float p = exp2f((score - m) * ORC_LOG2E);
                l += p;
                axpy_fma(o, vCache + (cs * nKVHeads + g) * headDim, p, headDim);
            }
            const float invL = 1.0f / l;
            float *outPtr = output + ((uint64_t) s * nHeads + qHead) * headDim;
            for (uint32_t d = 0; d < headDim; ++d) outPtr[d] = o[d] * invL;
        }
    }
}

void orc_attention_fused_cpu(const float *q, const float *kCache,
                             const float *vCache, float *output, uint32_t seqLen,
                             uint32_t cachePos, uint32_t nHeads,
                             uint32_t nKVHeads, uint32_t headDim) {
    orc_attention_fused_cpu_tasks(q, kCache, vCache, output, seqLen, cachePos,
                                  nHeads, nKVHeads, headDim, 0, seqLen * nKVHeads);
}

/* ------------------------------------------------------------------------- */
/* double-precision evaluation (bounds both implementations)                  */
/* ------------------------------------------------------------------------- */

/* Exact-softmax causal attention in double over dequantised / converted rows.
 * kind: 0 = f32 cache, 1 = fp16 cache, 2 = int8 store (k8/v8 + scales). */
void orc_attention_f64(const float *q, const void *kc, const void *vc,
                       const float *ks, const float *vs, int kind, double *out,
                       uint32_t seqLen, uint32_t nHeads, uint32_t nKV,
                       uint32_t cachePos, uint32_t hd, double scale) {
    const uint64_t maxRows = (uint64_t) cachePos + seqLen;
    double *sc = (double *) malloc(maxRows * sizeof(double));
    for (uint32_t s = 0; s < seqLen; ++s)
        for (uint32_t h = 0; h < nHeads; ++h) {
            const uint32_t g = h / (nHeads / nKV);
            const float *qp = q + ((uint64_t) s * nHeads + h) * hd;
            const uint64_t n = (uint64_t) cachePos + s + 1;
            double mx = -INFINITY;
            for (uint64_t cs = 0; cs < n; ++cs) {
                const uint64_t row = cs * nKV + g;
                double d = 0.0;
                for (uint32_t i = 0; i < hd; ++i) {
                    double kv;
                    if (kind == 2) kv = (double) ((float) ((const int8_t *) kc)[row * hd + i] * ks[row]);
                    else if (kind == 1) kv = (double) (float) ((const _Float16 *) kc)[row * hd + i];
                    else kv = (double) ((const float *) kc)[row * hd + i];
                    d += (double) qp[i] * kv;
                }
                sc[cs] = d * scale;
                if (sc[cs] > mx) mx = sc[cs];
            }
            double *op = out + ((uint64_t) s * nHeads + h) * hd;
            for (uint32_t i = 0; i < hd; ++i) op[i] = 0.0;
            double l = 0.0;
            for (uint64_t cs = 0; cs < n; ++cs) {
                const uint64_t row = cs * nKV + g;
                const double p = exp(sc[cs] - mx);
                l += p;
                for (uint32_t i = 0; i < hd; ++i) {
                    double vv;
                    if (kind == 2) vv = (double) ((float) ((const int8_t *) vc)[row * hd + i] * vs[row]);
                    else if (kind == 1) vv = (double) (float) ((const _Float16 *) vc)[row * hd + i];
                    else vv = (double) ((const float *) vc)[row * hd + i];
                    op[i] += p * vv;
                }
            }
            for (uint32_t i = 0; i < hd; ++i) op[i] /= l;
        }
    free(sc);
}

/* ------------------------------------------------------------------------- */
/* materialised fp16 prefill (cuBLAS detour of the dense path)                 */
/* ------------------------------------------------------------------------- */

/* The dense prefill of src/cpp/core/cuda/forward/GPUComputeForward.cu:3937-4026:
 * fp16 twins of q and of the stored K/V rows (kF32ToF16), scores = K_h . q in
 * f32 (fp16 products, f32 accumulate -- the order inside the library GEMM is
 * not defined, a plain ascending sum is used here), kAttnSoftmaxCausal
 * (include/gpu/GpuAttentionKernels.hpp:323-353: mx = max(score) * scale,
 * p = exp2f((score*scale - mx) * LOG2E) / sum, rounded to fp16, zero past the
 * causal limit), then out = P . V in f32.  q [S][nHeads][hd] f32,
 * k, v [S][nKV][hd] f32 (rows [0, S), cachePos == 0). */
/* One query row of one head: scores over K rows [0, lim], softmax, fp16 P, PV. */
static void prefill_f16_row(const float *qp, const float *k16, const float *v16, float *op,
                            uint32_t lim, uint32_t g, uint32_t nKV, uint32_t hd, float scale,
                            float *sc, float *p16) {
    float q16[256];
    for (uint32_t i = 0; i < hd; ++i) q16[i] = half_round(qp[i]);
    float mx = -1e30f;
    for (uint32_t c = 0; c <= lim; ++c) {
        const float *kp = k16 + ((uint64_t) c * nKV + g) * hd;
        float d = 0.0f;
        for (uint32_t i = 0; i < hd; ++i) d += q16[i] * kp[i];
        sc[c] = d;
        mx = fmaxf(mx, d);
    }
    mx *= scale;
    float sum = 0.0f;
    for (uint32_t c = 0; c <= lim; ++c)
        sum += exp2f((sc[c] * scale - mx) * ORC_LOG2E);
    const float inv = 1.0f / sum;
    for (uint32_t c = 0; c <= lim; ++c)
        p16[c] = half_round(exp2f((sc[c] * scale - mx) * ORC_LOG2E) * inv);
    for (uint32_t i = 0; i < hd; ++i) op[i] = 0.0f;
    for (uint32_t c = 0; c <= lim; ++c) {
        const float *vp = v16 + ((uint64_t) c * nKV + g) * hd;
        for (uint32_t i = 0; i < hd; ++i) op[i] += p16[c] * vp[i];
    }
}

/* The same contract for a SAMPLE of query rows and a cache that already holds
 * cachePos rows (query row s sits at position cachePos + s and sees K/V rows
 * [0, cachePos + s]; the reference takes this path only with cachePos == 0,
 * GPUComputeForward.cu:3828-3835 -- the rule itself is kAttnSoftmaxCausal's
 * `pos + row`).  q: [S][nHeads][hd]; k, v: [cachePos + S][nKV][hd]; rows[r] < S;
 * out: [nRows][nHeads][hd].  Lets a test check a long prompt without paying for
 * every row on the CPU. */
void orc_prefill_f16_rows(const float *q, const float *k, const float *v, float *out,
                          const uint32_t *rows, uint32_t nRows, uint32_t S, uint32_t cachePos,
                          uint32_t nHeads, uint32_t nKV, uint32_t hd, float scale) {
    const size_t total = (size_t) cachePos + S;
    float *sc = (float *) malloc(total * sizeof(float));
    float *p16 = (float *) malloc(total * sizeof(float));
    float *k16 = (float *) malloc(total * nKV * hd * sizeof(float));
    float *v16 = (float *) malloc(total * nKV * hd * sizeof(float));
    for (size_t i = 0; i < total * nKV * hd; ++i) {
        k16[i] = half_round(k[i]);
        v16[i] = half_round(v[i]);
    }
    for (uint32_t r = 0; r < nRows; ++r) {
        const uint32_t s = rows[r];
        for (uint32_t h = 0; h < nHeads; ++h)
            prefill_f16_row(q + ((uint64_t) s * nHeads + h) * hd, k16, v16,
                            out + ((uint64_t) r * nHeads + h) * hd, cachePos + s, h / (nHeads / nKV),
                            nKV, hd, scale, sc, p16);
    }
    free(sc);
    free(p16);
    free(k16);
    free(v16);
}

void orc_prefill_f16(const float *q, const float *k, const float *v, float *out,
                     uint32_t S, uint32_t nHeads, uint32_t nKV, uint32_t hd,
                     float scale) {
    uint32_t *rows = (uint32_t *) malloc((size_t) S * sizeof(uint32_t));
    for (uint32_t s = 0; s < S; ++s) rows[s] = s;
    orc_prefill_f16_rows(q, k, v, out, rows, S, S, 0, nHeads, nKV, hd, scale);
    free(rows);
}

/* ------------------------------------------------------------------------- */
/* RoPE tables, RoPE(Q), KV append                                            */
/* ------------------------------------------------------------------------- */

/* Model::ensureRoPETables (src/cpp/core/ModelPrimitives.cpp:112-127):
 * freq[j] = 1 / powf(theta, 2j / headDim); angle = float(p) * freq[j]. */
void orc_rope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t headDim,
                     float theta) {
    const uint32_t pairs = headDim / 2;
    for (uint32_t p = 0; p < rows; ++p)
        for (uint32_t j = 0; j < pairs; ++j) {
            const float freq = 1.0f / powf(theta, (float) (2 * j) / (float) headDim);
            const float angle = (float) p * freq;
            cosT[(uint64_t) p * pairs + j] = cosf(angle);
            sinT[(uint64_t) p * pairs + j] = sinf(angle);
        }
}

/* kRoPEQ (include/gpu/GpuElementwiseKernels.hpp:425-448): NEOX pairing
 * (j, j + hd/2), x0' = fmaf(x0, c, -x1*s), x1' = fmaf(x0, s, x1*c). */
void orc_rope_q(float *q, const float *cosT, const float *sinT, uint32_t seqLen,
                uint32_t qHeads, uint32_t headDim, uint32_t pos) {
    const uint32_t pairs = headDim / 2;
    for (uint32_t s = 0; s < seqLen; ++s) {
        const float *c = cosT + (uint64_t) (pos + s) * pairs;
        const float *sn = sinT + (uint64_t) (pos + s) * pairs;
        for (uint32_t h = 0; h < qHeads; ++h) {
            float *head = q + ((uint64_t) s * qHeads + h) * headDim;
            for (uint32_t j = 0; j < pairs; ++j) {
                const float x0 = head[j], x1 = head[j + pairs];
                head[j] = fmaf(x0, c[j], -x1 * sn[j]);
                head[j + pairs] = fmaf(x0, sn[j], x1 * c[j]);
            }
        }
    }
}

/* kStoreKVRope<KVT> (include/gpu/GpuElementwiseKernels.hpp:452-483) with
 * cos/sin given, kQ35StoreKV (include/gpu/GpuQwen35Kernels.hpp:497-516) with
 * cosT == NULL (K verbatim).  V is always stored verbatim.  Rows land at
 * cachePos + s; the rotation angle row is ropePos + s.  kvHalf stores fp16
 * (__float2half, round to nearest even). */
void orc_kv_append(const float *kSrc, const float *vSrc, void *kDst, void *vDst,
                   int kvHalf, uint32_t seqLen, uint32_t nKV, uint32_t headDim,
                   uint32_t cachePos, uint32_t ropePos, const float *cosT,
                   const float *sinT) {
    const uint32_t pairs = headDim / 2, kvSize = nKV * headDim;
    float *row = (float *) malloc(kvSize * sizeof(float));
    for (uint32_t s = 0; s < seqLen; ++s) {
        const float *ks = kSrc + (uint64_t) s * kvSize;
        const float *vs = vSrc + (uint64_t) s * kvSize;
        const uint64_t drow = (uint64_t) (cachePos + s) * kvSize;
        if (cosT) {
            const float *c = cosT + (uint64_t) (ropePos + s) * pairs;
            const float *sn = sinT + (uint64_t) (ropePos + s) * pairs;
            for (uint32_t h = 0; h < nKV; ++h)
                for (uint32_t j = 0; j < pairs; ++j) {
                    const uint32_t b = h * headDim + j;
                    const float k0 = ks[b], k1 = ks[b + pairs];
                    row[b] = fmaf(k0, c[j], -k1 * sn[j]);
                    row[b + pairs] = fmaf(k0, sn[j], k1 * c[j]);
                }
        } else {
            memcpy(row, ks, kvSize * sizeof(float));
        }
        if (kvHalf) {
            _Float16 *kd = (_Float16 *) kDst + drow, *vd = (_Float16 *) vDst + drow;
            for (uint32_t e = 0; e < kvSize; ++e) {
                kd[e] = (_Float16) row[e];
                vd[e] = (_Float16) vs[e];
            }
        } else {
            memcpy((float *) kDst + drow, row, kvSize * sizeof(float));
            memcpy((float *) vDst + drow, vs, kvSize * sizeof(float));
        }
    }
    free(row);
}

/* Model::storeKVWithRoPE (src/cpp/core/ModelPrimitives.cpp:188-219): the CPU
 * engine's append.  It writes x0*c - x1*sn and x0*sn + x1*c as two roundings
 * each (no explicit fused multiply-add), so it may differ from orc_kv_append in
 * the last bit; the f32 tolerance applies between the two. */
void orc_kv_append_cpu(const float *kSrc, const float *vSrc, float *kDst,
                       float *vDst, uint32_t seqLen, uint32_t cachePos,
                       uint32_t kHeads, uint32_t headDim, const float *cosT,
                       const float *sinT) {
    const uint32_t pairs = headDim / 2, kvSize = kHeads * headDim;
    for (uint32_t s = 0; s < seqLen; ++s) {
        const uint32_t p = cachePos + s;
        const float *c = cosT + (uint64_t) p * pairs, *sn = sinT + (uint64_t) p * pairs;
        const float *ks = kSrc + (uint64_t) s * kvSize;
        float *kd = kDst + (uint64_t) p * kvSize;
        for (uint32_t h = 0; h < kHeads; ++h)
            for (uint32_t j = 0; j < pairs; ++j) {
                const float x0 = ks[h * headDim + j], x1 = ks[h * headDim + j + pairs];
                const float a = x0 * c[j], b = x1 * sn[j];
                const float d = x0 * sn[j], e = x1 * c[j];
                kd[h * headDim + j] = a - b;
                kd[h * headDim + j + pairs] = d + e;
            }
        memcpy(vDst + (uint64_t) p * kvSize, vSrc + (uint64_t) s * kvSize,
               kvSize * sizeof(float));
    }
}

/* ------------------------------------------------------------------------- */
/* attention-output epilogues: Q8_1 blocks and the sigmoid gate               */
/* ------------------------------------------------------------------------- */

/* The Q8_1 fold of kAttnCombinePartialW4 (include/gpu/GpuAttentionKernels.hpp:
 * 1068-1096): per 32 consecutive outputs a 40-byte slot {fp16 d = amax/127,
 * fp16 sum, int8 q[32]}, q = roundf(v / d) (half away from zero), 0 when
 * amax == 0.  The block sum is folded with the xor-shuffle butterfly
 * 16,8,4,2,1, emulated here so that the fp16 sum is bit-exact. */
void orc_q8_1_blocks(const float *x, uint8_t *blocks, uint64_t nBlocks) {
    for (uint64_t b = 0; b < nBlocks; ++b) {
        const float *v = x + b * 32;
        float amax[32], sum[32];
        for (int l = 0; l < 32; ++l) {
            amax[l] = fabsf(v[l]);
            sum[l] = v[l];
        }
        for (int o = 16; o > 0; o >>= 1) {
            float a2[32], s2[32];
            for (int l = 0; l < 32; ++l) {
                a2[l] = fmaxf(amax[l], amax[l ^ o]);
                s2[l] = sum[l] + sum[l ^ o];
            }
            memcpy(amax, a2, sizeof(a2));
            memcpy(sum, s2, sizeof(s2));
        }
        const float d = amax[0] / 127.0f;
        uint8_t *blk = blocks + b * 40;
        _Float16 ds[2] = {(_Float16) d, (_Float16) sum[0]};
        memcpy(blk, ds, 4);
        for (int l = 0; l < 32; ++l)
            ((int8_t *) (blk + 4))[l] =
                    amax[0] == 0.0f ? (int8_t) 0 : (int8_t) roundf(v[l] / d);
    }
}

/* kQ35SigmoidGate (include/gpu/GpuQwen35Kernels.hpp:479-493):
 * attnOut[s][h][e] *= 1/(1+exp(-gate)), gate = qGate[s][h][hd + e]
 * (qGate rows are [nHeads][2*hd]). */
void orc_sigmoid_gate(float *attnOut, const float *qGate, uint32_t seqLen,
                      uint32_t nHeads, uint32_t hd) {
    for (uint32_t s = 0; s < seqLen; ++s)
        for (uint32_t h = 0; h < nHeads; ++h)
            for (uint32_t e = 0; e < hd; ++e) {
                const float g = qGate[((uint64_t) s * nHeads + h) * 2 * hd + hd + e];
                attnOut[((uint64_t) s * nHeads + h) * hd + e] *= 1.0f / (1.0f + expf(-g));
            }
}

/* kQ35QNormRoPE / kQ35KNormRoPE (include/gpu/GpuQwen35Kernels.hpp:55-137): one
 * 128-thread block per (token, head) slice.  Thread t folds x[t], x[t+128], ...
 * with fmaf, the 128 partial sums are folded by a shared-memory tree (64, 32,
 * ..., 1 apart); rms = rsqrtf(sum / hd + 1e-6f) -- 1/sqrtf here, the device
 * intrinsic differs from it in the last bits; y = x * rms * w; the first nDims
 * elements are rotated in NEOX pairs (j, j + nDims/2) by table row pos + s with
 * the fmaf form, the rest copied.  in rows have stride inStride (2*hd for the
 * gated q), out rows stride hd; in == out is allowed (the K kernel). */
void orc_norm_rope(const float *in, uint32_t inStride, float *out, const float *w,
                   uint32_t hd, uint32_t nDims, uint32_t heads, uint32_t seqLen,
                   uint32_t pos, const float *cosT, const float *sinT) {
    const uint32_t half = nDims / 2;
    float *tmp = (float *) malloc(sizeof(float) * hd);
    for (uint32_t s = 0; s < seqLen; ++s)
        for (uint32_t h = 0; h < heads; ++h) {
            const float *rp = in + ((uint64_t) s * heads + h) * inStride;
            float *op = out + ((uint64_t) s * heads + h) * hd;
            float part[128];
            for (uint32_t t = 0; t < 128; ++t) {
                float acc = 0.0f;
                for (uint32_t j = t; j < hd; j += 128) acc = fmaf(rp[j], rp[j], acc);
                part[t] = acc;
            }
            for (uint32_t st = 64; st > 0; st >>= 1)
                for (uint32_t t = 0; t < st; ++t) part[t] += part[t + st];
            const float rms = 1.0f / sqrtf(part[0] / (float) hd + 1e-6f);
            const float *c = cosT + (uint64_t) (pos + s) * half;
            const float *sn = sinT + (uint64_t) (pos + s) * half;
            for (uint32_t j = 0; j < half; ++j) {
                const float x0 = rp[j] * rms * w[j];
                const float x1 = rp[j + half] * rms * w[j + half];
                tmp[j] = fmaf(x0, c[j], -x1 * sn[j]);
                tmp[j + half] = fmaf(x0, sn[j], x1 * c[j]);
            }
            for (uint32_t j = nDims; j < hd; ++j) tmp[j] = rp[j] * rms * w[j];
            memcpy(op, tmp, sizeof(float) * hd);
        }
    free(tmp);
}

/* The MRoPE cache of the hybrid models
 * (src/cpp/core/cuda/forward/GPUComputeUpload.cu:1178-1203): [rows][nDims/2],
 * angle = float(p) * theta_j, theta_0 = 1, theta_{j+1} = theta_j * powf(base, -2/nDims). */
void orc_mrope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t nDims,
                      float thetaBase) {
    const uint32_t half = nDims / 2;
    const float scale = powf(thetaBase, -2.0f / (float) nDims);
    for (uint32_t p = 0; p < rows; ++p) {
        float theta = 1.0f;
        for (uint32_t j = 0; j < half; ++j) {
            cosT[(uint64_t) p * half + j] = cosf((float) p * theta);
            sinT[(uint64_t) p * half + j] = sinf((float) p * theta);
            theta *= scale;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* context planner                                                            */
/* ------------------------------------------------------------------------- */

typedef struct {
    uint32_t requested, modelMax, numLayers, numAttentionLayers, numKVHeads,
            headDim, ropeDims;
    uint32_t int8KvSupported, forceKv /* 0 f32, 1 i8 */, forceKvSet;
    uint64_t weightBytes, freeVram, availableRam, gpuFixedOverhead;
} orc_context_request;

typedef struct {
    uint32_t seqLen, maxAllowed, kv /* 0 f32, 1 i8 */, kvMirror, kvOnGpu,
            reduced;
    uint64_t kvBytes;
    char reason[256];
} orc_context_plan;

/* kvStoreBytesPerToken (src/cpp/core/ContextPlan.cpp:58-70). */
uint64_t orc_kv_store_bytes_per_token(const orc_context_request *r, int i8,
                                      int mirror) {
    const uint64_t kvHeads = r->numKVHeads, hd = r->headDim;
    uint64_t perLayer = 2ull * kvHeads * hd * (i8 ? 1ull : 4ull);
    if (i8) perLayer += 2ull * kvHeads * 4ull;
    if (!i8 && mirror) perLayer += 2ull * kvHeads * (hd + 4ull);
    return perLayer;
}

/* kvBytesPerToken (src/cpp/core/ContextPlan.cpp:72-78). */
uint64_t orc_kv_bytes_per_token(const orc_context_request *r, int i8, int mirror) {
    return (uint64_t) r->numAttentionLayers * orc_kv_store_bytes_per_token(r, i8, mirror) +
           4ull * (uint64_t) r->ropeDims;
}

static uint64_t sat_sub(uint64_t a, uint64_t b) { return a > b ? a - b : 0; }

/* planContext (src/cpp/core/ContextPlan.cpp:80-246): budget = free memory minus
 * the fixed overhead and a 256 MiB margin (GPU) or minus 2 GiB slack (RAM);
 * ladder f32+mirror -> f32 -> int8 (GPU, int8 rungs only when supported; a forced
 * precision drops the other rungs); fit = floor256(budget / bytesPerToken)
 * capped at the model max (4096 when unknown); auto asks for min(2048, best
 * fit); below 1024 nothing is granted; the first rung that holds the request
 * wins, otherwise the rung with the largest fit. */
void orc_plan_context(const orc_context_request *r, orc_context_plan *plan) {
    memset(plan, 0, sizeof(*plan));
    const uint64_t MiB = 1024ull * 1024ull;
    const uint32_t ceiling = r->modelMax ? r->modelMax : 4096u;
    const int gpu = r->freeVram != 0;
    const int unknownMax = r->modelMax == 0;
    const uint64_t baseBudget =
            gpu ? sat_sub(sat_sub(r->freeVram, r->gpuFixedOverhead), 256ull * MiB)
                : sat_sub(r->availableRam, 2048ull * MiB);
    struct { int i8, mirror; uint32_t fit; } rungs[3];
    int n = 0;
    const int cand[3][2] = {{0, 1}, {0, 0}, {1, 0}};
    for (int c = 0; c < 3; ++c) {
        const int i8 = cand[c][0], mirror = cand[c][1];
        if (gpu) {
            if ((mirror || i8) && !r->int8KvSupported) continue;
        } else if (i8 || mirror) continue;
        if (r->forceKvSet && i8 != (int) r->forceKv) continue;
        const uint64_t budget = sat_sub(baseBudget, gpu ? r->weightBytes : 0);
        const uint64_t bytes = orc_kv_bytes_per_token(r, i8, mirror);
        uint64_t fit = ceiling;
        if (bytes) {
            fit = (budget / bytes / 256ull) * 256ull;
            if (fit > ceiling) fit = ceiling;
        }
        rungs[n].i8 = i8;
        rungs[n].mirror = mirror;
        rungs[n].fit = (uint32_t) fit;
        ++n;
    }
    uint32_t bestFit = 0;
    for (int i = 0; i < n; ++i) bestFit = rungs[i].fit > bestFit ? rungs[i].fit : bestFit;
    const int clamped = r->requested > ceiling;
    const uint32_t want = r->requested ? (r->requested < ceiling ? r->requested : ceiling)
                                       : (2048u < bestFit ? 2048u : bestFit);
    char buf[256];
    plan->kvOnGpu = gpu;
    if (want < 1024u || bestFit < 1024u) {
        if (r->requested != 0 && r->requested < 1024u)
            snprintf(buf, sizeof(buf), "requested %u, below the 1024-token floor", r->requested);
        else
            snprintf(buf, sizeof(buf), "not even 1024 tokens fit");
        if (!gpu) strncat(buf, "; no GPU, RAM path", sizeof(buf) - strlen(buf) - 1);
        if (unknownMax) strncat(buf, "; model max unknown, assuming 4096", sizeof(buf) - strlen(buf) - 1);
        if (r->forceKvSet && !gpu)
            strncat(buf, r->forceKv ? "; an int8 K/V store needs the GPU" : "; f32 K/V pinned by the caller",
                    sizeof(buf) - strlen(buf) - 1);
        memcpy(plan->reason, buf, sizeof(buf));
        return;
    }
    int chosen = -1;
    for (int i = 0; i < n; ++i)
        if (rungs[i].fit >= want) { chosen = i; break; }
    const int reduced = chosen < 0;
    int widest = -1;
    for (int i = 0; i < n; ++i)
        if (rungs[i].fit == bestFit) { widest = i; break; }
    if (reduced) chosen = widest;
    plan->kv = (uint32_t) rungs[chosen].i8;
    plan->kvMirror = (uint32_t) rungs[chosen].mirror;
    plan->seqLen = want < rungs[chosen].fit ? want : rungs[chosen].fit;
    plan->maxAllowed = bestFit;
    plan->reduced = (uint32_t) reduced;
    plan->kvBytes = (uint64_t) plan->seqLen *
                    orc_kv_bytes_per_token(r, rungs[chosen].i8, rungs[chosen].mirror);
    size_t o = 0;
    if (r->requested) {
        o += snprintf(buf + o, sizeof(buf) - o, "requested %u", r->requested);
        if (clamped) o += snprintf(buf + o, sizeof(buf) - o, ", clamped to model max %u", ceiling);
    } else {
        o += snprintf(buf + o, sizeof(buf) - o, "auto");
        if (bestFit > plan->seqLen)
            o += snprintf(buf + o, sizeof(buf) - o, "; memory allows up to %u at %s%s", bestFit,
                          rungs[widest].i8 ? "int8 K/V" : "f32 K/V",
                          rungs[widest].mirror ? " + mirror" : "");
    }
    if (reduced)
        o += snprintf(buf + o, sizeof(buf) - o, ", limited by %s: %u tokens fit",
                      gpu ? "VRAM" : "RAM", rungs[chosen].fit);
    if (!gpu) o += snprintf(buf + o, sizeof(buf) - o, "; no GPU, RAM path");
    if (unknownMax) o += snprintf(buf + o, sizeof(buf) - o, "; model max unknown, assuming 4096");
    memcpy(plan->reason, buf, sizeof(buf));
}

/* Split-KV chunk geometry chosen at upload
 * (src/cpp/core/cuda/forward/GPUComputeUpload.cu:318-334): chunk starts at 16
 * (32 for 12 heads x 128), is raised to ceil(ceil(maxSeq/512)/32)*32 so that at
 * most 512 chunks cover the window. */
void orc_split_geometry(uint32_t maxSeqLen, uint32_t nHeads, uint32_t headDim,
                        uint32_t *chunk, uint32_t *chunks) {
    uint32_t c = (nHeads == 12 && headDim == 128) ? 32u : 16u;
    const uint32_t minChunk = ((maxSeqLen + 511u) / 512u + 31u) / 32u * 32u;
    if (minChunk > c) c = minChunk;
    uint32_t n = (maxSeqLen + c - 1) / c;
    if (n == 0) n = 1;
    *chunk = c;
    *chunks = n;
}
