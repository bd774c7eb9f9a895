// kv_write.cu -- KV-cache writers: int8 quantise+append, f32/fp16 append with the
// optional NEOX rotation of K (and of Q in place), and RoPE(Q) alone.
//
// All three are pure streaming kernels (HBM-bound, a few hundred KB to a few MB
// per call): one warp per (token, kv-head) row, 128-bit loads and stores, no
// shared memory.  Arithmetic follows the reference element for element so the
// int8 bytes, scales and rotated values are bit-identical to
// kQ35QuantKV8 (include/gpu/GpuQwen35Kernels.hpp:586-637) and
// kStoreKVRope / kRoPEQ (include/gpu/GpuElementwiseKernels.hpp:425-483).
#include "tc_common.cuh"

namespace tc {

// ---------------------------------------------------------------------------
// int8 quantise + append
// ---------------------------------------------------------------------------
// One warp per (token, kv head).  hd is a multiple of 4 and at most 1024; lane l
// owns the float4 groups l, l+32, ...  amax is an exact max, so the reduction
// order is free; the division is IEEE (__fdiv_rn) and the rounding is
// round-half-even (__float2int_rn), which is what lrintf does under the default
// rounding mode.
template <int MAXV>
__global__ void __launch_bounds__(256)
kvQuantKernel(const float *__restrict__ k, const float *__restrict__ v, int8_t *__restrict__ k8,
              int8_t *__restrict__ v8, float *__restrict__ ks, float *__restrict__ vs, uint32_t tokens,
              uint32_t nKV, uint32_t hd, uint64_t dstTokenBase, uint64_t srcTokenBase,
              const uint32_t *__restrict__ devDstBase, uint32_t batchMode, uint64_t rowsPerSeq,
              const uint64_t *__restrict__ rowBase, const uint32_t *__restrict__ devLens, int32_t lenAdd,
              uint64_t maxRows, unsigned int *__restrict__ err) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= static_cast<uint64_t>(tokens) * nKV) return;
    if (devDstBase != nullptr) dstTokenBase = devDstBase[0];
    const uint64_t t = row / nKV, h = row % nKV;
    const uint64_t src = ((srcTokenBase + t) * nKV + h) * hd;
    uint64_t dst = (dstTokenBase + t) * nKV + h;
    if (batchMode) {
        // source row t is the new token of sequence t; it goes behind that sequence's rows
        const uint64_t base = rowBase != nullptr ? rowBase[t] : t * rowsPerSeq;
        const uint64_t pos = devLens != nullptr ? static_cast<uint64_t>(static_cast<int64_t>(devLens[t]) + lenAdd)
                                                : dstTokenBase;
        dst = (base + pos) * nKV + h;
    }
    // A destination row read from device memory (a replayed graph past its window, a bad length)
    // is checked here, where it is known: the store is skipped and the error word says so.
    if (maxRows != 0 && dst >= maxRows * nKV) {
        if (lane == 0) atomicOr(err, kDevErrRowBound);
        return;
    }
    const uint32_t nvec = hd >> 2;
    float4 kx[MAXV], vx[MAXV];
    float mk = 0.0f, mv = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const uint32_t i = lane + 32u * j;
        if (i < nvec) {
            kx[j] = __ldg(reinterpret_cast<const float4 *>(k + src) + i);
            vx[j] = __ldg(reinterpret_cast<const float4 *>(v + src) + i);
            mk = fmaxf(mk, fmaxf(fmaxf(fabsf(kx[j].x), fabsf(kx[j].y)), fmaxf(fabsf(kx[j].z), fabsf(kx[j].w))));
            mv = fmaxf(mv, fmaxf(fmaxf(fabsf(vx[j].x), fabsf(vx[j].y)), fmaxf(fabsf(vx[j].z), fabsf(vx[j].w))));
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
    const float sk = mk > 0.0f ? __fdiv_rn(mk, 127.0f) : 1.0f;
    const float sv = mv > 0.0f ? __fdiv_rn(mv, 127.0f) : 1.0f;
    if (lane == 0) {
        ks[dst] = sk;
        vs[dst] = sv;
    }
    auto q8 = [](float x, float s) -> uint32_t {
        int q = __float2int_rn(__fdiv_rn(x, s));
        q = q < -128 ? -128 : (q > 127 ? 127 : q);
        return static_cast<uint32_t>(q) & 0xffu;
    };
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const uint32_t i = lane + 32u * j;
        if (i < nvec) {
            const uint32_t pk = q8(kx[j].x, sk) | (q8(kx[j].y, sk) << 8) | (q8(kx[j].z, sk) << 16) |
                                (q8(kx[j].w, sk) << 24);
            const uint32_t pv = q8(vx[j].x, sv) | (q8(vx[j].y, sv) << 8) | (q8(vx[j].z, sv) << 16) |
                                (q8(vx[j].w, sv) << 24);
            reinterpret_cast<uint32_t *>(k8 + dst * hd)[i] = pk;
            reinterpret_cast<uint32_t *>(v8 + dst * hd)[i] = pv;
        }
    }
}

// ---------------------------------------------------------------------------
// f32 / fp16 append, optional rotation
// ---------------------------------------------------------------------------
template <typename KVT>
__device__ __forceinline__ void storeElem(KVT *p, float x);
template <>
__device__ __forceinline__ void storeElem<float>(float *p, float x) { *p = x; }
template <>
__device__ __forceinline__ void storeElem<__half>(__half *p, float x) { *p = __float2half_rn(x); }

// One block per token.  Threads sweep (a) the q heads' rotation pairs, (b) V
// verbatim, (c) the K heads' rotation pairs (or K verbatim without tables).
// x0' = fmaf(x0, c, -(x1*s)), x1' = fmaf(x0, s, x1*c): the reference's form.
template <typename KVT>
__global__ void __launch_bounds__(256)
kvAppendKernel(float *__restrict__ q, const float *__restrict__ kSrc, const float *__restrict__ vSrc,
               KVT *__restrict__ kDst, KVT *__restrict__ vDst, uint32_t nHeads, uint32_t nKV, uint32_t hd,
               uint32_t cachePos, uint32_t ropePos, const uint32_t *__restrict__ devPos,
               const float *__restrict__ cosT, const float *__restrict__ sinT, uint32_t maxRows,
               unsigned int *__restrict__ err) {
    const uint32_t s = blockIdx.x;
    if (devPos != nullptr) {
        cachePos = devPos[0];
        ropePos = devPos[0];
    }
    const uint32_t pairs = hd >> 1;
    const uint32_t kvSize = nKV * hd;
    const float *c = cosT ? cosT + static_cast<size_t>(ropePos + s) * pairs : nullptr;
    const float *sn = sinT ? sinT + static_cast<size_t>(ropePos + s) * pairs : nullptr;
    if (q != nullptr && c != nullptr) {
        const uint32_t total = nHeads * pairs;
        for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
            const uint32_t h = idx / pairs, j = idx - h * pairs;
            float *head = q + (static_cast<size_t>(s) * nHeads + h) * hd;
            const float x0 = head[j], x1 = head[j + pairs];
            head[j] = fmaf(x0, c[j], -__fmul_rn(x1, sn[j]));
            head[j + pairs] = fmaf(x0, sn[j], __fmul_rn(x1, c[j]));
        }
    }
    if (kSrc == nullptr) return;
    if (maxRows != 0 && static_cast<uint64_t>(cachePos) + s >= maxRows) {
        // device-side position outside the window: no store, reported through the error word
        if (threadIdx.x == 0) atomicOr(err, kDevErrRowBound);
        return;
    }
    const float *ks = kSrc + static_cast<size_t>(s) * kvSize;
    const float *vs = vSrc + static_cast<size_t>(s) * kvSize;
    KVT *kd = kDst + static_cast<size_t>(cachePos + s) * kvSize;
    KVT *vd = vDst + static_cast<size_t>(cachePos + s) * kvSize;
    for (uint32_t e = threadIdx.x; e < kvSize; e += blockDim.x) storeElem<KVT>(vd + e, vs[e]);
    if (c != nullptr) {
        const uint32_t total = nKV * pairs;
        for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
            const uint32_t h = idx / pairs, j = idx - h * pairs;
            const uint32_t b = h * hd + j;
            const float k0 = ks[b], k1 = ks[b + pairs];
            storeElem<KVT>(kd + b, fmaf(k0, c[j], -__fmul_rn(k1, sn[j])));
            storeElem<KVT>(kd + b + pairs, fmaf(k0, sn[j], __fmul_rn(k1, c[j])));
        }
    } else {
        for (uint32_t e = threadIdx.x; e < kvSize; e += blockDim.x) storeElem<KVT>(kd + e, ks[e]);
    }
}

// attnOut[s][h][e] *= 1/(1+exp(-gate)); gate is the second half of each head's
// fused q+gate row.  The reference evaluates the sigmoid with __expf.
__global__ void __launch_bounds__(256)
sigmoidGateKernel(float *__restrict__ attnOut, const float *__restrict__ qGate, uint32_t nHeads, uint32_t hd) {
    const uint32_t s = blockIdx.x;
    const uint32_t total = nHeads * hd;
    for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const uint32_t h = idx / hd, e = idx - h * hd;
        const float g = qGate[(static_cast<size_t>(s) * nHeads + h) * 2 * hd + hd + e];
        attnOut[static_cast<size_t>(s) * total + idx] *= 1.0f / (1.0f + __expf(-g));
    }
}

}  // namespace tc

extern "C" {

int tc_kv_quantize_i8(const float *k, const float *v, int8_t *k8, int8_t *v8, float *ks, float *vs,
                      uint32_t tokens, uint32_t nKV, uint32_t hd, uint64_t dstTokenBase,
                      uint64_t srcTokenBase, const uint32_t *devDstBase, uint64_t maxRows, tc_stream stream) {
    TC_REQUIRE(k && v && k8 && v8 && ks && vs, TC_EINVAL, "tc_kv_quantize_i8: null pointer");
    TC_REQUIRE(nKV > 0 && hd > 0 && (hd % 4u) == 0 && hd <= 1024, TC_EUNSUPPORTED,
               "tc_kv_quantize_i8: hd=%u must be a multiple of 4 and <= 1024", hd);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0 &&
                       ((reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8)) & 3u) == 0,
               TC_EINVAL, "tc_kv_quantize_i8: k/v need 16-byte, k8/v8 4-byte alignment");
    if (tokens == 0) return TC_OK;
    if (devDstBase == nullptr && maxRows != 0 && dstTokenBase + tokens > maxRows) {
        tc::setError("tc_kv_quantize_i8: rows [%llu, %llu) pass the pool's %llu rows",
                     (unsigned long long) dstTokenBase, (unsigned long long) (dstTokenBase + tokens),
                     (unsigned long long) maxRows);
        return TC_ECONTEXT_FULL;
    }
    unsigned int *err = tc::devErrorWord();
    TC_REQUIRE(err != nullptr, TC_ECUDA, "tc_kv_quantize_i8: no device error word");
    const uint64_t rows = static_cast<uint64_t>(tokens) * nKV;
    const uint32_t warpsPerBlock = 8;
    const uint64_t blocks = (rows + warpsPerBlock - 1) / warpsPerBlock;
    TC_REQUIRE(blocks <= 0x7fffffffull, TC_EUNSUPPORTED, "tc_kv_quantize_i8: too many rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t nvec = hd / 4;
    if (nvec <= 32)
        tc::kvQuantKernel<1><<<static_cast<uint32_t>(blocks), 256, 0, st>>>(
                k, v, k8, v8, ks, vs, tokens, nKV, hd, dstTokenBase, srcTokenBase, devDstBase, 0u, 0ull, nullptr, nullptr, 0, maxRows, err);
    else if (nvec <= 64)
        tc::kvQuantKernel<2><<<static_cast<uint32_t>(blocks), 256, 0, st>>>(
                k, v, k8, v8, ks, vs, tokens, nKV, hd, dstTokenBase, srcTokenBase, devDstBase, 0u, 0ull, nullptr, nullptr, 0, maxRows, err);
    else
        tc::kvQuantKernel<8><<<static_cast<uint32_t>(blocks), 256, 0, st>>>(
                k, v, k8, v8, ks, vs, tokens, nKV, hd, dstTokenBase, srcTokenBase, devDstBase, 0u, 0ull, nullptr, nullptr, 0, maxRows, err);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

int tc_kv_quantize_i8_batch(const float *k, const float *v, int8_t *k8, int8_t *v8, float *ks, float *vs,
                            uint32_t batch, uint32_t nKV, uint32_t hd, uint64_t rowsPerSeq, const uint64_t *rowBase,
                            uint32_t pos, const uint32_t *lens, int32_t lenAdd, uint64_t totalRows, tc_stream stream) {
    TC_REQUIRE(k && v && k8 && v8 && ks && vs, TC_EINVAL, "tc_kv_quantize_i8_batch: null pointer");
    TC_REQUIRE(nKV > 0 && hd > 0 && (hd % 4u) == 0 && hd <= 1024, TC_EUNSUPPORTED,
               "tc_kv_quantize_i8_batch: hd=%u must be a multiple of 4 and <= 1024", hd);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0 &&
                       ((reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8)) & 3u) == 0,
               TC_EINVAL, "tc_kv_quantize_i8_batch: k/v need 16-byte, k8/v8 4-byte alignment");
    if (batch == 0) return TC_OK;
    if (lens == nullptr && rowBase == nullptr && totalRows != 0 &&
        static_cast<uint64_t>(batch - 1) * rowsPerSeq + pos >= totalRows) {
        tc::setError("tc_kv_quantize_i8_batch: row %u of sequence %u passes the pool's %llu rows", pos, batch - 1,
                     (unsigned long long) totalRows);
        return TC_ECONTEXT_FULL;
    }
    unsigned int *err = tc::devErrorWord();
    TC_REQUIRE(err != nullptr, TC_ECUDA, "tc_kv_quantize_i8_batch: no device error word");
    const uint64_t rows = static_cast<uint64_t>(batch) * nKV;
    const uint32_t blocks = static_cast<uint32_t>((rows + 7) / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t nvec = hd / 4;
    if (nvec <= 32)
        tc::kvQuantKernel<1><<<blocks, 256, 0, st>>>(k, v, k8, v8, ks, vs, batch, nKV, hd, pos, 0, nullptr, 1u, rowsPerSeq,
                                                     rowBase, lens, lenAdd, totalRows, err);
    else if (nvec <= 64)
        tc::kvQuantKernel<2><<<blocks, 256, 0, st>>>(k, v, k8, v8, ks, vs, batch, nKV, hd, pos, 0, nullptr, 1u, rowsPerSeq,
                                                     rowBase, lens, lenAdd, totalRows, err);
    else
        tc::kvQuantKernel<8><<<blocks, 256, 0, st>>>(k, v, k8, v8, ks, vs, batch, nKV, hd, pos, 0, nullptr, 1u, rowsPerSeq,
                                                     rowBase, lens, lenAdd, totalRows, err);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

static int appendCommon(float *q, const float *kSrc, const float *vSrc, void *kDst, void *vDst, int kvHalf,
                        uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos,
                        uint32_t ropePos, const uint32_t *devPos, const float *cosT, const float *sinT,
                        uint32_t maxRows, tc_stream stream, const char *who) {
    TC_REQUIRE(kSrc && vSrc && kDst && vDst, TC_EINVAL, "%s: null pointer", who);
    TC_REQUIRE(nKV > 0 && hd > 0 && (hd % 2u) == 0, TC_EUNSUPPORTED, "%s: hd=%u must be even", who, hd);
    TC_REQUIRE((cosT == nullptr) == (sinT == nullptr), TC_EINVAL, "%s: cos and sin tables come together", who);
    if (seqLen == 0) return TC_OK;
    if (devPos == nullptr && maxRows != 0 &&
        static_cast<uint64_t>(cachePos) + seqLen > static_cast<uint64_t>(maxRows)) {
        tc::setError("%s: rows [%u, %llu) pass the window of %u rows", who, cachePos,
                     (unsigned long long) cachePos + seqLen, maxRows);
        return TC_ECONTEXT_FULL;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int *err = tc::devErrorWord();
    TC_REQUIRE(err != nullptr, TC_ECUDA, "%s: no device error word", who);
    if (kvHalf)
        tc::kvAppendKernel<__half><<<seqLen, 256, 0, st>>>(q, kSrc, vSrc, static_cast<__half *>(kDst),
                                                          static_cast<__half *>(vDst), nHeads, nKV, hd,
                                                          cachePos, ropePos, devPos, cosT, sinT, maxRows, err);
    else
        tc::kvAppendKernel<float><<<seqLen, 256, 0, st>>>(q, kSrc, vSrc, static_cast<float *>(kDst),
                                                         static_cast<float *>(vDst), nHeads, nKV, hd, cachePos,
                                                         ropePos, devPos, cosT, sinT, maxRows, err);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

int tc_kv_append(const float *kSrc, const float *vSrc, void *kDst, void *vDst, int kvHalf, uint32_t seqLen,
                 uint32_t nKV, uint32_t hd, uint32_t cachePos, const uint32_t *devPos, uint32_t maxRows,
                 tc_stream stream) {
    return appendCommon(nullptr, kSrc, vSrc, kDst, vDst, kvHalf, seqLen, 0, nKV, hd, cachePos, 0, devPos,
                        nullptr, nullptr, maxRows, stream, "tc_kv_append");
}

int tc_kv_append_rope(float *q, const float *kSrc, const float *vSrc, void *kDst, void *vDst, int kvHalf,
                      uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos,
                      uint32_t ropePos, const uint32_t *devPos, const float *cosT, const float *sinT,
                      uint32_t maxRows, tc_stream stream) {
    TC_REQUIRE(cosT && sinT, TC_EINVAL, "tc_kv_append_rope: cos/sin tables are required");
    return appendCommon(q, kSrc, vSrc, kDst, vDst, kvHalf, seqLen, nHeads, nKV, hd, cachePos, ropePos, devPos,
                        cosT, sinT, maxRows, stream, "tc_kv_append_rope");
}

int tc_rope_q(float *q, const float *cosT, const float *sinT, uint32_t seqLen, uint32_t nHeads, uint32_t hd,
              uint32_t pos, const uint32_t *devPos, tc_stream stream) {
    TC_REQUIRE(q && cosT && sinT, TC_EINVAL, "tc_rope_q: null pointer");
    TC_REQUIRE(hd > 0 && (hd % 2u) == 0, TC_EUNSUPPORTED, "tc_rope_q: hd=%u must be even", hd);
    if (seqLen == 0) return TC_OK;
    tc::kvAppendKernel<float><<<seqLen, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            q, nullptr, nullptr, nullptr, nullptr, nHeads, 0, hd, 0, pos, devPos, cosT, sinT, 0u, nullptr);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

int tc_attn_sigmoid_gate(float *attnOut, const float *qGate, uint32_t seqLen, uint32_t nHeads, uint32_t hd,
                         tc_stream stream) {
    TC_REQUIRE(attnOut && qGate, TC_EINVAL, "tc_attn_sigmoid_gate: null pointer");
    if (seqLen == 0) return TC_OK;
    tc::sigmoidGateKernel<<<seqLen, 256, 0, static_cast<cudaStream_t>(stream)>>>(attnOut, qGate, nHeads, hd);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

}  // extern "C"
