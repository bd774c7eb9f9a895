// ref_gpu_shim.cu -- C entry points around the reference project's OWN CUDA
// attention / KV kernels.  TEST INFRASTRUCTURE ONLY: nothing that ships links or
// loads what this builds.
//
// oracle/Makefile (target `refgpu`) compiles this one translation unit, which
// includes the reference's kernel header set where it lies
// (include/GPUComputeInternal.hpp, all kernels in one anonymous namespace), into
// oracle/_ref/libtc_ref_gpu.so.  The wrappers add no arithmetic: each one issues
// exactly the launch the reference issues at the cited call site, on the default
// stream, and returns the CUDA error code after a synchronise.  The library is
// used (a) by tests/golden/make_ref_gpu_golden.py to record the reference kernels'
// outputs on seeded inputs, which pin the CPU restatement in oracle/tc_oracle.c,
// and (b) never by the product.
#define USE_CUDA 1
#include "GPUComputeInternal.hpp"

namespace tinycoder::gpu {

static int done() {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return static_cast<int>(e);
}

extern "C" {

// kQ35QuantKV8 as launched in src/cpp/core/cuda/forward/GPUComputeMoE.cu:3056-3063, 3103-3105
int ref_gpu_quant_kv8(const float *k, const float *v, int8_t *k8, int8_t *v8, float *ks, float *vs,
                      uint32_t tokens, uint32_t nKV, uint32_t hd, uint32_t dstTokenBase, uint32_t srcTokenBase) {
    kQ35QuantKV8<<<dim3(tokens, nKV), 128>>>(k, v, k8, v8, ks, vs, tokens, nKV, hd, dstTokenBase, srcTokenBase);
    return done();
}

// kQ35WarpAttention8Split + kAttnCombinePartial<256> (GPUComputeMoE.cu:3073-3083); hd must be 256
int ref_gpu_decode_i8_split(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                            float *pAcc, float *pM, float *pL, float *out, uint32_t nHeads, uint32_t nKV,
                            uint32_t cachePos, uint32_t numChunks, uint32_t chunkSize, float invSqrt) {
    kQ35WarpAttention8Split<<<dim3(1, numChunks, nHeads), dim3(32, 1)>>>(q, k8, v8, ks, vs, pAcc, pM, pL, nHeads, nKV,
                                                                          cachePos, numChunks, chunkSize, 256,
                                                                          invSqrt);
    kAttnCombinePartial<256><<<dim3(1, nHeads), 32>>>(pAcc, pM, pL, out, 1, nHeads, numChunks);
    return done();
}

// kQ35WarpAttention8 (GPUComputeMoE.cu:3085-3089); hd must be 256
int ref_gpu_decode_i8_eager(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                            float *out, uint32_t nHeads, uint32_t nKV, uint32_t cachePos, float invSqrt) {
    kQ35WarpAttention8<<<dim3((nHeads + 3) / 4), dim3(32, 4)>>>(q, k8, v8, ks, vs, out, nHeads, nKV, cachePos, 256,
                                                                invSqrt);
    return done();
}

// kQ35WarpAttention8Prefill<256, 4> (GPUComputeMoE.cu:3124-3129)
int ref_gpu_prefill_i8(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                       float *out, uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t cachePos,
                       float invSqrt) {
    kQ35WarpAttention8Prefill<256, 4><<<dim3(seqLen, (nHeads + 3) / 4), dim3(32, 4)>>>(
            q, k8, v8, ks, vs, out, seqLen, nHeads, nKV, cachePos, nullptr, invSqrt);
    return done();
}

// launchDecodeAttentionSplit (GPUComputeForward.cu:3897-3902): f32 cache, hd 32 / 64 / 128
int ref_gpu_decode_f32(const float *q, const float *kvK, const float *kvV, float *out, float *pAcc, float *pM,
                       float *pL, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t pos, uint32_t numChunks,
                       uint32_t chunkSize, float invSqrt, uint8_t *q81) {
    launchDecodeAttentionSplit(q, kvK, kvV, out, pAcc, pM, pL, 1, nHeads, nKV, hd, pos, false, nullptr, numChunks,
                               chunkSize, invSqrt, false, q81);
    return done();
}

// kWarpAttention<HD, float> (GPUComputeForward.cu:3920-3934)
int ref_gpu_attention_f32(const float *q, const float *kvK, const float *kvV, float *out, uint32_t seqLen,
                          uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos, float invSqrt) {
    dim3 grid(seqLen, (nHeads + 3) / 4), blk(32, 4);
    if (hd == 128) kWarpAttention<128, float><<<grid, blk>>>(q, kvK, kvV, out, seqLen, nHeads, nKV, cachePos, invSqrt);
    else if (hd == 64) kWarpAttention<64, float><<<grid, blk>>>(q, kvK, kvV, out, seqLen, nHeads, nKV, cachePos, invSqrt);
    else if (hd == 256) kWarpAttention<256, float><<<grid, blk>>>(q, kvK, kvV, out, seqLen, nHeads, nKV, cachePos, invSqrt);
    else return -1;
    return done();
}

// kRoPEQStoreKV<float> for seqLen == 1 is the same arithmetic; the two-launch form
// (GPUComputeForward.cu:3797-3799, 3892-3894) covers any seqLen
int ref_gpu_rope_store(float *q, const float *kSrc, const float *vSrc, float *kDst, float *vDst, uint32_t seqLen,
                       uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos, uint32_t pos,
                       const float *cosT, const float *sinT) {
    kRoPEQ<<<seqLen, 128>>>(q, cosT, sinT, seqLen, nHeads, hd, pos);
    kStoreKVRope<float><<<seqLen, 256>>>(kSrc, vSrc, kDst, vDst, seqLen, nKV, hd, cachePos, pos, cosT, sinT);
    return done();
}

// kAttnCombinePartialW4<128, 8> with the Q8_1 fold (GpuAttentionKernels.hpp:1195-1197)
int ref_gpu_combine_w8_q81(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t nHeads,
                           uint32_t numChunks, uint8_t *q81) {
    kAttnCombinePartialW4<128, 8><<<dim3(1, nHeads), 256>>>(pAcc, pM, pL, out, 1, nHeads, numChunks, q81);
    return done();
}

// kQ35SigmoidGate (GPUComputeMoE.cu:3205-3206)
int ref_gpu_sigmoid_gate(float *attnOut, const float *qGate, uint32_t seqLen, uint32_t nHeads, uint32_t hd) {
    kQ35SigmoidGate<<<seqLen, 256>>>(attnOut, qGate, seqLen, nHeads, hd);
    return done();
}

// kF32ToF16 + kAttnSoftmaxCausal (GPUComputeForward.cu:3957-3968, 4000-4003): the two
// non-library pieces of the materialised prefill; scores come from the caller
int ref_gpu_softmax_causal(const float *scores, __half *pOut, uint32_t seqLen, uint32_t nHeads, float scale) {
    kAttnSoftmaxCausal<<<dim3(seqLen, nHeads), 128>>>(scores, pOut, seqLen, seqLen * seqLen, 0, scale);
    return done();
}

// The whole materialised prefill of GPUComputeForward.cu:3957-4026 for one layer, call for call:
// kF32ToF16 twins of q and of the stored K/V rows, one cublasGemmStridedBatchedEx per q head
// for the scores (A = K of the head's group with batch stride 0, B = Q of the head, fp16
// operands, f32 output, f32 compute, CUBLAS_GEMM_DEFAULT_TENSOR_OP), kAttnSoftmaxCausal, one
// cublasGemmStridedBatchedEx per q head for P V into attnOut with the head stride.  The K/V
// rows are taken as already stored (the rotation / store kernels in front are pinned on their
// own); the scratch the engine keeps in scratch_ is allocated and freed here.
int ref_gpu_prefill_f16_gemm(const float *q, const float *kF, const float *vF, float *attnOut, uint32_t seqLen,
                             uint32_t nHeads, uint32_t nKV, uint32_t hd, float invSqrt) {
    const uint32_t qLen = nHeads * hd, kvLen = nKV * hd, pos = 0;
    const uint32_t s2 = seqLen * seqLen;
    __half *q16 = nullptr, *kv16 = nullptr, *p16 = nullptr;
    float *scores = nullptr;
    const uint64_t cap = seqLen;  // attnGemmCap
    if (cudaMalloc(&q16, sizeof(__half) * seqLen * qLen) != cudaSuccess ||
        cudaMalloc(&kv16, sizeof(__half) * 2 * cap * kvLen) != cudaSuccess ||
        cudaMalloc(&scores, sizeof(float) * static_cast<uint64_t>(nHeads) * s2) != cudaSuccess ||
        cudaMalloc(&p16, sizeof(__half) * static_cast<uint64_t>(nHeads) * s2) != cudaSuccess)
        return -2;
    cublasHandle_t handle = nullptr;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return -3;
    cublasSetStream(handle, nullptr);
    int rc = 0;
    {
        const uint32_t qElems = seqLen * qLen;
        kF32ToF16<<<(qElems + 511u) / 512u, 256>>>(q, reinterpret_cast<__half2 *>(q16), qElems / 2u);
        const uint32_t nRows = pos + seqLen;
        const uint32_t kvElems = nRows * kvLen;
        __half *k16 = kv16;
        __half *v16 = k16 + cap * kvLen;
        kF32ToF16<<<(kvElems + 511u) / 512u, 256>>>(kF, reinterpret_cast<__half2 *>(k16), kvElems / 2u);
        kF32ToF16<<<(kvElems + 511u) / 512u, 256>>>(vF, reinterpret_cast<__half2 *>(v16), kvElems / 2u);
        const uint32_t gw = nHeads / nKV;
        const float geAlpha = 1.0f, geBeta = 0.0f;
        for (uint32_t h0 = 0; h0 < nHeads && rc == 0; ++h0) {
            const uint32_t g = h0 / gw;
            cublasStatus_t st = cublasGemmStridedBatchedEx(
                    handle, CUBLAS_OP_T, CUBLAS_OP_N, static_cast<int>(seqLen), static_cast<int>(seqLen),
                    static_cast<int>(hd), &geAlpha, k16 + static_cast<uint64_t>(g) * hd, CUDA_R_16F,
                    static_cast<int>(kvLen), 0LL, q16 + static_cast<uint64_t>(h0) * hd, CUDA_R_16F,
                    static_cast<int>(qLen), static_cast<long long>(hd), &geBeta,
                    scores + static_cast<uint64_t>(h0) * s2, CUDA_R_32F, static_cast<int>(seqLen),
                    static_cast<long long>(s2), 1, CUDA_R_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
            if (st != CUBLAS_STATUS_SUCCESS) rc = -4;
        }
        kAttnSoftmaxCausal<<<dim3(seqLen, nHeads), 128>>>(scores, p16, seqLen, s2, pos, invSqrt);
        for (uint32_t h0 = 0; h0 < nHeads && rc == 0; ++h0) {
            const uint32_t g = h0 / gw;
            cublasStatus_t st = cublasGemmStridedBatchedEx(
                    handle, CUBLAS_OP_N, CUBLAS_OP_N, static_cast<int>(hd), static_cast<int>(seqLen),
                    static_cast<int>(seqLen), &geAlpha, v16 + static_cast<uint64_t>(g) * hd, CUDA_R_16F,
                    static_cast<int>(kvLen), 0LL, p16 + static_cast<uint64_t>(h0) * s2, CUDA_R_16F,
                    static_cast<int>(seqLen), static_cast<long long>(s2), &geBeta,
                    attnOut + static_cast<uint64_t>(h0) * hd, CUDA_R_32F, static_cast<int>(qLen),
                    static_cast<long long>(hd), 1, CUDA_R_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
            if (st != CUBLAS_STATUS_SUCCESS) rc = -5;
        }
    }
    const int e = done();
    cublasDestroy(handle);
    cudaFree(q16);
    cudaFree(kv16);
    cudaFree(scores);
    cudaFree(p16);
    return rc != 0 ? rc : e;
}

// kQ35QNormRoPE + kQ35KNormRoPE as launched at GPUComputeForward.cu:1330-1337
int ref_gpu_qk_norm_rope(const float *qGate, float *qOut, float *k, const float *wq, const float *wk, uint32_t hd,
                         uint32_t nDims, uint32_t nHeads, uint32_t nKV, uint32_t seqLen, uint32_t pos,
                         const float *cosT, const float *sinT) {
    kQ35QNormRoPE<<<dim3(seqLen, nHeads), 128, 128 * sizeof(float)>>>(qGate, qOut, wq, hd, nDims, nHeads, seqLen, pos,
                                                                     nullptr, cosT, sinT);
    kQ35KNormRoPE<<<dim3(seqLen, nKV), 128, 128 * sizeof(float)>>>(k, wk, hd, nDims, nKV, seqLen, pos, nullptr, cosT,
                                                                  sinT);
    return done();
}

}  // extern "C"

}  // namespace tinycoder::gpu
