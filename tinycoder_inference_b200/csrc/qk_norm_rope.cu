// qk_norm_rope.cu -- the step in front of attention in the hybrid (gated) models: per-head
// RMSNorm of Q and K fused with the partial NEOX rotation by the MRoPE tables.
//
// What it replaces: kQ35QNormRoPE and kQ35KNormRoPE (include/gpu/GpuQwen35Kernels.hpp:55-137),
// launched back to back in front of the KV store
// (src/cpp/core/cuda/forward/GPUComputeForward.cu:1330-1337):
//   rms = rsqrt(sum(x^2) / hd + 1e-6);  y_j = x_j * rms * w_j;
//   j < nDims/2:  out_j = fma(y_j, c_j, -y_{j+h} * s_j),  out_{j+h} = fma(y_j, s_j, y_{j+h} * c_j)
//   j >= nDims:   out_j = y_j                                   (h = nDims/2, tables [pos][h])
// Q is read from the projection's [token][head][2*hd] rows (q then gate) and written out of
// place as [token][head][hd]; K is normalised in place.
//
// One launch does both, one WARP per (token, head) slice with everything in registers (the
// reference uses a 128-thread block and a shared-memory tree per slice).  The sum of squares
// is folded in the reference's order -- element j belongs to thread j mod 128 of its block,
// threads are folded 64, 32, ..., 1 apart -- so the normaliser, and with it every output, is
// bit-identical: a lane carries the four "threads" lane, lane+32, lane+64, lane+96.
#include "tc_common.cuh"

namespace tc {

constexpr int kNormMaxPer = 4;  // elements per reference thread: hd <= 512

__global__ void __launch_bounds__(256)
qkNormRopeKernel(const float *__restrict__ qIn, uint32_t qInStride, float *qOut, float *k,
                 const float *__restrict__ wq, const float *__restrict__ wk, uint32_t hd, uint32_t nDims,
                 uint32_t nHeads, uint32_t nKV, uint32_t seqLen, uint32_t pos, const uint32_t *__restrict__ devPos,
                 const float *__restrict__ cosT, const float *__restrict__ sinT) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t slices = (qIn ? nHeads : 0u) + (k ? nKV : 0u);
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= static_cast<uint64_t>(seqLen) * slices) return;
    const uint32_t s = static_cast<uint32_t>(idx / slices);
    uint32_t h = static_cast<uint32_t>(idx % slices);
    const bool isQ = qIn != nullptr && h < nHeads;
    if (!isQ && qIn != nullptr) h -= nHeads;
    const float *rp = isQ ? qIn + (static_cast<uint64_t>(s) * nHeads + h) * qInStride
                          : k + (static_cast<uint64_t>(s) * nKV + h) * hd;
    float *op = isQ ? qOut + (static_cast<uint64_t>(s) * nHeads + h) * hd : k + (static_cast<uint64_t>(s) * nKV + h) * hd;
    const float *w = isQ ? wq : wk;

    // element j = lane + 32 i + 128 kk  (reference thread lane + 32 i, its kk-th element)
    float x[4][kNormMaxPer];
    float a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a[i] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < kNormMaxPer; ++kk) {
            const uint32_t j = lane + 32u * i + 128u * kk;
            x[i][kk] = j < hd ? rp[j] : 0.0f;
            if (j < hd) a[i] = fmaf(x[i][kk], x[i][kk], a[i]);
        }
    }
    float sum = (a[0] + a[2]) + (a[1] + a[3]);  // threads 64 apart, then 32 apart
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float rms = rsqrtf(sum / static_cast<float>(hd) + 1e-6f);
    const uint32_t p = (devPos != nullptr ? devPos[0] : pos) + s;
    const uint32_t half = nDims / 2;
    const float *c = cosT + static_cast<uint64_t>(p) * half;
    const float *sn = sinT + static_cast<uint64_t>(p) * half;
    // The partner of element j sits `half` away: it is fetched from global memory again rather
    // than shuffled (half is a run-time value; the row was just read and is in L1).  K is
    // rotated in place, so every read happens before the first write.
    float y[4][kNormMaxPer];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int kk = 0; kk < kNormMaxPer; ++kk) {
            const uint32_t j = lane + 32u * i + 128u * kk;
            y[i][kk] = 0.0f;
            if (j >= hd) continue;
            const float yj = x[i][kk] * rms * w[j];
            if (j < half) {
                const float y1 = rp[j + half] * rms * w[j + half];
                y[i][kk] = fmaf(yj, c[j], -y1 * sn[j]);
            } else if (j < nDims) {
                const uint32_t j0 = j - half;
                const float y0 = rp[j0] * rms * w[j0];
                y[i][kk] = fmaf(y0, sn[j0], yj * c[j0]);
            } else {
                y[i][kk] = yj;
            }
        }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int kk = 0; kk < kNormMaxPer; ++kk) {
            const uint32_t j = lane + 32u * i + 128u * kk;
            if (j < hd) op[j] = y[i][kk];
        }
}

}  // namespace tc

extern "C" int tc_qk_norm_rope(const float *qIn, uint32_t qInStride, float *qOut, float *k, const float *wq,
                               const float *wk, uint32_t hd, uint32_t nDims, uint32_t nHeads, uint32_t nKV,
                               uint32_t seqLen, uint32_t pos, const uint32_t *devPos, const float *cosT,
                               const float *sinT, uint32_t tableRows, tc_stream stream) {
    TC_REQUIRE(cosT && sinT, TC_EINVAL, "tc_qk_norm_rope: null table");
    TC_REQUIRE((qIn == nullptr) == (qOut == nullptr), TC_EINVAL, "tc_qk_norm_rope: q input and output go together");
    TC_REQUIRE(qIn != nullptr || k != nullptr, TC_EINVAL, "tc_qk_norm_rope: nothing to do");
    TC_REQUIRE((qIn == nullptr || wq != nullptr) && (k == nullptr || wk != nullptr), TC_EINVAL,
               "tc_qk_norm_rope: missing norm weight");
    TC_REQUIRE(hd >= 2 && hd <= 128u * tc::kNormMaxPer, TC_EUNSUPPORTED, "tc_qk_norm_rope: head_dim %u (max %u)", hd,
               128u * tc::kNormMaxPer);
    TC_REQUIRE(nDims <= hd && (nDims % 2u) == 0, TC_EINVAL, "tc_qk_norm_rope: %u rotated dims of %u", nDims, hd);
    TC_REQUIRE(qIn == nullptr || qInStride >= hd, TC_EINVAL, "tc_qk_norm_rope: q row stride %u < head_dim", qInStride);
    // in place on the same buffer the rotation would read partners it has already overwritten
    TC_REQUIRE(qIn == nullptr || static_cast<const void *>(qIn) != static_cast<const void *>(qOut), TC_EINVAL,
               "tc_qk_norm_rope: q must be written out of place");
    if (seqLen == 0) return TC_OK;
    if (devPos == nullptr && static_cast<uint64_t>(pos) + seqLen > tableRows) {
        tc::setError("tc_qk_norm_rope: positions [%u, %llu) pass the %u table rows", pos,
                     (unsigned long long) pos + seqLen, tableRows);
        return TC_ECONTEXT_FULL;
    }
    const uint64_t warps = static_cast<uint64_t>(seqLen) * ((qIn ? nHeads : 0u) + (k ? nKV : 0u));
    const uint32_t blocks = static_cast<uint32_t>((warps + 7) / 8);
    tc::qkNormRopeKernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            qIn, qInStride, qOut, k, wq, wk, hd, nDims, nHeads, nKV, seqLen, pos, devPos, cosT, sinT);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}
