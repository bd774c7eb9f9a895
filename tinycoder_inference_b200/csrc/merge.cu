// merge.cu -- log-sum-exp merge of split-KV partials into the attention output.
//
// The contract is the reference's (include/gpu/GpuAttentionKernels.hpp:909-946):
// for one (token, q-head) with chunk partials (m_c, l_c, acc_c[hd]):
//   M = max_c m_c;  w_c = exp2((m_c - M) * log2e);  chunks with l_c <= 0 skipped;
//   out = sum_c w_c acc_c / sum_c w_c l_c   (0 when nothing contributed).
// One block per (head, token), 8 warps; a lane owns 4 consecutive dims per
// 128-dim group (128-bit loads).  The same kernel merges partials gathered from
// other GPUs when the context axis is split across ranks.
//
// Optional epilogue: the Q8_1 blocks of the output for the GEMV that follows
// attention (40-byte slots {fp16 d, fp16 sum, int8 q[32]}, :1068-1096).  The
// block sum is folded in the reference's order (lane = element index inside the
// block, xor butterfly 16..1) so the fp16 sum matches bit for bit on equal input.
#include "tc_common.cuh"

namespace tc {

constexpr int kMergeMaxChunks = 1024;

// Phase 1: all 256 threads read (m, l) of the active chunks at once, the block
// takes the max, and the per-chunk weights w_c = exp2((m_c - M) * log2e) (0 for
// empty chunks) land in shared memory.  Phase 2: warp w accumulates chunks
// w, w+8, ... with independent 128-bit loads (nothing in the loop depends on a
// previous load, so all of a warp's reads are in flight together -- the merge is
// a latency problem, not a bandwidth one).  Phase 3: the 8 warp sums are added.
template <int NV4>
__global__ void __launch_bounds__(256)
mergePartialsKernel(const float *__restrict__ pAcc, const float *__restrict__ pM, const float *__restrict__ pL,
                    float *__restrict__ out, uint32_t nHeads, uint32_t numChunks, uint32_t activeHost,
                    uint32_t hd, const uint32_t *__restrict__ devLens, uint32_t lenAdd, uint32_t chunkTokens,
                    uint8_t *__restrict__ q81, uint32_t chunksPerRank, uint64_t rankStride) {
    constexpr int NW = 8;
    const uint32_t head = blockIdx.x, s = blockIdx.y;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // Slot c of this (token, head): plain layout [token][head][numChunks], or -- for partials
    // gathered from several ranks -- rank c / chunksPerRank, whose block (rankStride floats
    // further on in each of the three arrays) holds [token][head][chunksPerRank].
    const uint64_t headRow = static_cast<uint64_t>(s) * nHeads + head;
    // (the plain layout takes the branch without the divisions: they would sit in front of
    // every load of a kernel whose whole cost is latency)
    auto mlOff = [&](uint32_t c) -> uint64_t {
        if (rankStride == 0) return headRow * numChunks + c;
        const uint32_t r = c / chunksPerRank;
        return static_cast<uint64_t>(r) * rankStride + headRow * chunksPerRank + (c - r * chunksPerRank);
    };
    auto accOff = [&](uint32_t c) -> uint64_t {
        if (rankStride == 0) return (headRow * numChunks + c) * hd;
        const uint32_t r = c / chunksPerRank;
        return static_cast<uint64_t>(r) * rankStride + (headRow * chunksPerRank + (c - r * chunksPerRank)) * hd;
    };
    // under programmatic dependent launch: let the next grid start its prologue, then
    // wait until the grid that wrote the partials has finished (a no-op otherwise)
    gridDepLaunch();
    gridDepWait();
    // numChunks is the slot stride; only the first `active` slots were written
    uint32_t active = activeHost < numChunks ? activeHost : numChunks;
    if (devLens != nullptr) {
        const uint32_t len = devLens[s] + lenAdd;
        const uint32_t need = (len + chunkTokens - 1) / chunkTokens;
        // never past the slots the launch that wrote the partials covered (activeHost): a device
        // length beyond the host bound the plan was built from must not pull in stale slots
        active = need < active ? need : active;
    }
    __shared__ float sw[kMergeMaxChunks], sl[kMergeMaxChunks];
    __shared__ float sred[NW];
    __shared__ float4 sacc[NW][NV4][32];
    __shared__ float sout[NV4 * 128];

    // Everything a thread needs from global memory is requested before anything is
    // consumed: the (m, l) pair of the chunks it owns in phase 1 and the first batch
    // of accumulator rows of phase 2 (their addresses do not depend on the weights),
    // so the merge costs one round trip to L2 plus arithmetic, not one per chunk.
    const uint32_t nvec = hd >> 2;
    constexpr int kBatch = 16;
    float4 a[kBatch][NV4];
    auto loadBatch = [&](uint32_t c0) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const uint32_t c = c0 + u * NW;
            const uint32_t cc = c < active ? c : (active ? active - 1 : 0);  // always a valid address
            const float4 *pac = reinterpret_cast<const float4 *>(pAcc + accOff(cc));
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const uint32_t i = lane + 32u * j;
                a[u][j] = pac[i < nvec ? i : 0];
            }
        }
    };
    if (active) loadBatch(warp);
    // ---- phase 1: max, weights, normaliser ----
    float M = kNegBig;
    for (uint32_t c = threadIdx.x; c < active; c += 256) {
        const float m = pM[mlOff(c)];
        const float lc = pL[mlOff(c)];
        sw[c] = m;
        sl[c] = lc;
        M = fmaxf(M, m);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) sred[warp] = M;
    __syncthreads();
    M = sred[0];
#pragma unroll
    for (int w2 = 1; w2 < NW; ++w2) M = fmaxf(M, sred[w2]);
    __syncthreads();
    float lsum = 0.0f;
    for (uint32_t c = threadIdx.x; c < active; c += 256) {
        const float lc = sl[c];
        const float w = lc > 0.0f ? exp2f((sw[c] - M) * kLog2e) : 0.0f;
        sw[c] = w;
        lsum = fmaf(w, lc > 0.0f ? lc : 0.0f, lsum);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    if (lane == 0) sred[warp] = lsum;
    __syncthreads();  // also publishes the weights in sw[]
    lsum = 0.0f;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) lsum += sred[w2];

    // ---- phase 2: weighted sum of the accumulators ----
    // A chunk with weight 0 (empty, possibly never written) is dropped by a select
    // after the load, never multiplied in.
    float4 acc[NV4];
#pragma unroll
    for (int j = 0; j < NV4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t c0 = warp; c0 < active; c0 += NW * kBatch) {
        if (c0 != warp) loadBatch(c0);
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const uint32_t c = c0 + u * NW;
            const float w = c < active ? sw[c < active ? c : 0] : 0.0f;
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const bool use = w != 0.0f && (lane + 32u * j) < nvec;
                const float4 v = use ? a[u][j] : make_float4(0.f, 0.f, 0.f, 0.f);
                acc[j].x = fmaf(w, v.x, acc[j].x);
                acc[j].y = fmaf(w, v.y, acc[j].y);
                acc[j].z = fmaf(w, v.z, acc[j].z);
                acc[j].w = fmaf(w, v.w, acc[j].w);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NV4; ++j) sacc[warp][j][lane] = acc[j];
    __syncthreads();
    // ---- phase 3 ----
    if (warp == 0) {
        const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
        float4 *op = reinterpret_cast<float4 *>(out + (static_cast<uint64_t>(s) * nHeads + head) * hd);
#pragma unroll
        for (int j = 0; j < NV4; ++j) {
            float4 r = sacc[0][j][lane];
#pragma unroll
            for (int w2 = 1; w2 < NW; ++w2) {
                const float4 a = sacc[w2][j][lane];
                r.x += a.x;
                r.y += a.y;
                r.z += a.z;
                r.w += a.w;
            }
            const uint32_t i = lane + 32u * j;
            if (i < nvec) {
                r = make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
                op[i] = r;
                reinterpret_cast<float4 *>(sout)[i] = r;
            }
        }
    }
    if (q81 == nullptr) return;
    __syncthreads();
    const uint32_t nBlk = hd >> 5;
    for (uint32_t b = warp; b < nBlk; b += NW) {
        const float v = sout[b * 32 + lane];
        float amax = fabsf(v), sum = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
        }
        const float d = __fdiv_rn(amax, 127.0f);
        uint8_t *blk = q81 + ((static_cast<uint64_t>(s) * nHeads + head) * nBlk + b) * 40u;
        reinterpret_cast<int8_t *>(blk + 4)[lane] =
                amax == 0.0f ? static_cast<int8_t>(0) : static_cast<int8_t>(roundf(__fdiv_rn(v, d)));
        if (lane == 0) {
            __half *ds = reinterpret_cast<__half *>(blk);
            ds[0] = __float2half(d);
            ds[1] = __float2half(sum);
        }
    }
}

// The same merge cut into slices of 4 SL4 dims: grid (head, token, hd / (4 SL4)), so that the
// accumulator rows a block has to pull through one SM's L2 port shrink from chunks x hd floats to
// chunks x 4 SL4 (at 128 chunks x 128 dims that is 64 KB against 16 KB with 32-dim slices; the merge
// sits on the critical path of a batch-1 decode step and is pure latency).  Thread t owns float4
// t % SL4 of the slice and the chunks t / SL4, t / SL4 + CL, ...; (m, l) and the weights are recomputed
// by every slice's block -- a few hundred bytes.  No Q8_1 epilogue here (that needs the whole head).
// SL4 = float4 per slice (8: 32-dim slices, 4: 16-dim slices); 256 / SL4 chunk lanes.
template <int SL4, int T>
__global__ void __launch_bounds__(T)
mergeSliceKernel(const float *__restrict__ pAcc, const float *__restrict__ pM, const float *__restrict__ pL,
                 float *__restrict__ out, uint32_t nHeads, uint32_t numChunks, uint32_t activeHost, uint32_t hd,
                 const uint32_t *__restrict__ devLens, uint32_t lenAdd, uint32_t chunkTokens, uint32_t chunksPerRank,
                 uint64_t rankStride) {
    constexpr int NW = T / 32;
    const uint32_t head = blockIdx.x, s = blockIdx.y, slice = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    constexpr uint32_t CL = T / SL4;  // chunk lanes
    const uint32_t v4 = threadIdx.x % SL4, cl = threadIdx.x / SL4;
    const uint64_t headRow = static_cast<uint64_t>(s) * nHeads + head;
    auto mlOff = [&](uint32_t c) -> uint64_t {
        if (rankStride == 0) return headRow * numChunks + c;
        const uint32_t r = c / chunksPerRank;
        return static_cast<uint64_t>(r) * rankStride + headRow * chunksPerRank + (c - r * chunksPerRank);
    };
    auto accOff = [&](uint32_t c) -> uint64_t {
        if (rankStride == 0) return (headRow * numChunks + c) * hd;
        const uint32_t r = c / chunksPerRank;
        return static_cast<uint64_t>(r) * rankStride + (headRow * chunksPerRank + (c - r * chunksPerRank)) * hd;
    };
    gridDepLaunch();
    gridDepWait();
    uint32_t active = activeHost < numChunks ? activeHost : numChunks;
    if (devLens != nullptr) {
        const uint32_t len = devLens[s] + lenAdd;
        const uint32_t need = (len + chunkTokens - 1) / chunkTokens;
        // never past the slots the launch that wrote the partials covered (activeHost): a device
        // length beyond the host bound the plan was built from must not pull in stale slots
        active = need < active ? need : active;
    }
    __shared__ float sw[kMergeMaxChunks], sl[kMergeMaxChunks];
    __shared__ float sred[NW];
    __shared__ float4 sacc[NW][SL4];

    constexpr int kB = 256 / CL;  // kB x CL chunk lanes = 256 chunks per batch
    float4 a[kB];
    auto loadBatch = [&](uint32_t c0) {
#pragma unroll
        for (int u = 0; u < kB; ++u) {
            const uint32_t c = c0 + cl + CL * u;
            // lanes past the live chunks load nothing (their weight is zero below)
            if (c0 + CL * u < active) {
                const uint32_t cc = c < active ? c : active - 1;  // always a valid address
                a[u] = reinterpret_cast<const float4 *>(pAcc + accOff(cc) + 4u * SL4 * slice)[v4];
            } else {
                a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };
    if (active) loadBatch(0);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float lsum = 0.0f;
    if (active <= 64u) {
        // Up to 64 chunks (the usual case): every warp works out the maximum, the weights and the row
        // sum for itself -- lane c holds chunks c and c + 32 -- so nothing goes through shared memory
        // and no block-wide barrier stands between the loads and the weighted sum.
        float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
        if (lane < active) m0 = pM[mlOff(lane)], l0 = pL[mlOff(lane)];
        if (lane + 32u < active) m1 = pM[mlOff(lane + 32u)], l1 = pL[mlOff(lane + 32u)];
        float M = fmaxf(m0, m1);
#pragma unroll
        for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w0 = l0 > 0.0f ? exp2f((m0 - M) * kLog2e) : 0.0f;
        const float w1 = l1 > 0.0f ? exp2f((m1 - M) * kLog2e) : 0.0f;
        lsum = fmaf(w0, l0 > 0.0f ? l0 : 0.0f, w1 * (l1 > 0.0f ? l1 : 0.0f));
#pragma unroll
        for (int o = 16; o; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
#pragma unroll
        for (int u = 0; u < static_cast<int>(64u / CL); ++u) {
            const uint32_t c = cl + CL * u;  // its weight sits in lane c % 32, slot c / 32
            const float wa = __shfl_sync(0xffffffffu, w0, c & 31u), wb = __shfl_sync(0xffffffffu, w1, c & 31u);
            const float w = c < 32u ? wa : wb;
            const float4 v = w != 0.0f ? a[u] : make_float4(0.f, 0.f, 0.f, 0.f);  // empty chunk: select, never multiply
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
        }
    } else {
        float M = kNegBig;
        for (uint32_t c = threadIdx.x; c < active; c += T) {
            const float m = pM[mlOff(c)];
            sw[c] = m;
            sl[c] = pL[mlOff(c)];
            M = fmaxf(M, m);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        if (lane == 0) sred[warp] = M;
        __syncthreads();
        M = sred[0];
#pragma unroll
        for (int w2 = 1; w2 < NW; ++w2) M = fmaxf(M, sred[w2]);
        __syncthreads();
        for (uint32_t c = threadIdx.x; c < active; c += T) {
            const float lc = sl[c];
            const float w = lc > 0.0f ? exp2f((sw[c] - M) * kLog2e) : 0.0f;
            sw[c] = w;
            lsum = fmaf(w, lc > 0.0f ? lc : 0.0f, lsum);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
        if (lane == 0) sred[warp] = lsum;
        __syncthreads();  // also publishes the weights
        lsum = 0.0f;
#pragma unroll
        for (int w2 = 0; w2 < NW; ++w2) lsum += sred[w2];
        for (uint32_t c0 = 0; c0 < active; c0 += CL * kB) {
            if (c0) loadBatch(c0);
#pragma unroll
            for (int u = 0; u < kB; ++u) {
                const uint32_t c = c0 + cl + CL * u;
                const float w = c < active ? sw[c < active ? c : 0] : 0.0f;
                const float4 v = w != 0.0f ? a[u] : make_float4(0.f, 0.f, 0.f, 0.f);  // empty chunk: select, never multiply
                acc.x = fmaf(w, v.x, acc.x);
                acc.y = fmaf(w, v.y, acc.y);
                acc.z = fmaf(w, v.z, acc.z);
                acc.w = fmaf(w, v.w, acc.w);
            }
        }
    }  // more than 64 chunks
    // a warp holds 32 / SL4 chunk lanes x SL4 float4: fold the chunk lanes, then the warps
#pragma unroll
    for (int o = SL4; o <= 16; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (lane < SL4) sacc[warp][lane] = acc;
    __syncthreads();
    if (threadIdx.x < SL4) {
        float4 r = sacc[0][threadIdx.x];
#pragma unroll
        for (int w2 = 1; w2 < NW; ++w2) {
            const float4 x = sacc[w2][threadIdx.x];
            r.x += x.x;
            r.y += x.y;
            r.z += x.z;
            r.w += x.w;
        }
        const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
        reinterpret_cast<float4 *>(out + headRow * hd + 4u * SL4 * slice)[threadIdx.x] =
                make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
    }
}

int launchMerge(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t seqLen,
                uint32_t nHeads, uint32_t numChunks, uint32_t activeHost, uint32_t hd, const uint32_t *devLens,
                uint32_t lenAdd, uint32_t chunkTokens, uint8_t *q81, bool pdl, cudaStream_t st,
                uint32_t chunksPerRank, uint64_t rankStride) {
    if (chunksPerRank == 0) chunksPerRank = numChunks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nHeads, seqLen);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    // The sliced form (a block per head and 32-dim slice) is the faster merge in plain stream order.
    // Under programmatic dependent launch its blocks are resident next to the decode blocks they wait
    // for: with one sequence that still wins (7B shape, 32768 rows: 11.7 us per layer against 12.5 with
    // a block per head; 131072 rows of the 32B shape 48.1 against 49.2), with a batch of sequences the
    // 4x as many blocks get in the way (batch 8: 49.4 against 46.1 us; 64 ragged sequences 201 against
    // 190), so a batch keeps the block-per-head form there.
    if (q81 == nullptr && (!pdl || static_cast<uint64_t>(nHeads) * seqLen <= 64u)) {
        // one sequence: 16-dim slices, twice the blocks (7B shape at 32768 rows: 11.36 us per layer
        // against 11.67 with 32-dim slices, 11.38 with 8-dim, 12.17 with 4-dim ones)
        if (static_cast<uint64_t>(nHeads) * seqLen <= 64u) {
            cfg.gridDim = dim3(nHeads, seqLen, hd / 16u);
            TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergeSliceKernel<4, 256>, pAcc, pM, pL, out, nHeads, numChunks, activeHost, hd,
                                          devLens, lenAdd, chunkTokens, chunksPerRank, rankStride));
            return TC_OK;
        }
        cfg.gridDim = dim3(nHeads, seqLen, hd / 32u);
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergeSliceKernel<8, 256>, pAcc, pM, pL, out, nHeads, numChunks, activeHost, hd,
                                      devLens, lenAdd, chunkTokens, chunksPerRank, rankStride));
        return TC_OK;
    }
    if (hd <= 128)
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergePartialsKernel<1>, pAcc, pM, pL, out, nHeads, numChunks,
                                      activeHost, hd, devLens, lenAdd, chunkTokens, q81, chunksPerRank, rankStride));
    else
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergePartialsKernel<2>, pAcc, pM, pL, out, nHeads, numChunks,
                                      activeHost, hd, devLens, lenAdd, chunkTokens, q81, chunksPerRank, rankStride));
    return TC_OK;
}

}  // namespace tc

extern "C" {

int tc_attn_merge_partials(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t seqLen,
                           uint32_t nHeads, uint32_t numChunks, uint32_t hd, uint8_t *q81Out,
                           tc_stream stream) {
    TC_REQUIRE(pAcc && pM && pL && out, TC_EINVAL, "tc_attn_merge_partials: null pointer");
    TC_REQUIRE(hd >= 32 && hd <= 256 && (hd % 32u) == 0, TC_EUNSUPPORTED,
               "tc_attn_merge_partials: hd=%u must be a multiple of 32 in [32, 256]", hd);
    TC_REQUIRE(numChunks >= 1 && nHeads >= 1, TC_EINVAL, "tc_attn_merge_partials: empty shape");
    TC_REQUIRE(numChunks <= tc::kMergeMaxChunks, TC_EUNSUPPORTED, "tc_attn_merge_partials: %u chunks (max %d)",
               numChunks, tc::kMergeMaxChunks);
    TC_REQUIRE(seqLen <= 65535, TC_EUNSUPPORTED, "tc_attn_merge_partials: seqLen %u > 65535", seqLen);
    if (seqLen == 0) return TC_OK;
    return tc::launchMerge(pAcc, pM, pL, out, seqLen, nHeads, numChunks, numChunks, hd, nullptr, 0, 1, q81Out,
                           false, static_cast<cudaStream_t>(stream), 0, 0);
}

int tc_attn_merge_gathered(const float *gathered, float *out, uint32_t nHeads, uint32_t ranks,
                           uint32_t chunksPerRank, uint32_t hd, tc_stream stream) {
    TC_REQUIRE(gathered && out, TC_EINVAL, "tc_attn_merge_gathered: null pointer");
    TC_REQUIRE(hd >= 32 && hd <= 256 && (hd % 32u) == 0, TC_EUNSUPPORTED, "tc_attn_merge_gathered: hd=%u", hd);
    TC_REQUIRE(ranks >= 1 && chunksPerRank >= 1 && nHeads >= 1, TC_EINVAL, "tc_attn_merge_gathered: empty shape");
    TC_REQUIRE(static_cast<uint64_t>(ranks) * chunksPerRank <= tc::kMergeMaxChunks, TC_EUNSUPPORTED,
               "tc_attn_merge_gathered: %u x %u partials (max %d)", ranks, chunksPerRank, tc::kMergeMaxChunks);
    const uint64_t ml = static_cast<uint64_t>(nHeads) * chunksPerRank;
    const uint64_t block = ml * hd + 2 * ml;  // one rank's [acc | m | l]
    return tc::launchMerge(gathered, gathered + ml * hd, gathered + ml * hd + ml, out, 1, nHeads,
                           ranks * chunksPerRank, ranks * chunksPerRank, hd, nullptr, 0, 1, nullptr, false,
                           static_cast<cudaStream_t>(stream), chunksPerRank, block);
}

int tc_attn_workspace_bytes(uint32_t batch, uint32_t nHeads, uint32_t hd, uint32_t numChunks, size_t *accBytes,
                            size_t *mBytes, size_t *lBytes) {
    TC_REQUIRE(accBytes && mBytes && lBytes, TC_EINVAL, "tc_attn_workspace_bytes: null output");
    const size_t n = static_cast<size_t>(batch) * nHeads * numChunks;
    *accBytes = n * hd * sizeof(float);
    *mBytes = n * sizeof(float);
    *lBytes = n * sizeof(float);
    return TC_OK;
}

}  // extern "C"
