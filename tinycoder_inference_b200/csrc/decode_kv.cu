// decode_kv.cu -- grouped-query attention over an f32 KV cache: split-KV decode
// and, with query rows as columns, the unsplit causal kernel.
//
// What it replaces: launchDecodeAttentionSplit / kWarpAttentionSplit +
// kAttnCombinePartial(W4) and kWarpAttention / kWarpAttentionPos of the reference
// (include/gpu/GpuAttentionKernels.hpp:211-272, 537-599, 625-766, 909-1230), and
// (the fp16 cache, kvHalf, is served by the twin kernel in decode_kv16.cu) and
// the f32 twins kQ35WarpAttention / kQ35StoreKV-fed split path of the hybrid
// models (include/gpu/GpuQwen35Kernels.hpp:2437-2492): score = dot(q, k) *
// invSqrt, online softmax with exp2, out = sum p v / sum p, all f32.
//
// Same skeleton as the int8 kernel (decode_i8.cu): grid = (chunks, kv-head groups,
// sequences), one TMA producer warp feeding an mbarrier ring with 128-byte
// swizzled [tokens][32 floats] boxes, consumer warps that own a (kv head, 16
// token) tile per stage and serve every q head of that kv head, partials in the
// reference's layout, merge by merge.cu.  The arithmetic differs: K and V are
// arbitrary f32, so QK^T and PV run as 3xTF32 tensor-core products
// (mma.sync.m16n8k8: x = hi + lo with both parts tf32; hi*hi + lo*hi + hi*lo keeps
// ~21 mantissa bits and the full f32 exponent range, f32 accumulation).  f32 rows
// are four times the bytes of int8 rows, so per byte this costs a quarter of the
// instructions and the kernel stays HBM-bound.
#include "decode_shared.cuh"

namespace tc {

struct DecodeKvParams {
    const float *q;
    float *out;
    float *pAcc, *pM, *pL;
    const uint32_t *devPos;  // nullable: position read at kernel time
    uint64_t totalRows;
    uint32_t lenHost;        // rows to attend in heads mode when devPos == nullptr
    uint32_t nHeads, nKV, group;
    uint32_t colBase;  // heads mode: the 8 MMA columns are q heads colBase .. colBase + 7 of the kv head
    uint32_t chunkTokens, numChunks;
    uint32_t rowsMode, qRows, cachePos;  // rows mode: see decode_i8.cu
    float invSqrt;
    int directOut;
    unsigned int *err;
};

template <int HD, int NW, int HPC, int NSTAGE>
struct DecodeKvSmem {
    static constexpr int NB = HD / 32;                  // 32-float boxes per row
    static constexpr int kRows = NW * 16;               // (token, head) rows per stage
    static constexpr int T = kRows / HPC;               // tokens per stage
    static constexpr int kTileBytes = kRows * HD * 4;   // K (or V) bytes per stage
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kBarOffset = NSTAGE * kStageBytes;
    static constexpr int kTotal = kBarOffset + 2 * NSTAGE * 8 + 1024;
    static_assert(T % 8 == 0 && T <= 256, "box rows");
    static_assert(NW % HPC == 0, "warps per head");
};

__device__ __forceinline__ void splitTf32(float x, uint32_t &hi, uint32_t &lo) {
    hi = toTf32(x);
    lo = toTf32(x - __uint_as_float(hi));
}

template <int HD, int NW, int HPC, int NSTAGE>
__global__ void __launch_bounds__((NW + 1) * 32, 1)
decodeKvKernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const DecodeKvParams p) {
    using L = DecodeKvSmem<HD, NW, HPC, NSTAGE>;
    constexpr int T = L::T, NB = L::NB;
    constexpr int NSUB = NW / HPC;
    constexpr int KS = HD / 8;   // tf32 k-steps of the QK product
    constexpr int MTO = HD / 16;  // 16-dim output tiles

    const uint32_t chunk = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *fullBar = reinterpret_cast<uint64_t *>(smem + L::kBarOffset);
    uint64_t *emptyBar = fullBar + NSTAGE;
    __shared__ float pScratch[NW][16 * 8];

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&fullBar[s], 1);
            mbarInit(&emptyBar[s], NW);
        }
        fenceBarrierInit();
        tmaPrefetchDesc(&tmK);
        tmaPrefetchDesc(&tmV);
    }
    __syncthreads();

    uint32_t pos = p.devPos ? p.devPos[0] : 0u;
    uint32_t len;
    uint32_t rowsPos = p.cachePos;
    if (p.rowsMode) {
        if (p.devPos) rowsPos = pos;
        len = rowsPos + min(p.qRows, b * 8u + 8u);
    } else {
        len = p.devPos ? pos + 1u : p.lenHost;
    }
    const uint32_t t0 = chunk * p.chunkTokens;
    if (t0 >= len) return;
    const uint32_t t1 = min(len, t0 + p.chunkTokens);
    const uint32_t nTiles = (t1 - t0 + T - 1) / T;
    const uint32_t kvHead0 = p.rowsMode ? hg / p.group : hg * HPC;

    if (warp == NW) {
        if (lane == 0) {
            for (uint32_t it = 0; it < nTiles; ++it) {
                const uint32_t s = it % NSTAGE;
                if (it >= NSTAGE) {
                    if (!mbarWaitClock(&emptyBar[s], ((it / NSTAGE) - 1) & 1, p.err, kDevErrEmptyWait)) break;
                }
                uint8_t *st = smem + s * L::kStageBytes;
                const int row = static_cast<int>(t0 + it * T);
                mbarExpectTx(&fullBar[s], L::kStageBytes);
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
#pragma unroll
                    for (int bx = 0; bx < NB; ++bx) {
                        const int sub = (h * NB + bx) * T * 128;
                        tmaLoad3D(st + sub, &tmK, &fullBar[s], 32 * bx, kvHead0 + h, row);
                        tmaLoad3D(st + L::kTileBytes + sub, &tmV, &fullBar[s], 32 * bx, kvHead0 + h, row);
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t hL = warp % HPC, sub = warp / HPC;
    const uint32_t kvHead = kvHead0 + hL;
    auto colValid = [&](uint32_t j) { return p.rowsMode ? (b * 8u + j < p.qRows) : (p.colBase + j < p.group); };
    auto colIndex = [&](uint32_t j) -> size_t {
        return p.rowsMode ? (static_cast<size_t>(b) * 8u + j) * p.nHeads + hg
                          : static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + j;
    };
    auto colLen = [&](uint32_t j) { return p.rowsMode ? min(t1, rowsPos + b * 8u + j + 1u) : t1; };

    // q of column n = g as the B operand: k slot t / t+4 of step (bx, h, e) is
    // dim 32bx + 8t + 4h + 2e / +1 -- the order the swizzled 16-byte loads deliver.
    uint32_t qhi[KS][2], qlo[KS][2];
    {
        const bool valid = colValid(g);
        const float *qp = p.q + colIndex(valid ? g : 0) * HD;
#pragma unroll
        for (int bx = 0; bx < NB; ++bx)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float4 v = valid ? __ldg(reinterpret_cast<const float4 *>(qp + 32 * bx + 8 * t + 4 * h))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                const int ks = (bx * 2 + h) * 2;
                splitTf32(v.x, qhi[ks][0], qlo[ks][0]);
                splitTf32(v.y, qhi[ks][1], qlo[ks][1]);
                splitTf32(v.z, qhi[ks + 1][0], qlo[ks + 1][0]);
                splitTf32(v.w, qhi[ks + 1][1], qlo[ks + 1][1]);
            }
    }
    const float cs = p.invSqrt * kLog2e;
    const uint32_t len0 = colLen(2 * t), len1 = colLen(2 * t + 1);

    float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
    float o[MTO][4];
#pragma unroll
    for (int i = 0; i < MTO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float *pS = pScratch[warp];

    for (uint32_t it = 0; it < nTiles; ++it) {
        const uint32_t s = it % NSTAGE;
        if (!mbarWaitClock(&fullBar[s], (it / NSTAGE) & 1, p.err, kDevErrFullWait)) break;
        const uint8_t *st = smem + s * L::kStageBytes;
        const uint32_t tokA = t0 + it * T + sub * 16 + g, tokB = tokA + 8;

        // ---- S^T = K . Q^T (16 tokens x 8 columns), 3xTF32 ----
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) {
            const uint8_t *kT = st + ((hL * NB + bx) * T + sub * 16) * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t off = ((2 * t + h) ^ g) << 4;
                const float4 xa = *reinterpret_cast<const float4 *>(kT + g * 128 + off);
                const float4 xb = *reinterpret_cast<const float4 *>(kT + (g + 8) * 128 + off);
                const int ks = (bx * 2 + h) * 2;
                {
                    uint32_t h0, l0_, h1, l1_, h2, l2_, h3, l3_;
                    splitTf32(xa.x, h0, l0_);
                    splitTf32(xb.x, h1, l1_);
                    splitTf32(xa.y, h2, l2_);
                    splitTf32(xb.y, h3, l3_);
                    mmaTf32(sa, h0, h1, h2, h3, qhi[ks][0], qhi[ks][1]);
                    mmaTf32(sb, l0_, l1_, l2_, l3_, qhi[ks][0], qhi[ks][1]);
                    mmaTf32(sb, h0, h1, h2, h3, qlo[ks][0], qlo[ks][1]);
                }
                {
                    uint32_t h0, l0_, h1, l1_, h2, l2_, h3, l3_;
                    splitTf32(xa.z, h0, l0_);
                    splitTf32(xb.z, h1, l1_);
                    splitTf32(xa.w, h2, l2_);
                    splitTf32(xb.w, h3, l3_);
                    mmaTf32(sa, h0, h1, h2, h3, qhi[ks + 1][0], qhi[ks + 1][1]);
                    mmaTf32(sb, l0_, l1_, l2_, l3_, qhi[ks + 1][0], qhi[ks + 1][1]);
                    mmaTf32(sb, h0, h1, h2, h3, qlo[ks + 1][0], qlo[ks + 1][1]);
                }
            }
        }
        const float s00 = tokA < len0 ? (sa[0] + sb[0]) * cs : -INFINITY;
        const float s01 = tokA < len1 ? (sa[1] + sb[1]) * cs : -INFINITY;
        const float s10 = tokB < len0 ? (sa[2] + sb[2]) * cs : -INFINITY;
        const float s11 = tokB < len1 ? (sa[3] + sb[3]) * cs : -INFINITY;
        float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1)) {
            const float a0 = fastExp2(m0 - mn0), a1 = fastExp2(m1 - mn1);
#pragma unroll
            for (int i = 0; i < MTO; ++i) {
                o[i][0] *= a0;
                o[i][1] *= a1;
                o[i][2] *= a0;
                o[i][3] *= a1;
            }
            l0 *= a0;
            l1 *= a1;
            m0 = mn0;
            m1 = mn1;
        }
        const float p00 = fastExp2(s00 - m0), p01 = fastExp2(s01 - m1);
        const float p10 = fastExp2(s10 - m0), p11 = fastExp2(s11 - m1);
        l0 += p00 + p10;
        l1 += p01 + p11;
        // rows past the chunk may hold anything (stale rows, other sequences): a 0
        // probability must not meet a NaN/Inf value, so those V rows are zeroed below
        // transpose p to the B layout through the warp's scratch: [token][column]
        *reinterpret_cast<float2 *>(pS + g * 8 + 2 * t) = make_float2(p00, p01);
        *reinterpret_cast<float2 *>(pS + (g + 8) * 8 + 2 * t) = make_float2(p10, p11);
        __syncwarp();
        uint32_t phi[2][2], plo[2][2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            splitTf32(pS[(8 * kk + 2 * t) * 8 + g], phi[kk][0], plo[kk][0]);
            splitTf32(pS[(8 * kk + 2 * t + 1) * 8 + g], phi[kk][1], plo[kk][1]);
        }
        __syncwarp();
        // ---- O^T += V^T . P^T (HD dims x 8 columns), 3xTF32 ----
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const uint32_t ra = 8 * kk + 2 * t, rb = ra + 1;  // token rows of k slots t and t+4
            const bool okA = t0 + it * T + sub * 16 + ra < t1, okB = t0 + it * T + sub * 16 + rb < t1;
#pragma unroll
            for (int bx = 0; bx < NB; ++bx) {
                const uint8_t *vT = st + L::kTileBytes + ((hL * NB + bx) * T + sub * 16) * 128;
                float4 xa = *reinterpret_cast<const float4 *>(vT + ra * 128 + ((g ^ (ra & 7u)) << 4));
                float4 xb = *reinterpret_cast<const float4 *>(vT + rb * 128 + ((g ^ (rb & 7u)) << 4));
                if (!okA) xa = make_float4(0.f, 0.f, 0.f, 0.f);
                if (!okB) xb = make_float4(0.f, 0.f, 0.f, 0.f);
                {
                    uint32_t h0, l0_, h1, l1_, h2, l2_, h3, l3_;
                    splitTf32(xa.x, h0, l0_);
                    splitTf32(xa.y, h1, l1_);
                    splitTf32(xb.x, h2, l2_);
                    splitTf32(xb.y, h3, l3_);
                    mmaTf32(o[2 * bx], h0, h1, h2, h3, phi[kk][0], phi[kk][1]);
                    mmaTf32(o[2 * bx], l0_, l1_, l2_, l3_, phi[kk][0], phi[kk][1]);
                    mmaTf32(o[2 * bx], h0, h1, h2, h3, plo[kk][0], plo[kk][1]);
                }
                {
                    uint32_t h0, l0_, h1, l1_, h2, l2_, h3, l3_;
                    splitTf32(xa.z, h0, l0_);
                    splitTf32(xa.w, h1, l1_);
                    splitTf32(xb.z, h2, l2_);
                    splitTf32(xb.w, h3, l3_);
                    mmaTf32(o[2 * bx + 1], h0, h1, h2, h3, phi[kk][0], phi[kk][1]);
                    mmaTf32(o[2 * bx + 1], l0_, l1_, l2_, l3_, phi[kk][0], phi[kk][1]);
                    mmaTf32(o[2 * bx + 1], h0, h1, h2, h3, plo[kk][0], plo[kk][1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbarArrive(&emptyBar[s]);
    }

    // ---- fold the consumer warps of each kv head, write the chunk partial ----
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    namedBarSync(1, NW * 32);
    float *scr = reinterpret_cast<float *>(smem);
    constexpr int kWarpScr = 8 * HD + 16;
    float *wO = scr + warp * kWarpScr;
#pragma unroll
    for (int bx = 0; bx < NB; ++bx) {
        const int d = 32 * bx + 4 * g;
        *reinterpret_cast<float4 *>(wO + (2 * t) * HD + d) =
                make_float4(o[2 * bx][0], o[2 * bx][2], o[2 * bx + 1][0], o[2 * bx + 1][2]);
        *reinterpret_cast<float4 *>(wO + (2 * t + 1) * HD + d) =
                make_float4(o[2 * bx][1], o[2 * bx][3], o[2 * bx + 1][1], o[2 * bx + 1][3]);
    }
    if (g == 0) {
        wO[8 * HD + 2 * t] = m0;
        wO[8 * HD + 2 * t + 1] = m1;
        wO[8 * HD + 8 + 2 * t] = l0;
        wO[8 * HD + 8 + 2 * t + 1] = l1;
    }
    namedBarSync(1, NW * 32);
    constexpr int NV = HD / 4;  // float4 per output vector
    for (uint32_t idx = threadIdx.x; idx < HPC * 8 * NV; idx += NW * 32) {
        const uint32_t d4 = idx % NV, j = (idx / NV) & 7u, h = idx / (NV * 8);
        if (!colValid(j)) continue;
        float M = kNegBig;
#pragma unroll
        for (int sb2 = 0; sb2 < NSUB; ++sb2) M = fmaxf(M, scr[(sb2 * HPC + h) * kWarpScr + 8 * HD + j]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float lsum = 0.0f;
#pragma unroll
        for (int sb2 = 0; sb2 < NSUB; ++sb2) {
            const float *w = scr + (sb2 * HPC + h) * kWarpScr;
            const float wgt = fastExp2(w[8 * HD + j] - M);
            lsum += wgt * w[8 * HD + 8 + j];
            const float4 a = *reinterpret_cast<const float4 *>(w + j * HD + 4 * d4);
            acc.x = fmaf(wgt, a.x, acc.x);
            acc.y = fmaf(wgt, a.y, acc.y);
            acc.z = fmaf(wgt, a.z, acc.z);
            acc.w = fmaf(wgt, a.w, acc.w);
        }
        const size_t oidx = p.rowsMode ? (static_cast<size_t>(b) * 8u + j) * p.nHeads + hg
                                       : static_cast<size_t>(b) * p.nHeads + (kvHead0 + h) * p.group + p.colBase + j;
        if (p.directOut) {
            const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
            *reinterpret_cast<float4 *>(p.out + oidx * HD + 4 * d4) =
                    make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else {
            const size_t pidx = oidx * p.numChunks + chunk;
            *reinterpret_cast<float4 *>(p.pAcc + pidx * HD + 4 * d4) = acc;
            if (d4 == 0) {
                p.pM[pidx] = M > -1e29f ? M * 0.6931471805599453f : kNegBig;
                p.pL[pidx] = lsum;
            }
        }
    }
}

template <int HD, int NW, int HPC>
static int launchKv(const CUtensorMap &tmK, const CUtensorMap &tmV, const DecodeKvParams &prm, dim3 grid,
                    cudaStream_t st) {
    constexpr int NSTAGE = 3;
    using L = DecodeKvSmem<HD, NW, HPC, NSTAGE>;
    auto kern = decodeKvKernel<HD, NW, HPC, NSTAGE>;
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attrDone[dev] = true;
    }
    kern<<<grid, (NW + 1) * 32, L::kTotal, st>>>(tmK, tmV, prm);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

template <int HD, int NW>
static int launchKvHpc(uint32_t hpc, const CUtensorMap &tmK, const CUtensorMap &tmV, const DecodeKvParams &prm,
                       dim3 grid, cudaStream_t st) {
    if constexpr (NW % 4 == 0) {
        if (hpc == 4) return launchKv<HD, NW, 4>(tmK, tmV, prm, grid, st);
    }
    if (hpc == 2) return launchKv<HD, NW, 2>(tmK, tmV, prm, grid, st);
    return launchKv<HD, NW, 1>(tmK, tmV, prm, grid, st);
}

static int kvMaps(const void *kvK, const void *kvV, uint32_t nKV, uint32_t hd, uint64_t totalRows, uint32_t boxRows,
                  CUtensorMap *tmK, CUtensorMap *tmV) {
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.rank = 3;
    key.elemBytes = 4;
    key.swizzle = 3;
    key.dims[0] = hd;
    key.dims[1] = nKV;
    key.dims[2] = totalRows;
    key.strides[0] = static_cast<uint64_t>(hd) * 4;
    key.strides[1] = static_cast<uint64_t>(nKV) * hd * 4;
    key.box[0] = 32;
    key.box[1] = 1;
    key.box[2] = boxRows;
    key.base = kvK;
    int rc = getTensorMap(key, tmK);
    if (rc != TC_OK) return rc;
    key.base = kvV;
    return getTensorMap(key, tmV);
}

static int kvCommonChecks(const char *who, const float *q, const void *kvK, const void *kvV, float *out,
                          uint32_t nHeads, uint32_t nKV, uint32_t hd, uint64_t totalRows, int kvHalf) {
    TC_REQUIRE(q && kvK && kvV && out, TC_EINVAL, "%s: null pointer", who);
    TC_REQUIRE(hd == 64 || hd == 128 || (hd == 256 && !kvHalf), TC_EUNSUPPORTED,
               "%s: head_dim %u (built for 64, 128 and -- f32 cache only -- 256)", who, hd);
    TC_REQUIRE(nKV > 0 && nHeads % nKV == 0, TC_EINVAL, "%s: nHeads %u not a multiple of nKV %u", who, nHeads, nKV);
    TC_REQUIRE(nHeads / nKV <= 64, TC_EUNSUPPORTED, "%s: %u q heads per kv head (built for <= 64)", who, nHeads / nKV);
    TC_REQUIRE(totalRows >= 1 && totalRows < (1ull << 31), TC_EUNSUPPORTED, "%s: cache of %llu rows", who,
               (unsigned long long) totalRows);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(kvK) | reinterpret_cast<uintptr_t>(kvV) | reinterpret_cast<uintptr_t>(q) |
                 reinterpret_cast<uintptr_t>(out)) & 15u) == 0,
               TC_EINVAL, "%s: q/out/K/V need 16-byte alignment", who);
    return TC_OK;
}

// rows mode: causal attention of seqLen query rows (row s sees [0, cachePos + s])
static int prefillKv(const float *q, const void *kvK, const void *kvV, float *out, uint32_t seqLen, uint32_t nHeads,
                     uint32_t nKV, uint32_t hd, uint32_t cachePos, const uint32_t *devPos, uint64_t totalRows,
                     float invSqrt, int kvHalf, cudaStream_t st) {
    int rc = kvCommonChecks("prefill_kv", q, kvK, kvV, out, nHeads, nKV, hd, totalRows, kvHalf);
    if (rc != TC_OK) return rc;
    if (seqLen == 0) return TC_OK;
    if (devPos == nullptr && static_cast<uint64_t>(cachePos) + seqLen > totalRows) {
        setError("prefill_kv: rows [%u, %llu) pass the cache of %llu rows", cachePos,
                 (unsigned long long) cachePos + seqLen, (unsigned long long) totalRows);
        return TC_ECONTEXT_FULL;
    }
    const uint32_t rowBlocks = (seqLen + 7) / 8;
    TC_REQUIRE(rowBlocks <= 65535 && nHeads <= 65535, TC_EUNSUPPORTED, "prefill_kv: %u rows x %u heads", seqLen, nHeads);
    if (kvHalf)
        return prefillKv16(q, kvK, kvV, out, seqLen, nHeads, nKV, hd, cachePos, devPos, totalRows, invSqrt, st);
    const uint32_t nw = hd == 64 ? 8u : (hd == 128 ? 4u : 2u);  // consumer warps: 16 rows of K and V each per stage
    CUtensorMap tmK, tmV;
    rc = kvMaps(kvK, kvV, nKV, hd, totalRows, nw * 16u, &tmK, &tmV);
    if (rc != TC_OK) return rc;
    DecodeKvParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.q = q;
    prm.out = out;
    prm.devPos = devPos;
    prm.totalRows = totalRows;
    prm.nHeads = nHeads;
    prm.nKV = nKV;
    prm.group = nHeads / nKV;
    prm.chunkTokens = 0xffffff00u;
    prm.numChunks = 1;
    prm.rowsMode = 1;
    prm.qRows = seqLen;
    prm.cachePos = cachePos;
    prm.invSqrt = invSqrt;
    prm.directOut = 1;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "prefill_kv: no device error word");
    dim3 grid(1, nHeads, rowBlocks);
    if (hd == 64) return launchKv<64, 8, 1>(tmK, tmV, prm, grid, st);
    if (hd == 256) return launchKv<256, 2, 1>(tmK, tmV, prm, grid, st);
    return launchKv<128, 4, 1>(tmK, tmV, prm, grid, st);
}

}  // namespace tc

extern "C" {

int tc_attn_prefill_kv(const float *q, const void *kvK, const void *kvV, float *out, uint32_t seqLen,
                       uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos, const uint32_t *devPos,
                       uint64_t totalRows, float invSqrt, int kvHalf, tc_stream stream) {
    return tc::prefillKv(q, kvK, kvV, out, seqLen, nHeads, nKV, hd, cachePos, devPos, totalRows, invSqrt, kvHalf,
                         static_cast<cudaStream_t>(stream));
}

int tc_attn_decode_kv(const float *q, const void *kvK, const void *kvV, float *attnOut, float *pAcc, float *pM,
                      float *pL, uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t pos,
                      const uint32_t *devPos, uint64_t totalRows, uint32_t numChunks, uint32_t chunkSize,
                      float invSqrt, int kvHalf, uint8_t *q81Out, tc_stream stream) {
    using namespace tc;
    (void) chunkSize;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (seqLen != 1) {
        // the reference only splits single-token decode; several rows take the causal kernel
        TC_REQUIRE(q81Out == nullptr, TC_EUNSUPPORTED, "tc_attn_decode_kv: Q8_1 output needs seqLen == 1");
        return prefillKv(q, kvK, kvV, attnOut, seqLen, nHeads, nKV, hd, pos, devPos, totalRows, invSqrt, kvHalf, st);
    }
    int rc = kvCommonChecks("tc_attn_decode_kv", q, kvK, kvV, attnOut, nHeads, nKV, hd, totalRows, kvHalf);
    if (rc != TC_OK) return rc;
    TC_REQUIRE(static_cast<uint64_t>(pos) + 1 <= totalRows, TC_ECONTEXT_FULL,
               "tc_attn_decode_kv: position %u is outside the cache of %llu rows", pos,
               (unsigned long long) totalRows);
    TC_REQUIRE(numChunks >= 1, TC_EWORKSPACE, "tc_attn_decode_kv: no chunk slots");
    if (kvHalf)
        return decodeKv16(q, kvK, kvV, attnOut, pAcc, pM, pL, nHeads, nKV, hd, pos, devPos, totalRows, numChunks,
                          invSqrt, q81Out, st);
    const uint32_t nw = hd == 64 ? 8u : (hd == 128 ? 4u : 2u);
    DecodePlan pl = planDecode(1, nKV, pos + 1, numChunks, nw * 16u, true, nw >= 4u ? 4u : 2u);
    const bool direct = pl.chunksPerSeq == 1 && q81Out == nullptr;
    if (!direct) TC_REQUIRE(pAcc && pM && pL, TC_EWORKSPACE, "tc_attn_decode_kv: partial buffers are required");
    CUtensorMap tmK, tmV;
    rc = kvMaps(kvK, kvV, nKV, hd, totalRows, pl.tileTokens, &tmK, &tmV);
    if (rc != TC_OK) return rc;
    DecodeKvParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.q = q;
    prm.out = attnOut;
    prm.pAcc = pAcc;
    prm.pM = pM;
    prm.pL = pL;
    prm.devPos = devPos;
    prm.totalRows = totalRows;
    prm.lenHost = pos + 1;
    prm.nHeads = nHeads;
    prm.nKV = nKV;
    prm.group = nHeads / nKV;
    prm.chunkTokens = pl.chunkTokens;
    prm.numChunks = numChunks;
    prm.invSqrt = invSqrt;
    prm.directOut = direct ? 1 : 0;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "tc_attn_decode_kv: no device error word");
    dim3 grid(pl.chunksPerSeq, pl.headGroups, 1);
    for (uint32_t cb = 0; cb < prm.group; cb += 8) {  // 8 q heads of a kv head per launch
        prm.colBase = cb;
        rc = hd == 64    ? launchKvHpc<64, 8>(pl.hpc, tmK, tmV, prm, grid, st)
             : hd == 128 ? launchKvHpc<128, 4>(pl.hpc, tmK, tmV, prm, grid, st)
                         : launchKvHpc<256, 2>(pl.hpc, tmK, tmV, prm, grid, st);
        if (rc != TC_OK) return rc;
    }
    if (direct) return TC_OK;
    return launchMerge(pAcc, pM, pL, attnOut, 1, nHeads, numChunks, pl.chunksPerSeq, hd, devPos, devPos ? 1u : 0u,
                       pl.chunkTokens, q81Out, false, st);
}

}  // extern "C"
