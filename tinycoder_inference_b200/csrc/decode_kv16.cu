// decode_kv16.cu -- grouped-query attention over an fp16 KV cache: split-KV decode and,
// with query rows as columns, the unsplit causal kernel.
//
// What it replaces: the KVT = __half instantiations of kWarpAttentionSplit /
// kWarpAttention(Pos) behind launchDecodeAttentionSplit(..., kvHalf = true, ...)
// (include/gpu/GpuAttentionKernels.hpp:211-272, 537-599, 625-766, 1129-1230), i.e. the
// dense models' optional fp16 cache (src/cpp/core/cuda/forward/GPUComputeUpload.cu:1252):
// score = dot(q, float(k)) * invSqrt, online softmax with exp2, out = sum p float(v) / sum p.
//
// Same skeleton as the int8 kernel (decode_i8.cu) -- grid (chunks, kv-head groups, sequences
// or row blocks), a TMA producer warp feeding an mbarrier ring, eight consumer warps that own
// a (kv head, 16-token) tile per stage and serve every q head of the kv head -- with the
// natural operands: fp16 K and V go into mma.sync.m16n8k16 as they are (ldmatrix for K,
// ldmatrix.trans for V, both straight from the 128-byte-swizzled TMA tiles), q and p are
// carried as fp16 hi + lo pairs (two MMAs, ~22 mantissa bits) after a power-of-two
// normalisation of q, accumulation is f32.  Nothing is rounded that the reference does not
// round: float(k) and float(v) are exact.
#include "decode_shared.cuh"

namespace tc {

struct DecodeKv16Params {
    const float *q;
    float *out;
    float *pAcc, *pM, *pL;
    const uint32_t *devPos;  // nullable: position read at kernel time
    uint64_t totalRows;
    uint32_t lenHost;
    uint32_t nHeads, nKV, group;
    uint32_t colBase;  // heads mode: the 8 MMA columns are q heads colBase .. colBase + 7 of the kv head
    uint32_t chunkTokens, numChunks;
    uint32_t rowsMode, qRows, cachePos;  // rows mode: see decode_i8.cu
    float invSqrt;
    int directOut;
    unsigned int *err;
};

// A stage holds K then V; each as HD/64 half-tiles of [rows][64 halves = 128 bytes] (one
// swizzle span), half-tile a covering dims [64a, 64a + 64).
template <int HD, int HPC, int NW, int NSTAGE>
struct DecodeKv16Smem {
    static constexpr int kAtoms = HD / 64;
    static constexpr int kRows = NW * 16;            // (token, head) rows per stage
    static constexpr int T = kRows / HPC;            // tokens per stage
    static constexpr int kAtomBytes = kRows * 128;   // one half-tile, all HPC heads
    static constexpr int kTileBytes = kRows * HD * 2;
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kBarOffset = NSTAGE * kStageBytes;
    static constexpr int kTotal = kBarOffset + 2 * NSTAGE * 8 + 1024;
    static_assert(T % 8 == 0 && T <= 256, "box rows");
    static_assert(kTotal <= 227 * 1024, "ring exceeds the shared memory of an SM");
};

constexpr float kLazyLog2Kv16 = 8.0f;  // see decode_i8.cu: p stays <= 2^8, exact enough as fp16 hi + lo

template <int HD, int HPC, int NW, int NSTAGE>
__global__ void __launch_bounds__((NW + 1) * 32, 1)
decodeKv16Kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const DecodeKv16Params p) {
    using L = DecodeKv16Smem<HD, HPC, NW, NSTAGE>;
    constexpr int T = L::T;
    constexpr int NS = HD / 16;     // k16 steps of QK^T = 16-dim output tiles of PV
    constexpr int NSUB = NW / HPC;  // consumer warps per kv head

    const uint32_t chunk = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *fullBar = reinterpret_cast<uint64_t *>(smem + L::kBarOffset);
    uint64_t *emptyBar = fullBar + NSTAGE;

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

    const uint32_t pos = p.devPos ? p.devPos[0] : 0u;
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
                    for (int a = 0; a < L::kAtoms; ++a) {
                        uint8_t *dst = st + a * L::kAtomBytes + h * T * 128;
                        tmaLoad3D(dst, &tmK, &fullBar[s], 64 * a, kvHead0 + h, row);
                        tmaLoad3D(dst + L::kTileBytes, &tmV, &fullBar[s], 64 * a, kvHead0 + h, row);
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

    // q of column n = g as the B operand of k16 step s: b0 = dims 16s + 2t, +1; b1 = dims
    // 16s + 8 + 2t, +1.  Power-of-two normalised, split into fp16 hi + lo.
    uint32_t qhi[NS][2], qlo[NS][2];
    float headScale;
    {
        const bool valid = colValid(g);
        const float *qp = p.q + colIndex(valid ? g : 0) * HD;
        float2 qv[NS][2];
        float amax = 0.0f;
#pragma unroll
        for (int s = 0; s < NS; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                qv[s][h] = valid ? __ldg(reinterpret_cast<const float2 *>(qp + 16 * s + 8 * h + 2 * t))
                                 : make_float2(0.f, 0.f);
                amax = fmaxf(amax, fmaxf(fabsf(qv[s][h].x), fabsf(qv[s][h].y)));
            }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2 amax)
        e = amax > 0.0f ? max(-100, min(100, e)) : 0;
        const float down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2^-e
        const float up = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);    // 2^e
        headScale = p.invSqrt * up * kLog2e;
#pragma unroll
        for (int s = 0; s < NS; ++s)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float h0, l0, h1, l1;
                splitHalf(qv[s][h].x * down, h0, l0);
                splitHalf(qv[s][h].y * down, h1, l1);
                qhi[s][h] = packHalf2(h0, h1);
                qlo[s][h] = packHalf2(l0, l1);
            }
    }
    const float cs0 = __shfl_sync(0xffffffffu, headScale, (2 * t) * 4);
    const float cs1 = __shfl_sync(0xffffffffu, headScale, (2 * t + 1) * 4);
    const uint32_t len0 = colLen(2 * t), len1 = colLen(2 * t + 1);

    float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
    float o[NS][4];
#pragma unroll
    for (int i = 0; i < NS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    const uint32_t lr = (lane & 7u) + ((lane >> 3) & 1u) * 8u;  // ldmatrix row this lane addresses
    const uint32_t lco = lane >> 4;                             // and which 16-byte chunk of the pair
    const uint32_t lmOff = lr * 128;

    for (uint32_t it = 0; it < nTiles; ++it) {
        const uint32_t s = it % NSTAGE;
        if (!mbarWaitClock(&fullBar[s], (it / NSTAGE) & 1, p.err, kDevErrFullWait)) break;
        uint8_t *st = smem + s * L::kStageBytes;
        const uint32_t rowInTile = hL * T + sub * 16;
        const uint32_t tokW = t0 + it * T + sub * 16;  // first token of this warp's tile
        const uint32_t tokA = tokW + g, tokB = tokA + 8;

        // ---- S^T = K . Q^T (16 tokens x 8 columns) ----
        float sh[4] = {0.f, 0.f, 0.f, 0.f}, sl[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t kTile = smemAddr(st + rowInTile * 128);
#pragma unroll
        for (int ks = 0; ks < NS; ++ks) {
            const uint32_t sw = (((2 * (ks & 3) + lco) ^ (lr & 7u)) << 4) + (ks >> 2) * L::kAtomBytes;
            uint32_t r0, r1, r2, r3;  // rows 0-7 / 8-15 of dims 16ks..+7, then of dims 16ks+8..+15
            ldmatrixX4(r0, r1, r2, r3, kTile + lmOff + sw);
            mmaF16(sh, r0, r1, r2, r3, qhi[ks][0], qhi[ks][1]);
            mmaF16(sl, r0, r1, r2, r3, qlo[ks][0], qlo[ks][1]);
        }
        // a stale or foreign row behind the range may hold anything, NaN included: select, never scale
        const float s00 = tokA < len0 ? (sh[0] + sl[0]) * cs0 : -INFINITY;
        const float s01 = tokA < len1 ? (sh[1] + sl[1]) * cs1 : -INFINITY;
        const float s10 = tokB < len0 ? (sh[2] + sl[2]) * cs0 : -INFINITY;
        const float s11 = tokB < len1 ? (sh[3] + sl[3]) * cs1 : -INFINITY;
        float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = mx0 > m0 + kLazyLog2Kv16 ? mx0 : m0;
        const float mn1 = mx1 > m1 + kLazyLog2Kv16 ? mx1 : m1;
        if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1)) {
            const float a0 = fastExp2(m0 - mn0), a1 = fastExp2(m1 - mn1);
#pragma unroll
            for (int i = 0; i < NS; ++i) {
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
        // p as fp16 hi + lo, transposed to the B layout (tokens 2t, 2t+1 / 8+2t, 8+2t+1 of column g)
        uint32_t bh[2], bl[2];
        {
            const float p00 = fastExp2(s00 - m0), p01 = fastExp2(s01 - m1);
            const float p10 = fastExp2(s10 - m0), p11 = fastExp2(s11 - m1);
            l0 += p00 + p10;
            l1 += p01 + p11;
            float h0, q0, h1, q1;
            splitHalf(p00, h0, q0);
            splitHalf(p01, h1, q1);
            bh[0] = movmatrixTrans(packHalf2(h0, h1));
            bl[0] = movmatrixTrans(packHalf2(q0, q1));
            splitHalf(p10, h0, q0);
            splitHalf(p11, h1, q1);
            bh[1] = movmatrixTrans(packHalf2(h0, h1));
            bl[1] = movmatrixTrans(packHalf2(q0, q1));
        }
        // ---- O^T += V^T . P^T (HD dims x 8 columns), V read transposed ----
        // rows behind the chunk get probability 0, but 0 * NaN is NaN: clear those V rows.
        // Register halves of a transposed fragment are tokens 2t (low) and 2t+1 (high).
        uint32_t mk0 = 0xffffffffu, mk1 = 0xffffffffu;
        if (tokW + 16 > t1) {
            mk0 = (tokW + 2 * t < t1 ? 0x0000ffffu : 0u) | (tokW + 2 * t + 1 < t1 ? 0xffff0000u : 0u);
            mk1 = (tokW + 8 + 2 * t < t1 ? 0x0000ffffu : 0u) | (tokW + 8 + 2 * t + 1 < t1 ? 0xffff0000u : 0u);
        }
        const uint32_t vTile = smemAddr(st + L::kTileBytes + rowInTile * 128);
#pragma unroll
        for (int ks = 0; ks < NS; ++ks) {
            const uint32_t sw = (((2 * (ks & 3) + lco) ^ (lr & 7u)) << 4) + (ks >> 2) * L::kAtomBytes;
            uint32_t r0, r1, r2, r3;  // (tokens 0-7, dims lo) (tokens 8-15, dims lo) (0-7, dims hi) (8-15, dims hi)
            ldmatrixX4Trans(r0, r1, r2, r3, vTile + lmOff + sw);
            r0 &= mk0;
            r2 &= mk0;
            r1 &= mk1;
            r3 &= mk1;
            // A rows g / g+8 = dims 16ks + g / + 8 + g; k = tokens
            mmaF16(o[ks], r0, r2, r1, r3, bh[0], bh[1]);
            mmaF16(o[ks], r0, r2, r1, r3, bl[0], bl[1]);
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
    namedBarSync(1, NW * 32);  // every consumer is done reading the ring
    float *scr = reinterpret_cast<float *>(smem);
    constexpr int kWarpScr = 8 * HD + 16;
    float *wO = scr + warp * kWarpScr;  // [8 columns][HD], then m[8], l[8]
#pragma unroll
    for (int c = 0; c < NS; ++c) {
        const int d = 16 * c + g;
        wO[(2 * t) * HD + d] = o[c][0];
        wO[(2 * t + 1) * HD + d] = o[c][1];
        wO[(2 * t) * HD + d + 8] = o[c][2];
        wO[(2 * t + 1) * HD + d + 8] = o[c][3];
    }
    if (g == 0) {
        wO[8 * HD + 2 * t] = m0;
        wO[8 * HD + 2 * t + 1] = m1;
        wO[8 * HD + 8 + 2 * t] = l0;
        wO[8 * HD + 8 + 2 * t + 1] = l1;
    }
    namedBarSync(1, NW * 32);
    constexpr uint32_t V4 = HD / 4;
    for (uint32_t idx = threadIdx.x; idx < HPC * 8 * V4; idx += NW * 32) {
        const uint32_t d4 = idx % V4, j = (idx / V4) & 7u, h = idx / (8 * V4);
        if (!colValid(j)) continue;
        float M = kNegBig;
#pragma unroll
        for (int sb = 0; sb < NSUB; ++sb) M = fmaxf(M, scr[(sb * HPC + h) * kWarpScr + 8 * HD + j]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float lsum = 0.0f;
#pragma unroll
        for (int sb = 0; sb < NSUB; ++sb) {
            const float *w = scr + (sb * HPC + h) * kWarpScr;
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

template <int HD, int HPC>
static int launchKv16(const CUtensorMap &tmK, const CUtensorMap &tmV, const DecodeKv16Params &prm, dim3 grid,
                      cudaStream_t st) {
    constexpr int NW = 8, NSTAGE = HD == 128 ? 3 : 6;
    using L = DecodeKv16Smem<HD, HPC, NW, NSTAGE>;
    auto kern = decodeKv16Kernel<HD, HPC, NW, NSTAGE>;
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

template <int HD>
static int launchKv16Hpc(uint32_t hpc, const CUtensorMap &tmK, const CUtensorMap &tmV, const DecodeKv16Params &prm,
                         dim3 grid, cudaStream_t st) {
    if (hpc == 4) return launchKv16<HD, 4>(tmK, tmV, prm, grid, st);
    if (hpc == 2) return launchKv16<HD, 2>(tmK, tmV, prm, grid, st);
    return launchKv16<HD, 1>(tmK, tmV, prm, grid, st);
}

static int kv16Maps(const void *kvK, const void *kvV, uint32_t nKV, uint32_t hd, uint64_t totalRows,
                    uint32_t boxRows, CUtensorMap *tmK, CUtensorMap *tmV) {
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.rank = 3;
    key.elemBytes = 2;
    key.swizzle = 3;
    key.dims[0] = hd;
    key.dims[1] = nKV;
    key.dims[2] = totalRows;
    key.strides[0] = static_cast<uint64_t>(hd) * 2;
    key.strides[1] = static_cast<uint64_t>(nKV) * hd * 2;
    key.box[0] = 64;
    key.box[1] = 1;
    key.box[2] = boxRows;
    key.base = kvK;
    int rc = getTensorMap(key, tmK);
    if (rc != TC_OK) return rc;
    key.base = kvV;
    return getTensorMap(key, tmV);
}

// Called from decode_kv.cu when kvHalf is set; arguments were validated there.
int decodeKv16(const float *q, const void *kvK, const void *kvV, float *attnOut, float *pAcc, float *pM, float *pL,
               uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t pos, const uint32_t *devPos, uint64_t totalRows,
               uint32_t numChunks, float invSqrt, uint8_t *q81Out, cudaStream_t st) {
    DecodePlan pl = planDecode(1, nKV, pos + 1, numChunks, 8u * 16u);
    const bool direct = pl.chunksPerSeq == 1 && q81Out == nullptr;
    if (!direct) TC_REQUIRE(pAcc && pM && pL, TC_EWORKSPACE, "tc_attn_decode_kv: partial buffers are required");
    CUtensorMap tmK, tmV;
    int rc = kv16Maps(kvK, kvV, nKV, hd, totalRows, pl.tileTokens, &tmK, &tmV);
    if (rc != TC_OK) return rc;
    DecodeKv16Params prm;
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
        rc = hd == 64 ? launchKv16Hpc<64>(pl.hpc, tmK, tmV, prm, grid, st)
                      : launchKv16Hpc<128>(pl.hpc, tmK, tmV, prm, grid, st);
        if (rc != TC_OK) return rc;
    }
    if (direct) return TC_OK;
    return launchMerge(pAcc, pM, pL, attnOut, 1, nHeads, numChunks, pl.chunksPerSeq, hd, devPos, devPos ? 1u : 0u,
                       pl.chunkTokens, q81Out, false, st);
}

int prefillKv16(const float *q, const void *kvK, const void *kvV, float *out, uint32_t seqLen, uint32_t nHeads,
                uint32_t nKV, uint32_t hd, uint32_t cachePos, const uint32_t *devPos, uint64_t totalRows,
                float invSqrt, cudaStream_t st) {
    const uint32_t rowBlocks = (seqLen + 7) / 8;
    CUtensorMap tmK, tmV;
    int rc = kv16Maps(kvK, kvV, nKV, hd, totalRows, 8u * 16u, &tmK, &tmV);
    if (rc != TC_OK) return rc;
    DecodeKv16Params prm;
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
    if (hd == 64) return launchKv16<64, 1>(tmK, tmV, prm, grid, st);
    return launchKv16<128, 1>(tmK, tmV, prm, grid, st);
}

}  // namespace tc
