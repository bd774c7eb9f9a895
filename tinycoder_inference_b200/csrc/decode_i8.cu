// decode_i8.cu -- grouped-query decode attention over the int8 KV store.
//
// What it replaces: kQ35WarpAttention8Split + kAttnCombinePartial and the eager
// kQ35WarpAttention8 of the reference (include/gpu/GpuQwen35Kernels.hpp:519-581,
// 641-692): q f32 [nHeads][hd], K/V rows int8 with one f32 scale per (row, kv
// head), score = dot(q, float(k8)*sk) * invSqrt, online softmax with exp2,
// out = sum p * float(v8)*sv / sum p.
//
// How it is built for B200:
//   * split-K flash-decoding.  grid = (chunks, kv-head groups, sequences); a CTA
//     streams one contiguous token range of HPC kv heads and serves ALL q heads
//     of those kv heads, so every KV byte leaves HBM exactly once.
//   * KV streaming by TMA (cp.async.bulk.tensor, 128-byte swizzle) from one
//     producer warp into an mbarrier ring; the per-row scales ride in the same
//     stage through cp.async.  8 consumer warps, one (kv head, 16-token) tile
//     each per stage.
//   * at group 5..7 the dequant+FMA work (2*group flop per KV byte) is beyond the
//     CUDA cores at HBM speed, so QK^T and PV run on tensor cores
//     (mma.sync.m16n8k16): int8 is converted to fp16 exactly (prmt + one hsub2),
//     q and p*sv are carried as fp16 hi+lo pairs (two MMAs, ~22 mantissa bits)
//     after a power-of-two normalisation, accumulation is f32.  The per-row K
//     scale is applied to the score column after the MMA, the V scale is folded
//     into p before it.
//   * S is produced transposed (tokens x heads) so no MMA row is padding; the
//     probabilities reach the PV operand layout through movmatrix.trans.
//   * softmax reductions are warp shuffles; (m, l, acc) partials per chunk go to
//     the caller's partial buffers in the reference's layout and are merged by
//     the merge kernel (merge.cu).
#include "tc_common.cuh"

namespace tc {

int launchMerge(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t seqLen,
                uint32_t nHeads, uint32_t numChunks, uint32_t activeHost, uint32_t hd, const uint32_t *devLens,
                uint32_t lenAdd, uint32_t chunkTokens, uint8_t *q81, cudaStream_t st);

struct DecodeI8Params {
    const float *q;
    float *out;
    const float *ks, *vs;
    float *pAcc, *pM, *pL;
    const uint32_t *devLens;     // nullable
    const uint64_t *devRowBase;  // nullable
    uint64_t rowsPerSeq, totalRows;
    uint32_t lenHost, lenAdd;
    uint32_t nHeads, nKV, group;
    uint32_t chunkTokens, numChunks;
    float invSqrt;
    int directOut;
    unsigned int *err;
};

constexpr int kHD = 128;

template <int HPC, int NW, int NSTAGE>
struct DecodeI8Smem {
    static constexpr int T = NW * 16 / HPC;              // tokens per stage
    static constexpr int kTileBytes = NW * 16 * kHD;     // K (or V) bytes per stage, all HPC heads
    static constexpr int kScaleBytes = NW * 16 * 4;
    static constexpr int kStageBytes = 2 * kTileBytes + 2 * kScaleBytes;
    static constexpr int kBarOffset = NSTAGE * kStageBytes;
    static constexpr int kTotal = kBarOffset + 2 * NSTAGE * 8 + 1024;  // + alignment slack
    static_assert(kStageBytes % 1024 == 0, "stage must keep 1024-byte alignment for the 128B swizzle");
};

__device__ __forceinline__ bool mbarWaitClock(uint64_t *bar, uint32_t parity, unsigned int *err,
                                              uint32_t errBit) {
    // ~2^31 cycles (about a second) before giving up.
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbarTryWait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    atomicOr(err, errBit);
    return false;
}

template <int HPC, int NW, int NSTAGE, int MINB>
__global__ void __launch_bounds__((NW + 1) * 32, MINB)
decodeI8Kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const DecodeI8Params p) {
    using L = DecodeI8Smem<HPC, NW, NSTAGE>;
    constexpr int T = L::T;
    constexpr int NSUB = NW / HPC;  // consumer warps per kv head

    const uint32_t chunk = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
    const uint32_t len = p.devLens ? p.devLens[b] + p.lenAdd : p.lenHost;
    const uint32_t t0 = chunk * p.chunkTokens;
    if (t0 >= len) return;  // inactive chunk: the merge derives the active count from len
    const uint32_t t1 = min(len, t0 + p.chunkTokens);
    const uint32_t nTiles = (t1 - t0 + T - 1) / T;
    const uint64_t rowBase = p.devRowBase ? p.devRowBase[b] : static_cast<uint64_t>(b) * p.rowsPerSeq;

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *fullBar = reinterpret_cast<uint64_t *>(smem + L::kBarOffset);
    uint64_t *emptyBar = fullBar + NSTAGE;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbarInit(&fullBar[s], 1 + 32);
            mbarInit(&emptyBar[s], NW);
        }
        fenceBarrierInit();
        tmaPrefetchDesc(&tmK);
        tmaPrefetchDesc(&tmV);
    }
    __syncthreads();

    if (warp == NW) {
        // ------------------------------ producer ------------------------------
        const uint32_t kvHead0 = hg * HPC;
        for (uint32_t it = 0; it < nTiles; ++it) {
            const uint32_t s = it % NSTAGE;
            if (it >= NSTAGE) {
                if (!mbarWaitClock(&emptyBar[s], ((it / NSTAGE) - 1) & 1, p.err, kDevErrEmptyWait)) break;
            }
            uint8_t *st = smem + s * L::kStageBytes;
            const uint64_t row = rowBase + t0 + static_cast<uint64_t>(it) * T;
            if (lane == 0) {
                mbarExpectTx(&fullBar[s], 2 * L::kTileBytes);
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
                    tmaLoad3D(st + h * T * kHD, &tmK, &fullBar[s], 0, kvHead0 + h, static_cast<int>(row));
                    tmaLoad3D(st + L::kTileBytes + h * T * kHD, &tmV, &fullBar[s], 0, kvHead0 + h,
                              static_cast<int>(row));
                }
            }
            float *sK = reinterpret_cast<float *>(st + 2 * L::kTileBytes);
            float *sV = sK + NW * 16;
#pragma unroll
            for (int idx = lane; idx < HPC * T; idx += 32) {
                const int h = idx / T, tt = idx % T;
                uint64_t r = row + tt;
                r = r < p.totalRows ? r : p.totalRows - 1;
                cpAsync4(&sK[idx], p.ks + r * p.nKV + kvHead0 + h);
                cpAsync4(&sV[idx], p.vs + r * p.nKV + kvHead0 + h);
            }
            cpAsyncMbarArriveNoinc(&fullBar[s]);
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t hL = warp % HPC, sub = warp / HPC;
    const uint32_t kvHead = hg * HPC + hL;

    // q fragments for head column n = g of this kv head's group: power-of-two
    // normalised, split into fp16 hi + lo, laid out as the B operand whose k
    // slots follow the byte order ldmatrix hands out (dims 16c + 4t + {0..3}).
    uint32_t qhi[8][2], qlo[8][2];
    float headScale;
    {
        float4 qv[8];
        float amax = 0.0f;
        const bool valid = g < p.group;
        const float *qp = p.q + (static_cast<size_t>(b) * p.nHeads + kvHead * p.group + (valid ? g : 0)) * kHD;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            qv[c] = valid ? __ldg(reinterpret_cast<const float4 *>(qp + 16 * c + 4 * t))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(qv[c].x), fabsf(qv[c].y)), fmaxf(fabsf(qv[c].z), fabsf(qv[c].w))));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 127;  // floor(log2 amax)
        e = amax > 0.0f ? max(-100, min(100, e)) : 0;
        const float down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);  // 2^-e
        const float up = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);    // 2^e
        headScale = p.invSqrt * up * kLog2e;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float h0, l0, h1, l1, h2, l2, h3, l3;
            splitHalf(qv[c].x * down, h0, l0);
            splitHalf(qv[c].y * down, h1, l1);
            splitHalf(qv[c].z * down, h2, l2);
            splitHalf(qv[c].w * down, h3, l3);
            qhi[c][0] = packHalf2(h0, h1);
            qhi[c][1] = packHalf2(h2, h3);
            qlo[c][0] = packHalf2(l0, l1);
            qlo[c][1] = packHalf2(l2, l3);
        }
    }
    // score columns of this thread are heads 2t and 2t+1: fetch their scales
    const float cs0 = __shfl_sync(0xffffffffu, headScale, (2 * t) * 4);
    const float cs1 = __shfl_sync(0xffffffffu, headScale, (2 * t + 1) * 4);

    float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
    uint32_t Ebits = 0;  // running power-of-two scale of the V row scales (0 = unset)
    float invE = 0.0f;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    const uint32_t lr = (lane & 7u) + ((lane >> 3) & 1u) * 8u;  // ldmatrix row this lane addresses
    const uint32_t lco = lane >> 4;                             // and which chunk of the pair
    bool ok = true;

    for (uint32_t it = 0; it < nTiles; ++it) {
        const uint32_t s = it % NSTAGE;
        if (!mbarWaitClock(&fullBar[s], (it / NSTAGE) & 1, p.err, kDevErrFullWait)) {
            ok = false;
            break;
        }
        uint8_t *st = smem + s * L::kStageBytes;
        const float *sK = reinterpret_cast<const float *>(st + 2 * L::kTileBytes) + hL * T + sub * 16;
        const float *sV = sK + NW * 16;
        const uint32_t tok0 = t0 + it * T + sub * 16 + g;
        const bool v0 = tok0 < t1, v1 = tok0 + 8 < t1;
        const float skA = sK[g], skB = sK[g + 8];
        const float svA = v0 ? sV[g] : 0.0f, svB = v1 ? sV[g + 8] : 0.0f;

        // ---- S^T = K . Q^T (16 tokens x 8 heads) ----
        // two accumulators (hi and lo parts of q) keep the MMA dependency chains short
        float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t kTile = smemAddr(st + (hL * T + sub * 16) * kHD);
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {
            uint32_t r0, r1, r2, r3;
            const uint32_t chunkIdx = 2 * cp + lco;
            ldmatrixX4(r0, r1, r2, r3, kTile + lr * 128 + ((chunkIdx ^ (lr & 7u)) << 4));
            r0 ^= 0x80808080u;
            r1 ^= 0x80808080u;
            r2 ^= 0x80808080u;
            r3 ^= 0x80808080u;
            {
                const uint32_t a0 = biasedPairLo(r0), a1 = biasedPairLo(r1), a2 = biasedPairHi(r0),
                               a3 = biasedPairHi(r1);
                mmaF16(sc, a0, a1, a2, a3, qhi[2 * cp][0], qhi[2 * cp][1]);
                mmaF16(sc2, a0, a1, a2, a3, qlo[2 * cp][0], qlo[2 * cp][1]);
            }
            {
                const uint32_t a0 = biasedPairLo(r2), a1 = biasedPairLo(r3), a2 = biasedPairHi(r2),
                               a3 = biasedPairHi(r3);
                mmaF16(sc, a0, a1, a2, a3, qhi[2 * cp + 1][0], qhi[2 * cp + 1][1]);
                mmaF16(sc2, a0, a1, a2, a3, qlo[2 * cp + 1][0], qlo[2 * cp + 1][1]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i] += sc2[i];
        // log2-domain scores; rows past the range are masked out
        const float ninf = -INFINITY;
        const float s00 = v0 ? sc[0] * (skA * cs0) : ninf;
        const float s01 = v0 ? sc[1] * (skA * cs1) : ninf;
        const float s10 = v1 ? sc[2] * (skB * cs0) : ninf;
        const float s11 = v1 ? sc[3] * (skB * cs1) : ninf;
        float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // running power-of-two bound of the V scales (keeps p*sv inside fp16)
        uint32_t eb = __reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(svA, svB))) & 0x7f800000u;
        eb = min(eb, 253u << 23);
        float fE = 1.0f;
        if (eb > Ebits) {
            const float newInv = __uint_as_float((254u << 23) - eb);
            fE = Ebits ? __uint_as_float(Ebits) * newInv : 1.0f;
            Ebits = eb;
            invE = newInv;
        }
        const float a0s = fastExp2(m0 - mn0), a1s = fastExp2(m1 - mn1);
        const float al0 = a0s * fE, al1 = a1s * fE;
        m0 = mn0;
        m1 = mn1;
        if (__any_sync(0xffffffffu, al0 != 1.0f || al1 != 1.0f)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                o[i][0] *= al0;
                o[i][1] *= al1;
                o[i][2] *= al0;
                o[i][3] *= al1;
            }
        }
        const float p00 = fastExp2(s00 - mn0), p01 = fastExp2(s01 - mn1);
        const float p10 = fastExp2(s10 - mn0), p11 = fastExp2(s11 - mn1);
        l0 = l0 * a0s + (p00 + p10);
        l1 = l1 * a1s + (p01 + p11);
        // p * sv (scaled into fp16 range), hi + lo, then transposed to the B layout
        uint32_t bh0, bh1, bl0, bl1;
        {
            const float wA = svA * invE, wB = svB * invE;
            float h00, q00, h01, q01, h10, q10, h11, q11;
            splitHalf(p00 * wA, h00, q00);
            splitHalf(p01 * wA, h01, q01);
            splitHalf(p10 * wB, h10, q10);
            splitHalf(p11 * wB, h11, q11);
            bh0 = movmatrixTrans(packHalf2(h00, h01));
            bh1 = movmatrixTrans(packHalf2(h10, h11));
            bl0 = movmatrixTrans(packHalf2(q00, q01));
            bl1 = movmatrixTrans(packHalf2(q10, q11));
        }
        // ---- O^T += V^T . P^T (128 dims x 8 heads) ----
        const uint8_t *vTile = st + L::kTileBytes + (hL * T + sub * 16) * kHD;
        const uint32_t ra = 2 * t, rb = 2 * t + 1;  // token rows 2t, 2t+1 (and +8); (row & 7) is the swizzle key
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
            const uint32_t ch = 2 * blk + (g >> 2), off = 4 * (g & 3u);
            uint32_t w0 = *reinterpret_cast<const uint32_t *>(vTile + ra * 128 + ((ch ^ ra) << 4) + off);
            uint32_t w1 = *reinterpret_cast<const uint32_t *>(vTile + rb * 128 + ((ch ^ rb) << 4) + off);
            uint32_t w2 = *reinterpret_cast<const uint32_t *>(vTile + (ra + 8) * 128 + ((ch ^ ra) << 4) + off);
            uint32_t w3 = *reinterpret_cast<const uint32_t *>(vTile + (rb + 8) * 128 + ((ch ^ rb) << 4) + off);
            w0 ^= 0x80808080u;
            w1 ^= 0x80808080u;
            w2 ^= 0x80808080u;
            w3 ^= 0x80808080u;
            const uint32_t X = __byte_perm(w0, w1, 0x5140), Y = __byte_perm(w0, w1, 0x7362);
            const uint32_t X2 = __byte_perm(w2, w3, 0x5140), Y2 = __byte_perm(w2, w3, 0x7362);
            {
                const uint32_t a0 = biasedPairLo(X), a1 = biasedPairHi(X), a2 = biasedPairLo(X2),
                               a3 = biasedPairHi(X2);
                mmaF16(o[2 * blk], a0, a1, a2, a3, bh0, bh1);
                mmaF16(o[2 * blk], a0, a1, a2, a3, bl0, bl1);
            }
            {
                const uint32_t a0 = biasedPairLo(Y), a1 = biasedPairHi(Y), a2 = biasedPairLo(Y2),
                               a3 = biasedPairHi(Y2);
                mmaF16(o[2 * blk + 1], a0, a1, a2, a3, bh0, bh1);
                mmaF16(o[2 * blk + 1], a0, a1, a2, a3, bl0, bl1);
            }
        }
        __syncwarp();
        if (lane == 0) mbarArrive(&emptyBar[s]);
    }
    (void) ok;

    // ---- fold the consumer warps of each kv head, write the chunk partial ----
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    namedBarSync(1, NW * 32);  // every consumer is done reading the ring
    float *scr = reinterpret_cast<float *>(smem);
    float *wO = scr + warp * (8 * kHD + 16);  // [8 heads][128], then m[8], l[8]
    const float E = __uint_as_float(Ebits);
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
        const int d = 32 * blk + 4 * g;
        *reinterpret_cast<float4 *>(wO + (2 * t) * kHD + d) =
                make_float4(o[2 * blk][0] * E, o[2 * blk][2] * E, o[2 * blk + 1][0] * E, o[2 * blk + 1][2] * E);
        *reinterpret_cast<float4 *>(wO + (2 * t + 1) * kHD + d) =
                make_float4(o[2 * blk][1] * E, o[2 * blk][3] * E, o[2 * blk + 1][1] * E, o[2 * blk + 1][3] * E);
    }
    if (g == 0) {
        wO[8 * kHD + 2 * t] = m0;
        wO[8 * kHD + 2 * t + 1] = m1;
        wO[8 * kHD + 8 + 2 * t] = l0;
        wO[8 * kHD + 8 + 2 * t + 1] = l1;
    }
    namedBarSync(1, NW * 32);
    // NW*32 threads, HPC*8*32 float4 outputs
    for (uint32_t idx = threadIdx.x; idx < HPC * 8 * 32; idx += NW * 32) {
        const uint32_t d4 = idx & 31u, j = (idx >> 5) & 7u, h = idx >> 8;
        if (j >= p.group) continue;
        float M = kNegBig;
#pragma unroll
        for (int sb = 0; sb < NSUB; ++sb) M = fmaxf(M, scr[(sb * HPC + h) * (8 * kHD + 16) + 8 * kHD + j]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float lsum = 0.0f;
#pragma unroll
        for (int sb = 0; sb < NSUB; ++sb) {
            const float *w = scr + (sb * HPC + h) * (8 * kHD + 16);
            const float wgt = fastExp2(w[8 * kHD + j] - M);
            lsum += wgt * w[8 * kHD + 8 + j];
            const float4 a = *reinterpret_cast<const float4 *>(w + j * kHD + 4 * d4);
            acc.x = fmaf(wgt, a.x, acc.x);
            acc.y = fmaf(wgt, a.y, acc.y);
            acc.z = fmaf(wgt, a.z, acc.z);
            acc.w = fmaf(wgt, a.w, acc.w);
        }
        const uint32_t qHead = (hg * HPC + h) * p.group + j;
        if (p.directOut) {
            const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
            *reinterpret_cast<float4 *>(p.out + (static_cast<size_t>(b) * p.nHeads + qHead) * kHD + 4 * d4) =
                    make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else {
            const size_t pidx = (static_cast<size_t>(b) * p.nHeads + qHead) * p.numChunks + chunk;
            *reinterpret_cast<float4 *>(p.pAcc + pidx * kHD + 4 * d4) = acc;
            if (d4 == 0) {
                // back to natural-log units: the merge contract is w = exp2((m - M) * log2e)
                p.pM[pidx] = M > -1e29f ? M * 0.6931471805599453f : kNegBig;
                p.pL[pidx] = lsum;
            }
        }
    }
}

struct DecodePlan {
    uint32_t hpc, headGroups, chunkTokens, chunksPerSeq, tileTokens;
};

// One wave of CTAs over the SMs when the batch is small, a few waves when many
// ragged sequences need the hardware scheduler to even things out.
static DecodePlan planDecode(uint32_t batch, uint32_t nKV, uint32_t maxLen, uint32_t slots, int nw) {
    DecodePlan pl;
    pl.hpc = (nKV % 4u == 0) ? 4u : (nKV % 2u == 0 ? 2u : 1u);
    pl.headGroups = nKV / pl.hpc;
    pl.tileTokens = static_cast<uint32_t>(nw) * 16u / pl.hpc;
    const uint32_t tilesMax = (maxLen + pl.tileTokens - 1) / pl.tileTokens;
    const uint32_t sms = static_cast<uint32_t>(numSMs());
    const uint32_t waves = batch > 1 ? 2u : 1u;
    uint32_t want = (sms * waves) / (batch * pl.headGroups);
    want = want < 1u ? 1u : want;
    want = want > slots ? slots : want;
    want = want > tilesMax ? tilesMax : want;
    want = want < 1u ? 1u : want;
    const uint32_t tilesPerChunk = (tilesMax + want - 1) / want;
    pl.chunkTokens = tilesPerChunk * pl.tileTokens;
    pl.chunksPerSeq = (tilesMax + tilesPerChunk - 1) / tilesPerChunk;
    if (pl.chunksPerSeq == 0) pl.chunksPerSeq = 1;
    return pl;
}

template <int HPC>
static int launchDecodeI8(const CUtensorMap &tmK, const CUtensorMap &tmV, const DecodeI8Params &prm,
                          const DecodePlan &pl, uint32_t batch, cudaStream_t st) {
    constexpr int NW = 8, NSTAGE = 4, MINB = 1;
    using L = DecodeI8Smem<HPC, NW, NSTAGE>;
    auto kern = decodeI8Kernel<HPC, NW, NSTAGE, MINB>;
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attrDone[dev] = true;
    }
    dim3 grid(pl.chunksPerSeq, pl.headGroups, batch);
    kern<<<grid, (NW + 1) * 32, L::kTotal, st>>>(tmK, tmV, prm);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

static int decodeI8Common(const tc_decode_i8_batch *d, uint32_t lenHost, uint32_t lenAdd, cudaStream_t st) {
    TC_REQUIRE(d->q && d->out && d->k8 && d->v8 && d->ks && d->vs, TC_EINVAL, "decode_i8: null pointer");
    TC_REQUIRE(d->hd == kHD, TC_EUNSUPPORTED, "decode_i8: head_dim %u (built for 128)", d->hd);
    TC_REQUIRE(d->nKV > 0 && d->nHeads % d->nKV == 0, TC_EINVAL, "decode_i8: nHeads %u not a multiple of nKV %u",
               d->nHeads, d->nKV);
    const uint32_t group = d->nHeads / d->nKV;
    TC_REQUIRE(group <= 8, TC_EUNSUPPORTED, "decode_i8: %u q heads per kv head (built for <= 8)", group);
    TC_REQUIRE(d->batch >= 1 && d->batch <= 65535, TC_EINVAL, "decode_i8: batch %u", d->batch);
    TC_REQUIRE(d->maxLen >= 1, TC_EINVAL, "decode_i8: empty context");
    TC_REQUIRE(d->totalRows >= 1 && d->totalRows < (1ull << 31), TC_EUNSUPPORTED,
               "decode_i8: pool of %llu rows", (unsigned long long) d->totalRows);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(d->k8) | reinterpret_cast<uintptr_t>(d->v8) |
                 reinterpret_cast<uintptr_t>(d->q) | reinterpret_cast<uintptr_t>(d->out)) & 15u) == 0,
               TC_EINVAL, "decode_i8: q/out/k8/v8 need 16-byte alignment");
    TC_REQUIRE(d->numChunks >= 1, TC_EWORKSPACE, "decode_i8: no chunk slots");
    const DecodePlan pl = planDecode(d->batch, d->nKV, d->maxLen, d->numChunks, 8);
    const bool direct = pl.chunksPerSeq == 1 && !d->partialsOnly;
    if (!direct)
        TC_REQUIRE(d->pAcc && d->pM && d->pL, TC_EWORKSPACE, "decode_i8: partial buffers are required");
    if (d->chunksUsed) *d->chunksUsed = pl.chunksPerSeq;

    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.rank = 3;
    key.elemBytes = 1;
    key.swizzle = 3;
    key.dims[0] = kHD;
    key.dims[1] = d->nKV;
    key.dims[2] = d->totalRows;
    key.strides[0] = kHD;
    key.strides[1] = static_cast<uint64_t>(d->nKV) * kHD;
    key.box[0] = kHD;
    key.box[1] = 1;
    key.box[2] = pl.tileTokens;
    CUtensorMap tmK, tmV;
    key.base = d->k8;
    int rc = getTensorMap(key, &tmK);
    if (rc != TC_OK) return rc;
    key.base = d->v8;
    rc = getTensorMap(key, &tmV);
    if (rc != TC_OK) return rc;

    DecodeI8Params prm;
    prm.q = d->q;
    prm.out = d->out;
    prm.ks = d->ks;
    prm.vs = d->vs;
    prm.pAcc = d->pAcc;
    prm.pM = d->pM;
    prm.pL = d->pL;
    prm.devLens = d->lens;
    prm.devRowBase = d->rowBase;
    prm.rowsPerSeq = d->rowsPerSeq;
    prm.totalRows = d->totalRows;
    prm.lenHost = lenHost;
    prm.lenAdd = lenAdd;
    prm.nHeads = d->nHeads;
    prm.nKV = d->nKV;
    prm.group = group;
    prm.chunkTokens = pl.chunkTokens;
    prm.numChunks = d->numChunks;
    prm.invSqrt = d->invSqrt;
    prm.directOut = direct ? 1 : 0;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "decode_i8: no device error word");

    if (pl.hpc == 4) rc = launchDecodeI8<4>(tmK, tmV, prm, pl, d->batch, st);
    else if (pl.hpc == 2) rc = launchDecodeI8<2>(tmK, tmV, prm, pl, d->batch, st);
    else rc = launchDecodeI8<1>(tmK, tmV, prm, pl, d->batch, st);
    if (rc != TC_OK) return rc;
    if (direct || d->partialsOnly) return TC_OK;
    // merge: the active chunk count of a sequence follows from its length (read on
    // the device when the length lives there); slots past it were never written.
    return launchMerge(d->pAcc, d->pM, d->pL, d->out, d->batch, d->nHeads, d->numChunks, pl.chunksPerSeq, kHD,
                       d->lens, lenAdd, pl.chunkTokens, nullptr, st);
}

}  // namespace tc

extern "C" {

int tc_attn_decode_i8_batch(const tc_decode_i8_batch *d, tc_stream stream) {
    TC_REQUIRE(d != nullptr, TC_EINVAL, "tc_attn_decode_i8_batch: null descriptor");
    TC_REQUIRE(d->lens != nullptr, TC_EINVAL, "tc_attn_decode_i8_batch: lens (device) is required");
    return tc::decodeI8Common(d, 0, 0, static_cast<cudaStream_t>(stream));
}

int tc_attn_decode_i8(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                      float *out, float *pAcc, float *pM, float *pL, uint32_t nHeads, uint32_t nKV, uint32_t hd,
                      uint32_t cachePos, const uint32_t *devPos, uint64_t totalRows, uint32_t numChunks,
                      uint32_t chunkSize, float invSqrt, tc_stream stream) {
    (void) chunkSize;
    TC_REQUIRE(static_cast<uint64_t>(cachePos) + 1 <= totalRows, TC_ECONTEXT_FULL,
               "tc_attn_decode_i8: position %u is outside the pool of %llu rows", cachePos,
               (unsigned long long) totalRows);
    tc_decode_i8_batch d;
    memset(&d, 0, sizeof(d));
    d.q = q;
    d.out = out;
    d.k8 = k8;
    d.v8 = v8;
    d.ks = ks;
    d.vs = vs;
    d.pAcc = pAcc;
    d.pM = pM;
    d.pL = pL;
    d.lens = devPos;
    d.rowBase = nullptr;
    d.rowsPerSeq = 0;
    d.totalRows = totalRows;
    d.batch = 1;
    d.nHeads = nHeads;
    d.nKV = nKV;
    d.hd = hd;
    d.maxLen = cachePos + 1;
    d.numChunks = numChunks;
    d.invSqrt = invSqrt;
    return tc::decodeI8Common(&d, cachePos + 1, devPos ? 1u : 0u, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
