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
#include <cstdlib>
#include <mutex>

#include "decode_shared.cuh"

namespace tc {

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
    uint32_t colBase;  // heads mode: the 8 MMA columns are q heads colBase .. colBase + 7 of the kv head
    uint32_t chunkTokens, numChunks;
    uint32_t prefetchRows;  // rows [0, prefetchRows) of a sequence may be read before the dependency wait
    // rows mode (causal prefill over the store): the 8 MMA columns of a CTA are 8
    // consecutive query rows of ONE q head instead of the q heads of one kv head;
    // row s attends pool rows [0, cachePos + s].  grid = (1, nHeads, ceil(qRows / 8)).
    uint32_t rowsMode, qRows, cachePos;
    const uint32_t *devPos;
    float invSqrt;
    int directOut;
    int prefetchNext;  // tmKn / tmVn describe the pools of the next call: pull this block's rows of them into L2
    unsigned int *err;
};

constexpr int kHD = 128;

// TC_ATTN_LEGACY_DECODE=1 keeps head_dim 128 on the mma.sync kernel (comparison runs)
static bool forceLegacyDecode() {
    static const bool v = [] {
        const char *e = getenv("TC_ATTN_LEGACY_DECODE");
        return e != nullptr && e[0] == '1';
    }();
    return v;
}
// MT = 16-row MMA tiles one consumer warp folds per stage: 2 amortises the softmax
// bookkeeping over 32 tokens (large problems), 1 halves the work quantum so that a
// small problem still spreads evenly over 148 SMs x 8 warps.
//
// A stage holds K then V; each is stored as HD/128 half-tiles of [rows][128 bytes]
// (the 128-byte swizzle spans exactly one half-row), half-tile h covering dims
// [128h, 128h + 128).
template <int HD, int HPC, int NW, int NSTAGE, int MT>
struct DecodeI8Smem {
    static constexpr int kTokPerWarp = 16 * MT;
    static constexpr int kRows = NW * kTokPerWarp;       // (token, head) rows per stage
    static constexpr int T = kRows / HPC;                 // tokens per stage
    static constexpr int kHalfBytes = kRows * 128;        // one half-tile, all HPC heads
    static constexpr int kTileBytes = kRows * HD;         // K (or V) bytes per stage, all HPC heads
    static constexpr int kScaleBytes = kRows * 4;
    static constexpr int kStageBytes = 2 * kTileBytes + 2 * kScaleBytes;
    static constexpr int kBarOffset = NSTAGE * kStageBytes;
    static constexpr int kTotal = kBarOffset + 2 * NSTAGE * 8 + 1024;  // + alignment slack
    static_assert(kStageBytes % 1024 == 0, "stage must keep 1024-byte alignment for the 128B swizzle");
    static_assert(T <= 256, "TMA box rows");
};

// How far the running reference point of the softmax may lag behind the true
// maximum (log2 units) before the accumulators are rescaled.  p stays <= 2^8.
constexpr float kLazyLog2 = 8.0f;
// Stages a producer may request before the grids it depends on have completed.
constexpr uint32_t kEarlyStages = 1;

template <int HD, int HPC, int NW, int NSTAGE, int MT>
__global__ void __launch_bounds__((NW + 1) * 32, 1)
decodeI8Kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmKn, const __grid_constant__ CUtensorMap tmVn,
               const DecodeI8Params p) {
    using L = DecodeI8Smem<HD, HPC, NW, NSTAGE, MT>;
    constexpr int T = L::T;
    constexpr int NC = HD / 16;  // 16-dim groups of a head vector
    constexpr int kTokPerWarp = L::kTokPerWarp;
    constexpr int NR = 2 * MT;  // 8-token row groups of a warp's tile
    constexpr int NSUB = NW / HPC;  // consumer warps per kv head
    constexpr float k2p24 = 16777216.0f;

    const uint32_t chunk = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *fullBar = reinterpret_cast<uint64_t *>(smem + L::kBarOffset);
    uint64_t *emptyBar = fullBar + NSTAGE;

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
    gridDepLaunch();  // the dependent grid (the merge) may be scheduled as soon as room frees up

    // The length may live in device memory written by an earlier kernel; only a
    // host-known length lets the producer start before the dependency wait.
    uint32_t len = p.lenHost;
    const bool earlyOk = p.devLens == nullptr && p.devRowBase == nullptr && p.prefetchRows != 0 && !p.rowsMode;
    if (!earlyOk) {
        gridDepWait();
        if (p.devLens) len = p.devLens[b] + p.lenAdd;
    }
    uint32_t rowsPos = p.cachePos;  // rows mode: first query row sits at pool row rowsPos
    if (p.rowsMode) {
        if (p.devPos) rowsPos = p.devPos[0];
        const uint32_t sEnd = min(p.qRows, b * 8u + 8u);  // b = row block
        len = rowsPos + sEnd;                             // the block's last row sees [0, rowsPos + sEnd)
    }
    const uint32_t t0 = chunk * p.chunkTokens;
    if (t0 >= len) return;  // inactive chunk: the merge derives the active count from len
    const uint32_t t1 = min(len, t0 + p.chunkTokens);
    const uint32_t nTiles = (t1 - t0 + T - 1) / T;
    const uint64_t rowBase = p.rowsMode ? 0ull
                                        : (p.devRowBase ? p.devRowBase[b] : static_cast<uint64_t>(b) * p.rowsPerSeq);
    // kv heads of this CTA: heads mode streams HPC of them, rows mode the one behind q head `hg`
    const uint32_t kvHead0 = p.rowsMode ? hg / p.group : hg * HPC;

    if (warp == NW) {
        // ------------------------------ producer ------------------------------
        bool waited = !earlyOk;
        for (uint32_t it = 0; it < nTiles; ++it) {
            const uint32_t s = it % NSTAGE;
            if (it >= NSTAGE) {
                if (!mbarWaitClock(&emptyBar[s], ((it / NSTAGE) - 1) & 1, p.err, kDevErrEmptyWait)) break;
            }
            const uint32_t tok = t0 + it * T;
            if (!waited && (tok + T > p.prefetchRows || it >= kEarlyStages)) {
                // this tile may hold rows appended by the kernel we depend on -- or it is not
                // the first one: the kernels ahead (the merge above all) are short and
                // latency-bound, and a deeper prefetch would put a whole ring of KV loads
                // in front of theirs in the memory system
                gridDepWait();
                waited = true;
            }
            uint8_t *st = smem + s * L::kStageBytes;
            const uint64_t row = rowBase + tok;
            if (lane == 0) {
                mbarExpectTx(&fullBar[s], 2 * L::kTileBytes);
#pragma unroll
                for (int h = 0; h < HPC; ++h) {
#pragma unroll
                    for (int hf = 0; hf < HD / 128; ++hf) {
                        uint8_t *dst = st + hf * L::kHalfBytes + h * T * 128;
                        tmaLoad3D(dst, &tmK, &fullBar[s], hf * 128, kvHead0 + h, static_cast<int>(row));
                        tmaLoad3D(dst + L::kTileBytes, &tmV, &fullBar[s], hf * 128, kvHead0 + h,
                                  static_cast<int>(row));
                    }
                }
            }
            float *sK = reinterpret_cast<float *>(st + 2 * L::kTileBytes);
            float *sV = sK + L::kRows;
#pragma unroll
            for (int idx = lane; idx < L::kRows; idx += 32) {
                const int h = idx / T, tt = idx % T;
                uint64_t r = row + tt;
                r = r < p.totalRows ? r : p.totalRows - 1;
                cpAsync4(&sK[idx], p.ks + r * p.nKV + kvHead0 + h);
                cpAsync4(&sV[idx], p.vs + r * p.nKV + kvHead0 + h);
            }
            cpAsyncMbarArriveNoinc(&fullBar[s]);
        }
        if (p.prefetchNext && lane == 0) {
            // This block's own tiles are all requested.  DRAM would now idle through the fold, the
            // merge and the next call's start-up: have it fetch the same rows of the next call's
            // pools into L2 meanwhile (the next call's TMA loads then hit L2).
            for (uint32_t it = 0; it < nTiles; ++it) {
                const int row = static_cast<int>(rowBase + t0 + it * T);
#pragma unroll
                for (int h = 0; h < HPC; ++h)
#pragma unroll
                    for (int hf = 0; hf < HD / 128; ++hf) {
                        tmaPrefetchL2_3D(&tmKn, hf * 128, kvHead0 + h, row);
                        tmaPrefetchL2_3D(&tmVn, hf * 128, kvHead0 + h, row);
                    }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    if (earlyOk) gridDepWait();  // q comes from a kernel that may still be running
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t hL = warp % HPC, sub = warp / HPC;
    const uint32_t kvHead = kvHead0 + hL;
    // What MMA column j (0..7) of this warp stands for.
    auto colValid = [&](uint32_t j) { return p.rowsMode ? (b * 8u + j < p.qRows) : (p.colBase + j < p.group); };
    auto colIndex = [&](uint32_t j) -> size_t {  // index of the column's q / out vector, in units of HD
        return p.rowsMode ? (static_cast<size_t>(b) * 8u + j) * p.nHeads + hg
                          : static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + j;
    };
    // exclusive row bound of a column: everything in heads mode, causal in rows mode
    auto colLen = [&](uint32_t j) { return p.rowsMode ? min(t1, rowsPos + b * 8u + j + 1u) : t1; };

    // q fragments for head column n = g of this kv head's group: power-of-two
    // normalised, split into fp16 hi + lo, laid out as the B operand whose k
    // slots follow the byte order ldmatrix hands out (dims 16c + 4t + {0..3}).
    uint32_t qhi[NC][2], qlo[NC][2];
    float headScale, headOff;
    {
        float4 qv[NC];
        float amax = 0.0f;
        const bool valid = colValid(g);
        const float *qp = p.q + colIndex(valid ? g : 0) * HD;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
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
        float qsum = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            float h0, l0, h1, l1, h2, l2, h3, l3;
            splitHalf(qv[c].x * down, h0, l0);
            splitHalf(qv[c].y * down, h1, l1);
            splitHalf(qv[c].z * down, h2, l2);
            splitHalf(qv[c].w * down, h3, l3);
            qhi[c][0] = packHalf2(h0, h1);
            qhi[c][1] = packHalf2(h2, h3);
            qlo[c][0] = packHalf2(l0, l1);
            qlo[c][1] = packHalf2(l2, l3);
            // the column sum the MMA really sees: the fp16-rounded parts
            const __half2 a = *reinterpret_cast<__half2 *>(&qlo[c][0]), bb = *reinterpret_cast<__half2 *>(&qlo[c][1]);
            qsum += (h0 + __low2float(a)) + (h1 + __high2float(a)) + (h2 + __low2float(bb)) + (h3 + __high2float(bb));
        }
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
        headOff = 128.0f * qsum;  // K bytes enter the MMA as x + 128
    }
    // score columns of this thread are heads 2t and 2t+1: fetch their constants
    const float cs0 = __shfl_sync(0xffffffffu, headScale, (2 * t) * 4);
    const float cs1 = __shfl_sync(0xffffffffu, headScale, (2 * t + 1) * 4);
    const float off0 = __shfl_sync(0xffffffffu, headOff, (2 * t) * 4);
    const float off1 = __shfl_sync(0xffffffffu, headOff, (2 * t + 1) * 4);
    const uint32_t len0 = colLen(2 * t), len1 = colLen(2 * t + 1);

    float m0 = kNegBig, m1 = kNegBig, l0 = 0.0f, l1 = 0.0f;
    float ps0 = 0.0f, ps1 = 0.0f;  // sum of p*sv as fed to the PV MMA (V bytes enter as x + 128)
    uint32_t Ebits = 0;            // running power-of-two scale of the V row scales (0 = unset)
    float invE = 0.0f;
    float o[NC][4];
#pragma unroll
    for (int i = 0; i < NC; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    const uint32_t lr = (lane & 7u) + ((lane >> 3) & 1u) * 8u;  // ldmatrix row this lane addresses
    const uint32_t lco = lane >> 4;                             // and which chunk of the pair
    const uint32_t lmOff = lr * 128;

    for (uint32_t it = 0; it < nTiles; ++it) {
        const uint32_t s = it % NSTAGE;
        if (!mbarWaitClock(&fullBar[s], (it / NSTAGE) & 1, p.err, kDevErrFullWait)) break;
        uint8_t *st = smem + s * L::kStageBytes;
        const uint32_t rowInTile = hL * T + sub * kTokPerWarp;
        const float *sK = reinterpret_cast<const float *>(st + 2 * L::kTileBytes) + rowInTile;
        const float *sV = sK + L::kRows;
        const uint32_t tokBase = t0 + it * T + sub * kTokPerWarp + g;
        bool vl0[NR], vl1[NR];
        float skr[NR], svr[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {  // rows g, g+8, ... of this warp's tokens
            vl0[r] = tokBase + 8 * r < len0;
            vl1[r] = tokBase + 8 * r < len1;
            skr[r] = sK[g + 8 * r];
            svr[r] = tokBase + 8 * r < t1 ? sV[g + 8 * r] : 0.0f;
        }

        // ---- S^T = K . Q^T, two 16-token tiles x 8 heads ----
        float sh[MT][4], sl[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) sh[mt][i] = sl[mt][i] = 0.0f;
        const uint32_t kTile = smemAddr(st + rowInTile * 128);
#pragma unroll
        for (int cp = 0; cp < NC / 2; ++cp) {
            const uint32_t sw = (((2 * (cp & 3) + lco) ^ (lr & 7u)) << 4) + (cp >> 2) * L::kHalfBytes;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t r0, r1, r2, r3;
                ldmatrixX4(r0, r1, r2, r3, kTile + mt * 2048 + lmOff + sw);
                r0 ^= 0x80808080u;
                r1 ^= 0x80808080u;
                r2 ^= 0x80808080u;
                r3 ^= 0x80808080u;
                {
                    const uint32_t a0 = subnormalPair<0x4140>(r0), a1 = subnormalPair<0x4140>(r1),
                                   a2 = subnormalPair<0x4342>(r0), a3 = subnormalPair<0x4342>(r1);
                    mmaF16(sh[mt], a0, a1, a2, a3, qhi[2 * cp][0], qhi[2 * cp][1]);
                    mmaF16(sl[mt], a0, a1, a2, a3, qlo[2 * cp][0], qlo[2 * cp][1]);
                }
                {
                    const uint32_t a0 = subnormalPair<0x4140>(r2), a1 = subnormalPair<0x4140>(r3),
                                   a2 = subnormalPair<0x4342>(r2), a3 = subnormalPair<0x4342>(r3);
                    mmaF16(sh[mt], a0, a1, a2, a3, qhi[2 * cp + 1][0], qhi[2 * cp + 1][1]);
                    mmaF16(sl[mt], a0, a1, a2, a3, qlo[2 * cp + 1][0], qlo[2 * cp + 1][1]);
                }
            }
        }
        // log2-domain scores: undo the 2^-24 of the subnormal operand and the +128 offset,
        // apply the row's K scale; rows past the range are masked out
        float sc[NR][2];  // [row r][head 2t / 2t+1]
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = 2 * mt + hf;
                const float d0 = fmaf(sh[mt][2 * hf] + sl[mt][2 * hf], k2p24, -off0);
                const float d1 = fmaf(sh[mt][2 * hf + 1] + sl[mt][2 * hf + 1], k2p24, -off1);
                sc[r][0] = vl0[r] ? d0 * (skr[r] * cs0) : -INFINITY;
                sc[r][1] = vl1[r] ? d1 * (skr[r] * cs1) : -INFINITY;
            }
        }
        float mx0 = fmaxf(sc[0][0], sc[1][0]), mx1 = fmaxf(sc[0][1], sc[1][1]);
        float svmax = fmaxf(svr[0], svr[1]);
#pragma unroll
        for (int r = 2; r < NR; ++r) {
            mx0 = fmaxf(mx0, sc[r][0]);
            mx1 = fmaxf(mx1, sc[r][1]);
            svmax = fmaxf(svmax, svr[r]);
        }
#pragma unroll
        for (int off = 4; off <= 16; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        // lazy reference point: move it only when the maximum ran ahead by 2^8
        const float mn0 = mx0 > m0 + kLazyLog2 ? mx0 : m0;
        const float mn1 = mx1 > m1 + kLazyLog2 ? mx1 : m1;
        // running power-of-two bound of the V scales (keeps p*sv inside fp16)
        uint32_t eb = __reduce_max_sync(0xffffffffu, __float_as_uint(svmax)) & 0x7f800000u;
        eb = min(eb, 253u << 23);
        float fE = 1.0f;
        if (eb > Ebits) {
            const float newInv = __uint_as_float((254u << 23) - eb);
            fE = Ebits ? __uint_as_float(Ebits) * newInv : 1.0f;
            Ebits = eb;
            invE = newInv;
        }
        if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1 || fE != 1.0f)) {
            const float a0s = fastExp2(m0 - mn0), a1s = fastExp2(m1 - mn1);
            const float al0 = a0s * fE, al1 = a1s * fE;
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                o[i][0] *= al0;
                o[i][1] *= al1;
                o[i][2] *= al0;
                o[i][3] *= al1;
            }
            l0 *= a0s;
            l1 *= a1s;
            ps0 *= al0;
            ps1 *= al1;
            m0 = mn0;
            m1 = mn1;
        }
        // p, then p * sv scaled into fp16 range, hi + lo, transposed to the B layout
        uint32_t bh[MT][2], bl[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int r = 2 * mt + hf;
                const float p0 = fastExp2(sc[r][0] - m0), p1 = fastExp2(sc[r][1] - m1);
                l0 += p0;
                l1 += p1;
                const float w = svr[r] * invE;
                const float x0 = p0 * w, x1 = p1 * w;
                const uint32_t hi = packHalf2(x0, x1);
                const __half2 hh = *reinterpret_cast<const __half2 *>(&hi);
                const float r0 = x0 - __low2float(hh), r1 = x1 - __high2float(hh);
                const uint32_t lo = packHalf2(r0, r1);
                const __half2 ll = *reinterpret_cast<const __half2 *>(&lo);
                ps0 += __low2float(hh) + __low2float(ll);
                ps1 += __high2float(hh) + __high2float(ll);
                bh[mt][hf] = movmatrixTrans(hi);
                bl[mt][hf] = movmatrixTrans(lo);
            }
        }
        // ---- O^T += V^T . P^T (HD dims x 8 heads), V bytes read transposed ----
        const uint32_t vTile = smemAddr(st + L::kTileBytes + rowInTile * 128);
#pragma unroll
        for (int cp = 0; cp < NC / 2; ++cp) {
            const uint32_t sw = (((2 * (cp & 3) + lco) ^ (lr & 7u)) << 4) + (cp >> 2) * L::kHalfBytes;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t r0, r1, r2, r3;
                ldmatrixX4Trans(r0, r1, r2, r3, vTile + mt * 2048 + lmOff + sw);
                r0 ^= 0x80808080u;
                r1 ^= 0x80808080u;
                r2 ^= 0x80808080u;
                r3 ^= 0x80808080u;
                {
                    // rows g / g+8 of this MMA tile are dims 16c+2g / 16c+2g+1, c = 2cp
                    const uint32_t a0 = subnormalPair<0x4240>(r0), a1 = subnormalPair<0x4341>(r0),
                                   a2 = subnormalPair<0x4240>(r1), a3 = subnormalPair<0x4341>(r1);
                    mmaF16(o[2 * cp], a0, a1, a2, a3, bh[mt][0], bh[mt][1]);
                    mmaF16(o[2 * cp], a0, a1, a2, a3, bl[mt][0], bl[mt][1]);
                }
                {
                    const uint32_t a0 = subnormalPair<0x4240>(r2), a1 = subnormalPair<0x4341>(r2),
                                   a2 = subnormalPair<0x4240>(r3), a3 = subnormalPair<0x4341>(r3);
                    mmaF16(o[2 * cp + 1], a0, a1, a2, a3, bh[mt][0], bh[mt][1]);
                    mmaF16(o[2 * cp + 1], a0, a1, a2, a3, bl[mt][0], bl[mt][1]);
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
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, off);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, off);
    }
    namedBarSync(1, NW * 32);  // every consumer is done reading the ring
    float *scr = reinterpret_cast<float *>(smem);
    constexpr int kWarpScr = 8 * HD + 16;
    float *wO = scr + warp * kWarpScr;  // [8 heads][HD], then m[8], l[8]
    {
        // true accumulator = 2^24 * raw - 128 * sum(p*sv), then back from the E-scaled domain
        const float E = __uint_as_float(Ebits);
        const float c0 = 128.0f * ps0, c1 = 128.0f * ps1;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int d = 16 * c + 2 * g;
            *reinterpret_cast<float2 *>(wO + (2 * t) * HD + d) =
                    make_float2(fmaf(o[c][0], k2p24, -c0) * E, fmaf(o[c][2], k2p24, -c0) * E);
            *reinterpret_cast<float2 *>(wO + (2 * t + 1) * HD + d) =
                    make_float2(fmaf(o[c][1], k2p24, -c1) * E, fmaf(o[c][3], k2p24, -c1) * E);
        }
    }
    if (g == 0) {
        wO[8 * HD + 2 * t] = m0;
        wO[8 * HD + 2 * t + 1] = m1;
        wO[8 * HD + 8 + 2 * t] = l0;
        wO[8 * HD + 8 + 2 * t + 1] = l1;
    }
    namedBarSync(1, NW * 32);
    // NW*32 threads, HPC*8*(HD/4) float4 outputs
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
        // column -> output vector (same rule as colIndex, for kv head kvHead0 + h)
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
                // back to natural-log units: the merge contract is w = exp2((m - M) * log2e)
                p.pM[pidx] = M > -1e29f ? M * 0.6931471805599453f : kNegBig;
                p.pL[pidx] = lsum;
            }
        }
    }
}

template <int HD, int HPC, int MT>
static int launchDecodeI8(const CUtensorMap &tmK, const CUtensorMap &tmV, const CUtensorMap &tmKn,
                          const CUtensorMap &tmVn, const DecodeI8Params &prm, const DecodePlan &pl, uint32_t batch,
                          bool pdl, cudaStream_t st) {
    constexpr int NW = 8, NSTAGE = (MT == 2 || HD == 256) ? 3 : 6;
    using L = DecodeI8Smem<HD, HPC, NW, NSTAGE, MT>;
    static_assert(L::kTotal <= 227 * 1024, "stage ring exceeds the shared memory of an SM");
    auto kern = decodeI8Kernel<HD, HPC, NW, NSTAGE, MT>;
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
        attrDone[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.chunksPerSeq, pl.headGroups, batch);
    cfg.blockDim = dim3((NW + 1) * 32);
    cfg.dynamicSmemBytes = L::kTotal;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    TC_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmK, tmV, tmKn, tmVn, prm));
    return TC_OK;
}

static int decodeI8Common(const tc_decode_i8_batch *d, uint32_t lenHost, uint32_t lenAdd, cudaStream_t st) {
    TC_REQUIRE(d->q && d->out && d->k8 && d->v8 && d->ks && d->vs, TC_EINVAL, "decode_i8: null pointer");
    TC_REQUIRE(d->hd == 128 || d->hd == 256, TC_EUNSUPPORTED, "decode_i8: head_dim %u (built for 128 and 256)",
               d->hd);
    const uint32_t hd = d->hd;
    TC_REQUIRE(d->nKV > 0 && d->nHeads % d->nKV == 0, TC_EINVAL, "decode_i8: nHeads %u not a multiple of nKV %u",
               d->nHeads, d->nKV);
    const uint32_t group = d->nHeads / d->nKV;
    TC_REQUIRE(group <= 64, TC_EUNSUPPORTED, "decode_i8: %u q heads per kv head (built for <= 64)", group);
    TC_REQUIRE(d->batch >= 1 && d->batch <= 65535, TC_EINVAL, "decode_i8: batch %u", d->batch);
    TC_REQUIRE(d->maxLen >= 1, TC_EINVAL, "decode_i8: empty context");
    TC_REQUIRE(d->totalRows >= 1 && d->totalRows < (1ull << 31), TC_EUNSUPPORTED,
               "decode_i8: pool of %llu rows", (unsigned long long) d->totalRows);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(d->k8) | reinterpret_cast<uintptr_t>(d->v8) |
                 reinterpret_cast<uintptr_t>(d->q) | reinterpret_cast<uintptr_t>(d->out)) & 15u) == 0,
               TC_EINVAL, "decode_i8: q/out/k8/v8 need 16-byte alignment");
    TC_REQUIRE(d->numChunks >= 1, TC_EWORKSPACE, "decode_i8: no chunk slots");
    // head_dim 128 runs on the tcgen05 integer path; this file's mma.sync kernel keeps head_dim
    // 256 and the causal rows mode
    TC_REQUIRE((d->appendK == nullptr) == (d->appendV == nullptr), TC_EINVAL, "decode_i8: appendK and appendV come together");
    if (hd == 128 && !forceLegacyDecode()) return decodeI8Tc(d, lenHost, lenAdd, st);
    if (d->appendK != nullptr) {
        // this file's kernel reads the pool only: the new rows go in with the quantise launch
        const int rc = tc_kv_quantize_i8_batch(d->appendK, d->appendV, const_cast<int8_t *>(d->k8),
                                               const_cast<int8_t *>(d->v8), const_cast<float *>(d->ks),
                                               const_cast<float *>(d->vs), d->batch, d->nKV, hd, d->rowsPerSeq, d->rowBase,
                                               lenHost - 1u, d->lens, static_cast<int32_t>(lenAdd) - 1, d->totalRows, st);
        if (rc != TC_OK) return rc;
    }
    // work quantum: 32 tokens per warp when every warp of the machine gets at least ~12
    // of them, 16 otherwise (see DecodeI8Smem)
    const uint64_t warpTiles32 = static_cast<uint64_t>(d->batch) * d->nKV * ((d->maxLen + 31) / 32);
    // (head_dim 256: a 32-token tile of K and V no longer leaves room for a second stage)
    const uint32_t mt = hd == 128 && warpTiles32 >= 2ull * 8ull * static_cast<uint64_t>(numSMs()) ? 2u : 1u;
    const DecodePlan pl = planDecode(d->batch, d->nKV, d->maxLen, d->numChunks, 8u * 16u * mt, d->lens == nullptr);
    const bool pdl = (d->flags & TC_DECODE_PDL) != 0;
    const bool direct = pl.chunksPerSeq == 1 && !d->partialsOnly;
    if (!direct)
        TC_REQUIRE(d->pAcc && d->pM && d->pL, TC_EWORKSPACE, "decode_i8: partial buffers are required");
    if (d->chunksUsed) *d->chunksUsed = pl.chunksPerSeq;

    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.rank = 3;
    key.elemBytes = 1;
    key.swizzle = 3;
    key.dims[0] = hd;
    key.dims[1] = d->nKV;
    key.dims[2] = d->totalRows;
    key.strides[0] = hd;
    key.strides[1] = static_cast<uint64_t>(d->nKV) * hd;
    key.box[0] = 128;  // one swizzle span; a 256-dim row is fetched as two boxes
    key.box[1] = 1;
    key.box[2] = pl.tileTokens;
    CUtensorMap tmK, tmV;
    key.base = d->k8;
    int rc = getTensorMap(key, &tmK);
    if (rc != TC_OK) return rc;
    key.base = d->v8;
    rc = getTensorMap(key, &tmV);
    if (rc != TC_OK) return rc;
    // the pools of the next call, for the L2 prefetch hint (same geometry)
    CUtensorMap tmKn = tmK, tmVn = tmV;
    // Only when a call's rows fit into L2 next to the rows still in flight: a prefetch of more than
    // that is evicted before it is used and costs the DRAM traffic twice (8 sequences of 32768 rows,
    // 277 MB per call: 0.87 of the copy peak without the hint, 0.74 with it).
    const uint64_t callBytes = static_cast<uint64_t>(d->batch) * d->maxLen * d->nKV * hd * 2ull;
    const bool prefetchNext = d->nextK8 != nullptr && d->nextV8 != nullptr && callBytes <= (48ull << 20);
    if (prefetchNext) {
        TC_REQUIRE(((reinterpret_cast<uintptr_t>(d->nextK8) | reinterpret_cast<uintptr_t>(d->nextV8)) & 15u) == 0,
                   TC_EINVAL, "decode_i8: nextK8/nextV8 need 16-byte alignment");
        key.base = d->nextK8;
        rc = getTensorMap(key, &tmKn);
        if (rc != TC_OK) return rc;
        key.base = d->nextV8;
        rc = getTensorMap(key, &tmVn);
        if (rc != TC_OK) return rc;
    }

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
    prm.prefetchRows = pdl ? d->prefetchRows : 0;
    prm.rowsMode = 0;
    prm.qRows = 0;
    prm.cachePos = 0;
    prm.devPos = nullptr;
    prm.invSqrt = d->invSqrt;
    prm.directOut = direct ? 1 : 0;
    prm.prefetchNext = prefetchNext ? 1 : 0;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "decode_i8: no device error word");

    // a launch serves 8 q heads per kv head (the MMA columns); wider groups take one launch per
    // block of 8 and stream the rows again
    for (uint32_t cb = 0; cb < group; cb += 8) {
        prm.colBase = cb;
        if (hd == 256) {
            if (pl.hpc == 4) rc = launchDecodeI8<256, 4, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else if (pl.hpc == 2) rc = launchDecodeI8<256, 2, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else rc = launchDecodeI8<256, 1, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
        } else if (mt == 2) {
            if (pl.hpc == 4) rc = launchDecodeI8<128, 4, 2>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else if (pl.hpc == 2) rc = launchDecodeI8<128, 2, 2>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else rc = launchDecodeI8<128, 1, 2>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
        } else {
            if (pl.hpc == 4) rc = launchDecodeI8<128, 4, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else if (pl.hpc == 2) rc = launchDecodeI8<128, 2, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
            else rc = launchDecodeI8<128, 1, 1>(tmK, tmV, tmKn, tmVn, prm, pl, d->batch, pdl, st);
        }
        if (rc != TC_OK) return rc;
    }
    if (rc != TC_OK) return rc;
    if (direct || d->partialsOnly) return TC_OK;
    // merge: the active chunk count of a sequence follows from its length (read on
    // the device when the length lives there); slots past it were never written.
    return launchMerge(d->pAcc, d->pM, d->pL, d->out, d->batch, d->nHeads, d->numChunks, pl.chunksPerSeq, hd,
                       d->lens, lenAdd, pl.chunkTokens, nullptr, pdl, st);
}

// Causal prefill over the int8 store: the decode kernel with query rows as MMA columns.
static int prefillI8(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                     float *out, uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos,
                     const uint32_t *devPos, uint64_t totalRows, float invSqrt, cudaStream_t st) {
    TC_REQUIRE(q && k8 && v8 && ks && vs && out, TC_EINVAL, "prefill_i8: null pointer");
    TC_REQUIRE(hd == 128 || hd == 256, TC_EUNSUPPORTED, "prefill_i8: head_dim %u (built for 128 and 256)", hd);
    TC_REQUIRE(nKV > 0 && nHeads % nKV == 0, TC_EINVAL, "prefill_i8: nHeads %u not a multiple of nKV %u", nHeads,
               nKV);
    TC_REQUIRE(totalRows >= 1 && totalRows < (1ull << 31), TC_EUNSUPPORTED, "prefill_i8: pool of %llu rows",
               (unsigned long long) totalRows);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8) | reinterpret_cast<uintptr_t>(q) |
                 reinterpret_cast<uintptr_t>(out)) & 15u) == 0,
               TC_EINVAL, "prefill_i8: q/out/k8/v8 need 16-byte alignment");
    if (seqLen == 0) return TC_OK;
    if (devPos == nullptr && static_cast<uint64_t>(cachePos) + seqLen > totalRows) {
        setError("prefill_i8: rows [%u, %llu) pass the pool of %llu rows", cachePos,
                 (unsigned long long) cachePos + seqLen, (unsigned long long) totalRows);
        return TC_ECONTEXT_FULL;
    }
    const uint32_t rowBlocks = (seqLen + 7) / 8;
    TC_REQUIRE(rowBlocks <= 65535 && nHeads <= 65535, TC_EUNSUPPORTED, "prefill_i8: %u rows x %u heads", seqLen,
               nHeads);
    // tokens per stage: 8 warps x 32 rows (head_dim 128) or x 16 rows (head_dim 256)
    const uint32_t tileTokens = hd == 256 ? 128u : 256u;
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.rank = 3;
    key.elemBytes = 1;
    key.swizzle = 3;
    key.dims[0] = hd;
    key.dims[1] = nKV;
    key.dims[2] = totalRows;
    key.strides[0] = hd;
    key.strides[1] = static_cast<uint64_t>(nKV) * hd;
    key.box[0] = 128;
    key.box[1] = 1;
    key.box[2] = tileTokens;
    CUtensorMap tmK, tmV;
    key.base = k8;
    int rc = getTensorMap(key, &tmK);
    if (rc != TC_OK) return rc;
    key.base = v8;
    rc = getTensorMap(key, &tmV);
    if (rc != TC_OK) return rc;
    DecodeI8Params prm;
    memset(&prm, 0, sizeof(prm));
    prm.q = q;
    prm.out = out;
    prm.ks = ks;
    prm.vs = vs;
    prm.totalRows = totalRows;
    prm.nHeads = nHeads;
    prm.nKV = nKV;
    prm.group = nHeads / nKV;
    prm.chunkTokens = 0xffffff00u;  // one chunk: a block streams its whole causal prefix
    prm.numChunks = 1;
    prm.rowsMode = 1;
    prm.qRows = seqLen;
    prm.cachePos = cachePos;
    prm.devPos = devPos;
    prm.invSqrt = invSqrt;
    prm.directOut = 1;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "prefill_i8: no device error word");
    DecodePlan pl;
    pl.hpc = 1;
    pl.headGroups = nHeads;
    pl.chunksPerSeq = 1;
    pl.chunkTokens = prm.chunkTokens;
    pl.tileTokens = tileTokens;
    // heaviest row blocks first would need a reversed grid; the hardware scheduler
    // hands out blocks in z-major order, so late (long) blocks start last -- acceptable here
    if (hd == 256) return launchDecodeI8<256, 1, 1>(tmK, tmV, tmK, tmV, prm, pl, rowBlocks, false, st);
    return launchDecodeI8<128, 1, 2>(tmK, tmV, tmK, tmV, prm, pl, rowBlocks, false, st);
}

}  // namespace tc

extern "C" {

int tc_attn_prefill_i8(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                       float *out, uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos,
                       const uint32_t *devPos, uint64_t totalRows, float invSqrt, tc_stream stream) {
    return tc::prefillI8(q, k8, v8, ks, vs, out, seqLen, nHeads, nKV, hd, cachePos, devPos, totalRows, invSqrt,
                         static_cast<cudaStream_t>(stream));
}

int tc_attn_decode_i8_batch(const tc_decode_i8_batch *d, tc_stream stream) {
    TC_REQUIRE(d != nullptr, TC_EINVAL, "tc_attn_decode_i8_batch: null descriptor");
    return tc::decodeI8Common(d, d->maxLen, 0, static_cast<cudaStream_t>(stream));
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

// ---------------------------------------------------------------------------------
// A decode entry point that allocates nothing
// ---------------------------------------------------------------------------------
// Some callers hold no allocator they may use at the moment attention runs: a host
// that hands this library bare device pointers from a memory plan frozen at load
// time, or a latency-critical serving loop that must not touch the device allocator
// once it is running.  For them the split-KV partials (the only scratch this kernel needs)
// live in a fixed array inside the library's own device image instead of in
// caller-provided buffers.  Every GPU that loads the library carries the array
// (kNoAllocBytes, about 5.3 MB) until the process exits.
constexpr uint32_t kNoAllocMaxHeads = 64;    // q heads
constexpr uint32_t kNoAllocChunks = 160;     // chunk slots per head (one per SM and a few spare)
constexpr size_t kNoAllocAccFloats = static_cast<size_t>(kNoAllocMaxHeads) * kNoAllocChunks * tc::kHD;
constexpr size_t kNoAllocMLFloats = static_cast<size_t>(kNoAllocMaxHeads) * kNoAllocChunks;
constexpr size_t kNoAllocBytes = (kNoAllocAccFloats + 2 * kNoAllocMLFloats) * sizeof(float);
static __device__ __align__(256) float g_noAllocScratch[kNoAllocAccFloats + 2 * kNoAllocMLFloats];

// In host code the array's name is only a handle for the runtime, not a device
// address, so the address is asked for once per device (with that device current)
// and remembered.
static int noAllocScratch(float **ptr) {
    static std::mutex mu;
    static float *addr[64] = {nullptr};
    int dev = 0;
    TC_CUDA_OK(cudaGetDevice(&dev));
    TC_REQUIRE(dev >= 0 && dev < 64, TC_EUNSUPPORTED, "tc_attn_decode_i8_noalloc: device ordinal %d", dev);
    std::lock_guard<std::mutex> lk(mu);
    if (addr[dev] == nullptr) {
        void *p = nullptr;
        TC_CUDA_OK(cudaGetSymbolAddress(&p, g_noAllocScratch));
        addr[dev] = static_cast<float *>(p);
    }
    *ptr = addr[dev];
    return TC_OK;
}

int tc_attn_decode_i8_noalloc(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                              float *out, uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t cachePos,
                              uint64_t totalRows, float invSqrt, tc_stream stream) {
    TC_REQUIRE(nHeads >= 1 && nHeads <= kNoAllocMaxHeads, TC_EWORKSPACE,
               "tc_attn_decode_i8_noalloc: %u q heads, the built-in scratch holds at most %u", nHeads,
               kNoAllocMaxHeads);
    TC_REQUIRE(hd == static_cast<uint32_t>(tc::kHD), TC_EWORKSPACE,
               "tc_attn_decode_i8_noalloc: head_dim %u, the built-in scratch is laid out for %d", hd, tc::kHD);
    TC_REQUIRE(static_cast<uint64_t>(cachePos) + 1 <= totalRows, TC_ECONTEXT_FULL,
               "tc_attn_decode_i8_noalloc: position %u is outside the pool of %llu rows", cachePos,
               (unsigned long long) totalRows);
    float *scratch = nullptr;
    const int rc = noAllocScratch(&scratch);
    if (rc != TC_OK) return rc;
    tc_decode_i8_batch d;
    memset(&d, 0, sizeof(d));
    d.q = q;
    d.out = out;
    d.k8 = k8;
    d.v8 = v8;
    d.ks = ks;
    d.vs = vs;
    // the three partial arrays are carved out of the one array; nothing in them has to
    // start at zero (the merge reads only the chunk slots this call wrote)
    d.pAcc = scratch;
    d.pM = scratch + kNoAllocAccFloats;
    d.pL = scratch + kNoAllocAccFloats + kNoAllocMLFloats;
    d.totalRows = totalRows;
    d.batch = 1;
    d.nHeads = nHeads;
    d.nKV = nKV;
    d.hd = hd;
    d.maxLen = cachePos + 1;
    d.numChunks = kNoAllocChunks;
    d.invSqrt = invSqrt;
    return tc::decodeI8Common(&d, cachePos + 1, 0u, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
