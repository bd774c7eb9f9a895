// decode_i8_tc.cu -- split-KV decode attention over the int8 store on the 5th-generation
// tensor cores (tcgen05.mma kind::i8, accumulators in TMEM), head_dim 128.
//
// What it replaces: kQ35WarpAttention8Split (+ kAttnCombinePartial) and the eager
// kQ35WarpAttention8 of the reference (include/gpu/GpuQwen35Kernels.hpp:519-581, 641-692):
// score = dot(q, float(k8) * sk) * invSqrt, online softmax with exp2, out = sum p * float(v8) * sv.
//
// Why integer tensor cores in an HBM-bound kernel: at 5..8 q heads per kv head the dequantise +
// FMA work is beyond the CUDA cores at HBM speed, and the mma.sync form of this kernel
// (decode_i8.cu) is bound by the ~770 warp instructions it spends per 32 tokens on unpacking
// bytes into fp16 fragments.  Here the K and V tiles go from TMA straight into the tensor core:
//   * S^T[128 tokens x 32] = K[128 x 128 int8] . Qd^T, where Qd holds each q head as three
//     signed base-128 digit planes (q = 2^e * sum_i d_i 128^-i, 21 bits): the A operand is the K
//     tile exactly as TMA wrote it (K-major, 128-byte swizzle), int32 results in TMEM.
//   * a softmax thread owns one token: it reads its 24 integers (tcgen05.ld), rebuilds the 8
//     scores in f32, applies the row's K scale, exponentiates against a reference point that
//     all threads of the warpgroup share (moved only when a score runs ahead by 2^8), and
//     writes p * sv as a 32-bit fixed-point number per head -- whose four bytes ARE four
//     unsigned base-256 digit planes -- into the B operand tile in shared memory.
//   * O^T[128 dims x 32] = V^T[128 x 128 tokens] . Pd (A = the V tile as stored, MN-major;
//     B unsigned digits): int32 per tile in TMEM, folded into f32 registers (thread = dim)
//     with the tile's scale and reference point.  Integer accumulation never spans more than
//     one 128-token tile.
// Every product is exact; the only roundings are the 21-bit q digits, the 2^-24 fixed-point
// step of p * sv, and the f32 folds -- below the f32 arithmetic noise of the reference.
//
// CTA = one kv head x one token range (grid: chunks, kv heads, sequences), 17 warps:
// warps 0-3 / 4-7 two softmax warpgroups taking alternate tiles (scores -> probabilities only),
// warps 8-11 the fold warpgroup (thread = head dimension: every tile's integer P.V out of TMEM into
// one f32 accumulator per head, so a softmax warpgroup's next tile does not wait for the previous
// one's fold), warp 12 TMA producer (six-stage ring of K, V and their scales), warps 13-16 issue the
// MMAs (score / P.V products of even / odd tiles: a tcgen05.mma costs its issuing thread about a
// hundred cycles whatever its shape, threads of different warps issue concurrently).  Partials
// leave in the reference's layout for the merge kernel (merge.cu).
#include <cstdlib>

#include "tc_tcgen05.cuh"
#include "decode_shared.cuh"

namespace tc {

struct DecodeTcParams {
    const float *q;
    float *out;
    const float *ks, *vs;
    const float *appendK, *appendV;  // nullable: [batch][nKV][128] rows to quantise into row len - 1 first
    int8_t *k8w, *v8w;               // the pools, for that row
    const int8_t *nextK8, *nextV8;  // nullable: pools of the next call (L2 prefetch)
    float *pAcc, *pM, *pL;
    uint32_t *tickets;           // nullable: [batch][nKV] arrival counters of the in-kernel merge (zero between calls)
    const uint32_t *devLens;     // nullable
    const uint64_t *devRowBase;  // nullable
    uint64_t rowsPerSeq, totalRows;
    uint32_t lenHost, lenAdd;
    uint32_t nHeads, nKV, group, colBase;
    uint32_t chunkTokens, numChunks;
    uint32_t prefetchRows;
    float invSqrt;
    int directOut;
    int prefetchNext;
    uint32_t earlyStages;   // tiles the producer may request before the dependency wait
    int l2Hints;            // bit 0: own tiles evict_first, bit 1: next pools evict_last
    unsigned int *err;
#ifdef TC_TRACE
    unsigned long long *trace;  // [160 blocks][32 stamps]
#endif
};

#ifdef TC_TRACE
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TC_STAMP(slot) do { if (p.trace) p.trace[(blockIdx.x + gridDim.x * blockIdx.y) * 32 + (slot)] = gtime(); } while (0)
#else
#define TC_STAMP(slot) do { } while (0)
#endif

constexpr int kTcTile = 128;      // tokens per tile = MMA M of the score product
constexpr float kTcLazyLog2 = 8.0f;

// NWG softmax warpgroups take the tiles round-robin (tile j belongs to warpgroup j % NWG and uses its
// buffer (j / NWG) & 1); NS ring stages.  Warps: [0, 4 NWG) softmax, 4 NWG the TMA producer, then
// four MMA issuers.
template <int NWG, int NS>
struct DecodeTcSmem {
    static constexpr int kThreads = (4 * NWG + 4 + 5) * 32;   // softmax warpgroups, the fold warpgroup, producer, 4 MMA issuers
    static constexpr int kTileBytes = kTcTile * 128;              // K (or V) tile: 128 rows x 128 B
    static constexpr int kStageBytes = 2 * kTileBytes + 1024;     // + 128 K scales + 128 V scales
    static constexpr int kQd = NS * kStageBytes;                  // 32 rows x 128 B digit planes of q
    static constexpr int kP = kQd + 4096;                         // 2 NWG probability tiles of 128 x 32 B
    static constexpr int kRed = kP + 2 * NWG * 4096;              // [NWG warpgroups][4 warps][12] floats
    static constexpr int kHs = kRed + NWG * 4 * 12 * 4;           // head scales [8]
    static constexpr int kMeta = kHs + 64;                        // per (warpgroup, buffer): reference points [8], tile scale
    static constexpr int kBars = kMeta + 2 * NWG * 12 * 4;
    // full[NS], empty[NS], sFull[2 NWG], pFull[2 NWG], oFull[2 NWG], oFree[2 NWG], qFull
    static constexpr int kNumBars = 2 * NS + 8 * NWG + 1;
    static constexpr int kTmemCols = 128 * NWG;                   // S and O buffers of 32 columns each
    static constexpr int kTmemSlot = kBars + kNumBars * 8;
    static constexpr int kTotal = kTmemSlot + 16 + 1024;
    static_assert(kStageBytes % 1024 == 0, "stages keep the 1024-byte alignment of the 128-byte swizzle");
    static_assert(kTotal <= 227 * 1024, "shared memory of an SM");
};

// ---- helpers local to this kernel ---------------------------------------------------------
__device__ __forceinline__ uint64_t tcDesc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t swz) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(swz) << 61;  // 2 = 128-byte swizzle, 6 = 32-byte swizzle
    return d;
}
// kind::i8 instruction descriptor: int32 accumulator (c_format 2 at bit 4), a/b format at bits
// 7 / 10 (1 = signed, 0 = unsigned 8-bit), a/b major at bits 15 / 16 (1 = MN-major), N >> 3 at 17,
// M >> 4 at 24.
__host__ __device__ constexpr uint32_t tcIdescI8(uint32_t M, uint32_t N, uint32_t aMN, uint32_t bMN, uint32_t aSigned,
                                                 uint32_t bSigned) {
    return (2u << 4) | (aSigned << 7) | (bSigned << 10) | (aMN << 15) | (bMN << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
__device__ __forceinline__ void tcMmaI8If(uint32_t issue, uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "setp.ne.b32 q, %5, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
            "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(issue)
            : "memory");
}
__device__ __forceinline__ void tmemLd16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
}
__device__ __forceinline__ void tmemLd8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// all `threads` threads of named barrier `id` arrive; returns the OR of their predicates
__device__ __forceinline__ bool barOr(uint32_t id, uint32_t threads, bool pred) {
    uint32_t r;
    asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 q, %3, 0;\n\t"
            "bar.red.or.pred p, %1, %2, q;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(r)
            : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(pred))
            : "memory");
    return r != 0;
}
__device__ __forceinline__ float i2f(uint32_t x) { return __int2float_rn(static_cast<int>(x)); }

// The new token's K and V row of one kv head into the int8 pool, by one warp (the arithmetic of
// kvQuantKernel: amax / 127, IEEE divide, round-half-even; lane i owns dims 4 i .. 4 i + 3 of the 128).
// Blocks that share the kv head write the same bytes.  Both rows are loaded at once (they were pulled
// towards L2 when the block started); the block's own TMA load and scale copies read the row back, so
// the stores are ordered before the async proxy and nothing wider.  srcK / srcV: the rows' 32 float4;
// dst: row x nKV + kv head of the pool.
__device__ __forceinline__ void appendNewRow(const float4 *srcK, const float4 *srcV, uint32_t *k8w, uint32_t *v8w,
                                             float *ksw, float *vsw, uint64_t dst, uint32_t lane) {
    const float4 kx = __ldg(srcK + lane);
    const float4 vx = __ldg(srcV + lane);
    float mk = fmaxf(fmaxf(fabsf(kx.x), fabsf(kx.y)), fmaxf(fabsf(kx.z), fabsf(kx.w)));
    float mv = fmaxf(fmaxf(fabsf(vx.x), fabsf(vx.y)), fmaxf(fabsf(vx.z), fabsf(vx.w)));
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
    const float sk = mk > 0.0f ? __fdiv_rn(mk, 127.0f) : 1.0f;
    const float sv = mv > 0.0f ? __fdiv_rn(mv, 127.0f) : 1.0f;
    if (lane == 0) {
        ksw[dst] = sk;
        vsw[dst] = sv;
    }
    auto q8 = [](float x, float sc) -> uint32_t {
        int qv = __float2int_rn(__fdiv_rn(x, sc));
        qv = qv < -128 ? -128 : (qv > 127 ? 127 : qv);
        return static_cast<uint32_t>(qv) & 0xffu;
    };
    k8w[dst * 32u + lane] = q8(kx.x, sk) | (q8(kx.y, sk) << 8) | (q8(kx.z, sk) << 16) | (q8(kx.w, sk) << 24);
    v8w[dst * 32u + lane] = q8(vx.x, sv) | (q8(vx.y, sv) << 8) | (q8(vx.z, sv) << 16) | (q8(vx.w, sv) << 24);
    asm volatile("fence.proxy.async.global;" ::: "memory");
    __syncwarp();
}

// APPEND: the instantiation for calls that hand in the new token's rows.  It is a kernel of its own
// because the mere presence of that (cold) code -- inlined or called, inside or behind the producer's
// loop -- cost the 7B-shaped batch-1 step 0.5 us; calls without new rows run the other instantiation.
template <int NWG, int NS, bool APPEND, bool TICKETS>
__global__ void __launch_bounds__((4 * NWG + 9) * 32, 1)
decodeI8TcKernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmKn, const __grid_constant__ CUtensorMap tmVn,
                 const DecodeTcParams p) {
    using L = DecodeTcSmem<NWG, NS>;
    constexpr uint32_t kWG = NWG, kSoftThreads = 128u * NWG, kAllBar = NWG + 1u, kEndBar = NWG + 2u;
    constexpr uint32_t kFoldWarp0 = 4u * NWG, kProducerWarp = 4u * NWG + 4u, kMmaWarp0 = 4u * NWG + 5u;
    constexpr uint32_t kEndThreads = 32u * kProducerWarp;   // softmax + fold threads
    constexpr uint32_t T = kTcTile;
    const uint32_t chunk = blockIdx.x, kvHead = blockIdx.y, b = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kBars);
    uint64_t *fullBar = bars, *emptyBar = bars + NS, *sFull = bars + 2 * NS, *pFull = sFull + 2 * NWG,
             *oFull = pFull + 2 * NWG, *oFree = oFull + 2 * NWG, *qFull = oFree + 2 * NWG;
    uint32_t *tmemSlot = reinterpret_cast<uint32_t *>(smem + L::kTmemSlot);
    float *sHs = reinterpret_cast<float *>(smem + L::kHs);

    if (threadIdx.x == 0) {
        TC_STAMP(0);
        for (uint32_t s = 0; s < NS; ++s) {
            mbarInit(&fullBar[s], 1 + 32);
            mbarInit(&emptyBar[s], 1);
        }
        for (int i = 0; i < 2 * NWG; ++i) {
            mbarInit(&sFull[i], 1);
            mbarInit(&pFull[i], 128);
            mbarInit(&oFull[i], 1);
            mbarInit(&oFree[i], 128);
        }
        mbarInit(qFull, 256);
        fenceBarrierInit();
        tmaPrefetchDesc(&tmK);
        tmaPrefetchDesc(&tmV);
    }
    __syncthreads();
    gridDepLaunch();  // the dependent grid (the merge) may be scheduled as soon as room frees up

    // The length may live in device memory written by an earlier kernel; only a host-known
    // length lets the producer start before the dependency wait.
    uint32_t len = p.lenHost;
    const bool earlyOk = p.devLens == nullptr && p.devRowBase == nullptr && p.prefetchRows != 0;
    if (!earlyOk) {
        gridDepWait();
        if (p.devLens) len = p.devLens[b] + p.lenAdd;
    }
    const uint32_t t0 = chunk * p.chunkTokens;
    if (t0 >= len) return;  // inactive chunk (block-uniform): the merge derives the active count from len
    const uint32_t t1 = min(len, t0 + p.chunkTokens);
    const uint32_t nTiles = (t1 - t0 + T - 1) / T;
    const uint64_t rowBase = p.devRowBase ? p.devRowBase[b] : static_cast<uint64_t>(b) * p.rowsPerSeq;

    if (warp == 0) {
        tmemAlloc(tmemSlot, L::kTmemCols);
        tmemRelinquish();
        tcFenceBefore();
    }
    __syncthreads();
    tcFenceAfter();
    const uint32_t tmemBase = *reinterpret_cast<volatile uint32_t *>(tmemSlot);
    if (threadIdx.x == 0) TC_STAMP(1);
    // S of (warpgroup w, buffer bb) at columns 32 (2w + bb); O of the same pair 64 NWG columns further on

    if (warp == kProducerWarp) {
        // ------------------------------ TMA producer ------------------------------
        const uint64_t polFirst = l2PolicyEvictFirst(), polLast = l2PolicyEvictLast();
        auto prefetchNextPools = [&]() {
            // the same rows of the next call's pools into L2 (that call's TMA loads then hit L2)
            for (uint32_t it = 0; it < nTiles; ++it) {
                const int row = static_cast<int>(rowBase + t0 + it * T);
                if (p.l2Hints & 2) {
                    tmaPrefetchL2_3DHint(&tmKn, 0, kvHead, row, polLast);
                    tmaPrefetchL2_3DHint(&tmVn, 0, kvHead, row, polLast);
                } else {
                    tmaPrefetchL2_3D(&tmKn, 0, kvHead, row);
                    tmaPrefetchL2_3D(&tmVn, 0, kvHead, row);
                }
            }
        };
        if (APPEND && p.appendK != nullptr && t1 == len && lane < 8u) {
            // the rows this block will append, towards L2 (their final contents arrive there too)
            const char *src = reinterpret_cast<const char *>((lane < 4u ? p.appendK : p.appendV) +
                                                             (static_cast<size_t>(b) * p.nKV + kvHead) * 128u) + (lane & 3u) * 128u;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
        }
        bool waited = !earlyOk;
        auto requestTile = [&](uint32_t it) -> bool {
            const uint32_t s = it % NS;
            if (it >= NS && !mbarWaitClock(&emptyBar[s], ((it / NS) - 1u) & 1u, p.err, kDevErrEmptyWait)) return false;
            const uint32_t tok = t0 + it * T;
            if (!waited && (tok + T > p.prefetchRows || it >= p.earlyStages)) {
                // rows the kernel in front may still be writing, or further ahead of the dependency
                // than the caller allows
                gridDepWait();
                waited = true;
            }
            uint8_t *st = smem + s * L::kStageBytes;
            const uint64_t row = rowBase + tok;
            if (lane == 0) {
                mbarExpectTx(&fullBar[s], 2 * L::kTileBytes);
                if (p.l2Hints & 1) {
                    tmaLoad3DHint(st, &tmK, &fullBar[s], 0, kvHead, static_cast<int>(row), polFirst);
                    tmaLoad3DHint(st + L::kTileBytes, &tmV, &fullBar[s], 0, kvHead, static_cast<int>(row), polFirst);
                } else {
                    tmaLoad3D(st, &tmK, &fullBar[s], 0, kvHead, static_cast<int>(row));
                    tmaLoad3D(st + L::kTileBytes, &tmV, &fullBar[s], 0, kvHead, static_cast<int>(row));
                }
            }
            float *sK = reinterpret_cast<float *>(st + 2 * L::kTileBytes);
            float *sV = sK + T;
#pragma unroll
            for (uint32_t idx = lane; idx < T; idx += 32) {
                uint64_t r = row + idx;
                r = r < p.totalRows ? r : p.totalRows - 1;
                cpAsync4(&sK[idx], p.ks + r * p.nKV + kvHead);
                cpAsync4(&sV[idx], p.vs + r * p.nKV + kvHead);
            }
            cpAsyncMbarArriveNoinc(&fullBar[s]);
            if (lane == 0) { if (it == 0) TC_STAMP(13); TC_STAMP(14); }
            return true;
        };
        // The tile that holds the row of a token being appended (the last tile of the sequence's last
        // chunk) is requested apart from the loop: the row goes into the pool first, once the kernels
        // ahead have completed.
        const bool appendHere = APPEND && p.appendK != nullptr && t1 == len;
        const uint32_t nLoop = appendHere ? nTiles - 1u : nTiles;
        bool okP = true;
        for (uint32_t it = 0; okP && it < nLoop; ++it) okP = requestTile(it);
        if (appendHere && okP) {
            if (!waited) {
                gridDepWait();
                waited = true;
            }
            const size_t srcRow = (static_cast<size_t>(b) * p.nKV + kvHead) * 32u;
            const uint64_t dst = (rowBase + len - 1u) * p.nKV + kvHead;
            // a length read from device memory is checked where it is known: outside the pool the
            // store is skipped and the error word says so
            if (rowBase + len - 1u >= p.totalRows) {
                if (lane == 0) atomicOr(p.err, kDevErrRowBound);
            } else {
                appendNewRow(reinterpret_cast<const float4 *>(p.appendK) + srcRow,
                             reinterpret_cast<const float4 *>(p.appendV) + srcRow, reinterpret_cast<uint32_t *>(p.k8w),
                             reinterpret_cast<uint32_t *>(p.v8w), const_cast<float *>(p.ks), const_cast<float *>(p.vs), dst,
                             lane);
            }
            requestTile(nTiles - 1u);
        }
        // all tiles of this block are requested: the next call's rows follow them into L2 (requested
        // earlier they sit in front of this block's own tiles in the queue: 10.2 against 9.1 us)
        if (p.prefetchNext && lane == 0) prefetchNextPools();
    } else if (warp > kProducerWarp) {
        // -------------------------------- MMA issuers --------------------------------
        // One tcgen05.mma costs its issuing thread about a hundred cycles whatever its shape, and
        // threads of different warps issue concurrently: four issuing warps -- score products and
        // P.V products of the even (warpgroup 0) and of the odd (warpgroup 1) tiles.  Warp-uniform
        // control flow; lane 0 executes the tcgen05 instructions.
        const uint32_t issue = lane == 0 ? 1u : 0u;
        const uint32_t par = (warp - kMmaWarp0) & 1u;       // which tiles: j = par, par + 2, ...
        const bool pvRole = warp >= kMmaWarp0 + 2u;
        if (!pvRole) {
            constexpr uint32_t idQK = tcIdescI8(128, 32, 0, 0, 1, 1);   // K-major A (K tile), K-major B (q digits)
            const uint64_t dQd = tcDesc(smemAddr(smem + L::kQd), 16, 1024, 2);
            bool ok = mbarWaitClock(qFull, 0, p.err, kDevErrFullWait);
            if (lane == 0 && par == 0) TC_STAMP(15);
            for (uint32_t j = par; ok && j < nTiles; j += 2u) {
                const uint32_t s = j % NS, w = j % kWG, bb = (j / kWG) & 1u;
                // the S buffer's previous contents (tile j - 2 NWG) have been read once that tile's P is out
                if (j >= 2u * kWG)
                    ok = mbarWaitClock(&pFull[2u * w + bb], ((j - 2u * kWG) / (2u * kWG)) & 1u, p.err, kDevErrMmaWait);
                ok = ok && mbarWaitClock(&fullBar[s], (j / NS) & 1u, p.err, kDevErrFullWait);
                if (lane == 0 && j < 8u) TC_STAMP(20 + j);
                if (!ok) break;
                tcFenceAfter();
                const uint64_t dK = tcDesc(smemAddr(smem + s * L::kStageBytes), 16, 1024, 2);
                const uint32_t tS = tmemBase + 32u * (2u * w + bb);
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k)  // 32 dims per instruction = 32 bytes inside the swizzle span
                    tcMmaI8If(issue, tS, dK + ((k * 32u) >> 4), dQd + ((k * 32u) >> 4), idQK, k > 0 ? 1u : 0u);
                umaCommitIf(issue, &sFull[2u * w + bb]);
            }
        } else {
            constexpr uint32_t idPV = tcIdescI8(128, 32, 1, 1, 1, 0);   // MN-major A (V tile), MN-major unsigned B (p digits)
            bool ok = true;
            for (uint32_t j = par; ok && j < nTiles; j += 2u) {
                const uint32_t s = j % NS, w = j % kWG, bb = (j / kWG) & 1u;
                // P of tile j published
                ok = mbarWaitClock(&pFull[2u * w + bb], (j / (2u * kWG)) & 1u, p.err, kDevErrMmaWait);
                // and the fold warpgroup has read the O buffer's previous contents (tile j - 2 NWG)
                if (ok && j >= 2u * kWG)
                    ok = mbarWaitClock(&oFree[2u * w + bb], ((j - 2u * kWG) / (2u * kWG)) & 1u, p.err, kDevErrMmaWait);
                if (!ok) break;
                tcFenceAfter();
                const uint64_t dV = tcDesc(smemAddr(smem + s * L::kStageBytes + L::kTileBytes), 16, 1024, 2);
                const uint64_t dP = tcDesc(smemAddr(smem + L::kP + (2u * w + bb) * 4096u), 16, 256, 6);
                const uint32_t tO = tmemBase + 64u * kWG + 32u * (2u * w + bb);
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k)  // 32 tokens per instruction: 4096 B of V, 1024 B of P
                    tcMmaI8If(issue, tO, dV + ((k * 4096u) >> 4), dP + ((k * 1024u) >> 4), idPV, k > 0 ? 1u : 0u);
                umaCommitIf(issue, &oFull[2u * w + bb]);
                // K and V of the stage are consumed once these products are done (the score product
                // of the tile completed before its P could be written)
                umaCommitIf(issue, &emptyBar[s]);
                if (lane == 0) TC_STAMP(16);
            }
        }
    } else if (warp >= kFoldWarp0) {
        // ------------------------------ fold warpgroup ------------------------------
        // thread = one head dimension: takes every tile's integer P.V out of TMEM in tile order and
        // folds it into ONE f32 accumulator per head, against a running reference point of its own
        // (the two softmax warpgroups keep separate ones; a tile arrives with the reference it was
        // exponentiated against and with its fixed-point scale)
        const uint32_t wq = warp & 3u;
        const uint32_t row = wq * 32u + lane;
        const uint32_t laneBase = (wq * 32u) << 16;
        const float *meta = reinterpret_cast<const float *>(smem + L::kMeta);
        float o[8], M[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) o[h] = 0.0f, M[h] = kNegBig;
        bool ok = true;
        for (uint32_t j = 0; ok && j < nTiles; ++j) {
            const uint32_t w = j % kWG, bb = (j / kWG) & 1u, par = (j / (2u * kWG)) & 1u;
            ok = mbarWaitClock(&oFull[2u * w + bb], par, p.err, kDevErrMmaWait);
            if (!ok) break;
            tcFenceAfter();
            uint32_t r[32];
            tmemLd32(tmemBase + 64u * kWG + 32u * (2u * w + bb) + laneBase, r);
            const float *mt = meta + (2u * w + bb) * 12u;
            float tmr[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) tmr[h] = mt[h];
            const float esc = mt[8];
            tmemLdWait();
            tcFenceBefore();
            mbarArrive(&oFree[2u * w + bb]);   // the buffer and its meta slot may be reused
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                // column 4h + i carries byte i of the fixed-point probability: weight 256^i
                const float c = fmaf(fmaf(fmaf(i2f(r[4 * h + 3]), 256.0f, i2f(r[4 * h + 2])), 256.0f, i2f(r[4 * h + 1])),
                                     256.0f, i2f(r[4 * h]));
                const float mn = fmaxf(M[h], tmr[h]);
                o[h] = fmaf(c, esc * fastExp2(tmr[h] - mn), o[h] * fastExp2(M[h] - mn));
                M[h] = mn;
            }
            if (threadIdx.x == kFoldWarp0 * 32u && j + 1u == nTiles) TC_STAMP(10);
        }
        // every P tile has been consumed (its O was waited for above): their space is the scratch
        float *scr = reinterpret_cast<float *>(smem + L::kP);
        namedBarSync(kEndBar, kEndThreads);
#pragma unroll
        for (int h = 0; h < 8; ++h) scr[h * 128u + row] = o[h];
        if (threadIdx.x == kFoldWarp0 * 32u) {
#pragma unroll
            for (int h = 0; h < 8; ++h) scr[8 * 128 + h] = M[h];
        }
        namedBarSync(kEndBar, kEndThreads);
    } else {
        // ---------------------------- softmax warpgroups ----------------------------
        const uint32_t w = warp >> 2;                       // warpgroup: tiles j = w, w + NWG, ...
        const uint32_t wq = warp & 3u;                      // TMEM lane quarter of this warp
        const uint32_t row = wq * 32u + lane;               // token of the tile
        const uint32_t laneBase = (wq * 32u) << 16;
        const uint32_t wgBar = 1u + w;                      // named barrier of the warpgroup
        float *red = reinterpret_cast<float *>(smem + L::kRed) + w * 48u;
        float *meta = reinterpret_cast<float *>(smem + L::kMeta);

        // pull q towards L2 while waiting (harmless if the kernel in front is still writing it)
        if (lane == 0 && warp < 8u && p.colBase + warp < p.group)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q + (static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + warp) * 128u));
        gridDepWait();  // q comes from a kernel that may still be running
        if (threadIdx.x == 0) TC_STAMP(2);
        // ---- q of head `warp` of this kv head -> three signed base-128 digit planes ----
        if (warp < 8u) {
            const uint32_t h = warp;  // 8 softmax warps = the 8 MMA columns
            const bool valid = p.colBase + h < p.group;
            const float4 qv = valid ? __ldg(reinterpret_cast<const float4 *>(
                                              p.q + (static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + h) * 128u) + lane)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
            float amax = fmaxf(fmaxf(fabsf(qv.x), fabsf(qv.y)), fmaxf(fabsf(qv.z), fabsf(qv.w)));
#pragma unroll
            for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            // |q| * 2^-e < 1 with e = floor(log2 amax) + 1; digits of X = rint(q * 2^(20 - e)), |X| <= 2^20
            int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 126;
            e = amax > 0.0f ? max(-100, min(100, e)) : 0;
            const float toFix = __uint_as_float(static_cast<uint32_t>(127 + 20 - e) << 23);
            auto digits = [&](float x, int &d0, int &d1, int &d2) {
                const int X = __float2int_rn(x * toFix);
                d2 = ((X + 64) & 127) - 64;
                const int X1 = (X - d2) >> 7;
                d1 = ((X1 + 64) & 127) - 64;
                d0 = (X1 - d1) >> 7;
            };
            int d0[4], d1[4], d2[4];
            digits(qv.x, d0[0], d1[0], d2[0]);
            digits(qv.y, d0[1], d1[1], d2[1]);
            digits(qv.z, d0[2], d1[2], d2[2]);
            digits(qv.w, d0[3], d1[3], d2[3]);
            auto pack = [](const int (&d)[4]) {
                return (static_cast<uint32_t>(d[0]) & 0xffu) | ((static_cast<uint32_t>(d[1]) & 0xffu) << 8) |
                       ((static_cast<uint32_t>(d[2]) & 0xffu) << 16) | ((static_cast<uint32_t>(d[3]) & 0xffu) << 24);
            };
            // row n = plane * 8 + head, 128 bytes of dims, 16-byte units xor-swizzled by the row (128-byte swizzle)
            uint8_t *qd = smem + L::kQd;
            const uint32_t unit = lane >> 2, inUnit = (lane & 3u) * 4u;
            auto put = [&](uint32_t n, uint32_t word) {
                *reinterpret_cast<uint32_t *>(qd + n * 128u + ((unit ^ (n & 7u)) << 4) + inUnit) = word;
            };
            put(h, pack(d0));
            put(8u + h, pack(d1));
            put(16u + h, pack(d2));
            put(24u + h, 0u);
            // log2-domain scale of this head's integer scores: invSqrt * log2(e) * 2^(e - 20)
            if (lane == 0)
                sHs[h] = valid ? p.invSqrt * kLog2e * __uint_as_float(static_cast<uint32_t>(127 + e - 20) << 23) : 0.0f;
            fenceProxyAsync();
            mbarArrive(qFull);
        }
        if (threadIdx.x == 0) TC_STAMP(3);
        namedBarSync(kAllBar, kSoftThreads);  // head scales visible to every warpgroup
        float hs[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) hs[h] = sHs[h];

        float mref[8], l[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) mref[h] = kNegBig, l[h] = 0.0f;
        float Eref = 0.0f, invW = 0.0f;  // power of two above every V scale seen; 2^24 / Eref
        bool ok = true;

        for (uint32_t j = w; j < nTiles; j += kWG) {
            const uint32_t s = j % NS, bb = (j / kWG) & 1u;
            // ---- this thread's token against the 8 heads ----
            if (!mbarWaitClock(&sFull[2u * w + bb], (j / (2u * kWG)) & 1u, p.err, kDevErrMmaWait)) {
                ok = false;
                break;
            }
            tcFenceAfter();
            if (threadIdx.x == 0 && j == 0) TC_STAMP(4);
            uint32_t ra[16], rb[8];
            const uint32_t tS = tmemBase + 32u * (2u * w + bb) + laneBase;
            tmemLd16(tS, ra);
            tmemLd8(tS + 16u, rb);
            const float *sK = reinterpret_cast<const float *>(smem + s * L::kStageBytes + 2 * L::kTileBytes);
            const bool valid = t0 + j * T + row < t1;
            const float skr = sK[row];
            const float svr = valid ? sK[T + row] : 0.0f;
            tmemLdWait();
            float sc[8];
            bool need = svr >= Eref;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                const float f = fmaf(fmaf(i2f(ra[h]), 128.0f, i2f(ra[8 + h])), 128.0f, i2f(rb[h]));
                sc[h] = valid ? f * (skr * hs[h]) : -INFINITY;
                need = need || sc[h] > mref[h] + kTcLazyLog2;
            }
            if (barOr(wgBar, 128, need)) {
                // rare: the reference point of a head (or the bound of the V scales) has to move --
                // tile maxima over the warpgroup, then every thread applies the same update
                float tm[9];
#pragma unroll
                for (int h = 0; h < 8; ++h) tm[h] = sc[h];
                tm[8] = svr;
#pragma unroll
                for (int i = 0; i < 9; ++i)
#pragma unroll
                    for (int off = 16; off; off >>= 1) tm[i] = fmaxf(tm[i], __shfl_xor_sync(0xffffffffu, tm[i], off));
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < 9; ++i) red[wq * 12u + i] = tm[i];
                }
                namedBarSync(wgBar, 128);
#pragma unroll
                for (int i = 0; i < 9; ++i) tm[i] = fmaxf(fmaxf(red[i], red[12 + i]), fmaxf(red[24 + i], red[36 + i]));
                namedBarSync(wgBar, 128);  // red may be rewritten by the next rare pass
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float mn = fmaxf(mref[h], tm[h]);
                    l[h] *= fastExp2(mref[h] - mn);
                    mref[h] = mn;
                }
                if (tm[8] >= Eref) {
                    uint32_t eb = (__float_as_uint(tm[8]) & 0x7f800000u) + 0x00800000u;  // 2^(floor(log2) + 1)
                    eb = min(max(eb, 24u << 23), 253u << 23);
                    Eref = __uint_as_float(eb);
                    invW = __uint_as_float((127u + 24u + 127u) * (1u << 23) - eb);  // 2^24 / Eref
                }
            }
            // p, l, and p * sv as 32-bit fixed point (8.24 against Eref): its bytes are the digit planes
            const float wv = svr * invW;
            uint32_t X[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                const float pr = fastExp2(sc[h] - mref[h]);
                l[h] += pr;
                X[h] = __float2uint_rn(pr * wv);
            }
            // The P tile and the meta slot of this buffer were last used by tile j - 2 NWG: that tile's
            // P.V product is complete and folded once the fold warpgroup has said so on oFree (long
            // ago, as a rule: two tiles of this warpgroup lie in between).
            if (j >= 2u * kWG &&
                !mbarWaitClock(&oFree[2u * w + bb], ((j - 2u * kWG) / (2u * kWG)) & 1u, p.err, kDevErrMmaWait)) {
                ok = false;
                break;
            }
            uint8_t *pt = smem + L::kP + (2u * w + bb) * 4096u + row * 32u;
            const uint32_t sw = (row >> 2) & 1u;  // 32-byte swizzle: 16-byte halves swap on rows 4..7 of every 8
            *reinterpret_cast<uint4 *>(pt + ((0u ^ sw) << 4)) = make_uint4(X[0], X[1], X[2], X[3]);
            *reinterpret_cast<uint4 *>(pt + ((1u ^ sw) << 4)) = make_uint4(X[4], X[5], X[6], X[7]);
            if (row == 0) {
                // what the fold warpgroup needs with this tile: the reference points its probabilities
                // were taken against and the scale of their fixed-point form
                float *mt = meta + (2u * w + bb) * 12u;
#pragma unroll
                for (int h = 0; h < 8; ++h) mt[h] = mref[h];
                mt[8] = Eref * 5.9604644775390625e-8f;  // Eref * 2^-24
            }
            fenceProxyAsync();
            tcFenceBefore();
            mbarArrive(&pFull[2u * w + bb]);
            if (threadIdx.x == 0 && j / kWG < 4u) TC_STAMP(5 + j / kWG);
        }

        // ---- row sums of this warpgroup, then the end of the block ----
#pragma unroll
        for (int h = 0; h < 8; ++h)
#pragma unroll
            for (int off = 16; off; off >>= 1) l[h] += __shfl_xor_sync(0xffffffffu, l[h], off);
        float *scr = reinterpret_cast<float *>(smem + L::kP);
        float *oS = scr;                          // [8][128] from the fold warpgroup, then its reference points [8]
        float *mF = scr + 8 * 128;
        float *mS = mF + 8;                       // [NWG][8]
        float *lS = mS + NWG * 8;                 // [4 NWG warps][8]
        namedBarSync(kEndBar, kEndThreads);       // the fold warpgroup is through: every P tile has been consumed
        if (lane == 0) {
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                lS[warp * 8u + h] = l[h];
                if (wq == 0) mS[w * 8u + h] = mref[h];
            }
        }
        namedBarSync(kEndBar, kEndThreads);
        if (threadIdx.x == 0) TC_STAMP(11);
        if (warp < 8u) {
            const uint32_t tid = threadIdx.x;  // 0..255: head tid / 32, dims 4 (tid % 32) ..
            const uint32_t h = tid >> 5, d4 = tid & 31u;
            if (p.colBase + h < p.group) {
                // the accumulator is relative to the fold warpgroup's reference point, which is the
                // largest of the warpgroups' (a reference only ever grows)
                const float M = mF[h];
                const float4 acc = *reinterpret_cast<const float4 *>(oS + h * 128u + 4u * d4);
                float lsum = 0.0f;
#pragma unroll
                for (int g = 0; g < NWG; ++g) {
                    const float a = fastExp2(mS[g * 8 + h] - M);   // a warpgroup without tiles: exp2(-1e30) = 0
                    const float lg = (lS[(4 * g) * 8 + h] + lS[(4 * g + 1) * 8 + h]) +
                                     (lS[(4 * g + 2) * 8 + h] + lS[(4 * g + 3) * 8 + h]);
                    lsum = fmaf(a, lg, lsum);
                }
                const size_t oidx = static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + h;
                if (p.directOut) {
                    const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
                    *reinterpret_cast<float4 *>(p.out + oidx * 128u + 4u * d4) =
                            make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
                } else {
                    const size_t pidx = oidx * p.numChunks + chunk;
                    *reinterpret_cast<float4 *>(p.pAcc + pidx * 128u + 4u * d4) = acc;
                    if (d4 == 0) {
                        // natural-log units: the merge contract is w = exp2((m - M) * log2e)
                        p.pM[pidx] = M > -1e29f ? M * 0.6931471805599453f : kNegBig;
                        p.pL[pidx] = lsum;
                    }
                }
            }
        }
        if (TICKETS && !p.directOut && p.tickets != nullptr) {
            // ---- merge inside the kernel: the block that arrives last at its (sequence, kv head)
            // counter folds all chunk partials of the kv head's q heads.  Nobody waits: every block
            // publishes its partial, takes a ticket and leaves unless the ticket is the last one.
            uint32_t *sTicket = reinterpret_cast<uint32_t *>(lS + 4 * NWG * 8);
            __threadfence();  // this thread's partial stores are visible device-wide before the ticket
            namedBarSync(kAllBar, kSoftThreads);
            uint32_t *ctr = p.tickets + static_cast<size_t>(b) * p.nKV + kvHead;
            if (threadIdx.x == 0) *sTicket = atomicAdd(ctr, 1u);
            namedBarSync(kAllBar, kSoftThreads);
            const uint32_t nActive = min((len + p.chunkTokens - 1u) / p.chunkTokens, gridDim.x);
            if (*sTicket == nActive - 1u) {
                __threadfence();
                if (threadIdx.x == 0) *ctr = 0u;  // ready for the next call on this stream
                const uint32_t h = warp;          // one warp per q head, lane = four dims
                if (warp < 8u && p.colBase + h < p.group) {
                    const size_t oidx = static_cast<size_t>(b) * p.nHeads + kvHead * p.group + p.colBase + h;
                    const float *gm = p.pM + oidx * p.numChunks, *gl = p.pL + oidx * p.numChunks;
                    const float *ga = p.pAcc + oidx * p.numChunks * 128u + 4u * lane;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    float M = kNegBig, Lsum = 0.0f;
                    // chunk partials in groups of 32: lane c holds (m, l) of chunk c0 + c
                    for (uint32_t c0 = 0; c0 < nActive; c0 += 32u) {
                        const uint32_t c = c0 + lane;
                        const float lc = c < nActive ? __ldcg(gl + c) : 0.0f;
                        const float mc = (c < nActive && lc > 0.0f) ? __ldcg(gm + c) : kNegBig;
                        float gmx = mc;
#pragma unroll
                        for (int off = 16; off; off >>= 1) gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, off));
                        const float Mn = fmaxf(M, gmx);
                        const float sOld = fastExp2((M - Mn) * kLog2e);
                        acc.x *= sOld, acc.y *= sOld, acc.z *= sOld, acc.w *= sOld;
                        Lsum *= sOld;
                        M = Mn;
                        const float wc = lc > 0.0f ? fastExp2((mc - M) * kLog2e) : 0.0f;
                        float wl = wc * lc;
#pragma unroll
                        for (int off = 16; off; off >>= 1) wl += __shfl_xor_sync(0xffffffffu, wl, off);
                        Lsum += wl;
                        const uint32_t n = min(32u, nActive - c0);
#pragma unroll 8
                        for (uint32_t i = 0; i < n; ++i) {
                            const float wi = __shfl_sync(0xffffffffu, wc, i);
                            const float4 a = __ldcg(reinterpret_cast<const float4 *>(ga + static_cast<size_t>(c0 + i) * 128u));
                            acc.x = fmaf(wi, a.x, acc.x);
                            acc.y = fmaf(wi, a.y, acc.y);
                            acc.z = fmaf(wi, a.z, acc.z);
                            acc.w = fmaf(wi, a.w, acc.w);
                        }
                    }
                    const float inv = Lsum > 0.0f ? 1.0f / Lsum : 0.0f;
                    *reinterpret_cast<float4 *>(p.out + oidx * 128u + 4u * lane) =
                            make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
                }
            }
        }
    }
    if (threadIdx.x == 0) TC_STAMP(12);
    tcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        tcFenceAfter();
        tmemDealloc(tmemBase, L::kTmemCols);
    }
}

// Host side: arguments were validated by the caller (decodeI8Common in decode_i8.cu).
int decodeI8Tc(const tc_decode_i8_batch *d, uint32_t lenHost, uint32_t lenAdd, cudaStream_t st) {
    const uint32_t hd = 128;
    const uint32_t group = d->nHeads / d->nKV;
    const DecodePlan pl = planDecode(d->batch, d->nKV, d->maxLen, d->numChunks, kTcTile, d->lens == nullptr, 1u);
    const bool pdl = (d->flags & TC_DECODE_PDL) != 0;
    const bool direct = pl.chunksPerSeq == 1 && !d->partialsOnly;
    if (!direct) TC_REQUIRE(d->pAcc && d->pM && d->pL, TC_EWORKSPACE, "decode_i8: partial buffers are required");
    if (d->chunksUsed) *d->chunksUsed = pl.chunksPerSeq;
    TC_REQUIRE(d->nKV <= 65535, TC_EUNSUPPORTED, "decode_i8: %u kv heads", d->nKV);

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
    key.box[0] = 128;
    key.box[1] = 1;
    key.box[2] = kTcTile;
    CUtensorMap tmK, tmV;
    key.base = d->k8;
    int rc = getTensorMap(key, &tmK);
    if (rc != TC_OK) return rc;
    key.base = d->v8;
    rc = getTensorMap(key, &tmV);
    if (rc != TC_OK) return rc;
    CUtensorMap tmKn = tmK, tmVn = tmV;
    // the next call's pools, pulled into L2 behind this call's rows -- only when a call's rows fit
    // there next to the rows still in flight (a larger prefetch is evicted before it is used)
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

    DecodeTcParams prm;
    prm.q = d->q;
    prm.out = d->out;
    prm.ks = d->ks;
    prm.vs = d->vs;
    prm.nextK8 = d->nextK8;
    prm.nextV8 = d->nextV8;
    prm.appendK = d->appendK;
    prm.appendV = d->appendV;
    prm.k8w = const_cast<int8_t *>(d->k8);
    prm.v8w = const_cast<int8_t *>(d->v8);
    prm.pAcc = d->pAcc;
    prm.pM = d->pM;
    prm.pL = d->pL;
    // the in-kernel merge serves one launch per call (q-head groups of at most 8) and needs the output
    const bool fused = d->mergeTickets != nullptr && !direct && !d->partialsOnly && group <= 8;
    prm.tickets = fused ? d->mergeTickets : nullptr;
    prm.devLens = d->lens;
    prm.devRowBase = d->rowBase;
    prm.rowsPerSeq = d->rowsPerSeq;
    prm.totalRows = d->totalRows;
    prm.lenHost = lenHost;
    prm.lenAdd = lenAdd;
    prm.nHeads = d->nHeads;
    prm.nKV = d->nKV;
    prm.group = group;
    prm.colBase = 0;
    prm.chunkTokens = pl.chunkTokens;
    prm.numChunks = d->numChunks;
    prm.prefetchRows = pdl ? d->prefetchRows : 0;
    prm.invSqrt = d->invSqrt;
    prm.directOut = direct ? 1 : 0;
    prm.prefetchNext = prefetchNext ? 1 : 0;
    // Under programmatic dependent launch the producer requests a whole ring of old rows while the
    // kernels ahead drain (7B shape, 32768 rows, batch 1: 12.4 us per layer against 13.5 with one
    // stage).  The block's own tiles are read once (evict-first); the next call's rows pulled in
    // behind them are kept (evict-last) -- with plain policies the hint gained nothing.
    prm.earlyStages = 6;
    prm.l2Hints = 3;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "decode_i8: no device error word");
#ifdef TC_TRACE
    {
        extern unsigned long long *g_tcTrace;
        static unsigned callNo = 0;
        prm.trace = g_tcTrace ? g_tcTrace + static_cast<size_t>((callNo++) & 3u) * 160 * 32 : nullptr;
    }
#endif

    // (Four softmax warpgroups with a five-stage ring were measured and dropped: 11.5 against 8.3 us
    // per layer for the split launch alone at 32768 rows, 53.9 against 47.0 us at batch 8.)
    using Smem = DecodeTcSmem<2, 6>;
    // (the in-kernel merge is an instantiation of its own for the same reason as the append)
    auto kern = d->appendK != nullptr ? (fused ? decodeI8TcKernel<2, 6, true, true> : decodeI8TcKernel<2, 6, true, false>)
                                      : (fused ? decodeI8TcKernel<2, 6, false, true> : decodeI8TcKernel<2, 6, false, false>);
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(decodeI8TcKernel<2, 6, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Smem::kTotal));
        TC_CUDA_OK(cudaFuncSetAttribute(decodeI8TcKernel<2, 6, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Smem::kTotal));
        TC_CUDA_OK(cudaFuncSetAttribute(decodeI8TcKernel<2, 6, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Smem::kTotal));
        TC_CUDA_OK(cudaFuncSetAttribute(decodeI8TcKernel<2, 6, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Smem::kTotal));
        attrDone[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.chunksPerSeq, d->nKV, d->batch);
    cfg.blockDim = dim3(Smem::kThreads);
    cfg.dynamicSmemBytes = Smem::kTotal;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    // a launch serves 8 q heads per kv head (the MMA columns); wider groups take one launch per
    // block of 8 and stream the rows again
    for (uint32_t cb = 0; cb < group; cb += 8) {
        prm.colBase = cb;
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmK, tmV, tmKn, tmVn, prm));
    }
    if (direct || d->partialsOnly || fused) return TC_OK;
    return launchMerge(d->pAcc, d->pM, d->pL, d->out, d->batch, d->nHeads, d->numChunks, pl.chunksPerSeq, hd, d->lens,
                       lenAdd, pl.chunkTokens, nullptr, pdl, st);
}

#ifdef TC_TRACE
unsigned long long *g_tcTrace = nullptr;
#endif

}  // namespace tc

#ifdef TC_TRACE
extern "C" void tc_debug_trace(unsigned long long *buf) { tc::g_tcTrace = buf; }
#endif
