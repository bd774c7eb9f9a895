// prefill_f16.cu -- causal prefill attention on tcgen05 tensor cores (fp16 operands,
// f32 accumulation in TMEM).
//
// What it replaces: the reference's materialised dense prefill -- kF32ToF16 twins of
// q and of the stored K/V rows, one cuBLAS GEMM per q head for QK^T (f32 scores of
// seqLen^2 per head), kAttnSoftmaxCausal, one cuBLAS GEMM per q head for PV
// (src/cpp/core/cuda/forward/GPUComputeForward.cu:3937-4026;
// include/gpu/GpuAttentionKernels.hpp:323-353).  Same arithmetic contract: fp16
// products, f32 accumulation, f32 softmax with exp2 and the scale applied to the
// scores, probabilities rounded to fp16 -- but flash-style, so the score matrix
// never exists and the sequence length is not capped at 512.
//
// One persistent block per SM walks work items: a q head x 256 query rows = two 128-row query
// tiles A and B (one tile per item for short calls and at head_dim 256), KV tiles of 64 tokens (32
// at head_dim 256).  The first item of a block is its index, the following ones come from a
// counter, heavy (late) query blocks first; the mbarriers are initialised once, every ring index
// counts on from item to item, so the next item's loads and first score products run under the
// current item's epilogue.  Warp roles:
//   warps 0-3 / 4-7  softmax of tile A / B: thread r owns query row r, reads its scores of a KV
//              tile from TMEM (tcgen05.ld), keeps (m, l), writes the fp16 probabilities over the
//              first columns of the same S buffer (tcgen05.st) as the A operand of the PV product,
//              rescales O in TMEM only when the row maximum ran ahead by 2^8 (lazy rescale);
//              packed f32x2 arithmetic; normalises and stores the output rows (32-byte stores);
//   warp 8     TMA producer and scheduler: the query tiles and K_0, K_1 per item, then a four-stage
//              ring whose stage j holds what step j of the MMA warps consumes, K_{j+2} and V_j
//              (cp.async.bulk.tensor, 128-byte swizzle = the canonical UMMA shared-memory layout,
//              so no register pass touches the operands); draws the next item late in the current;
//   warps 9, 10  issue the score products of tile A / B: S_X(t) = Q_X K^T (M128 N64 K16 per
//              instruction), tcgen05.commit onto the softmax warps' barrier;
//   warps 11, 12  issue the P.V products of tile A / B: O_X += P_X(t) V (A from TMEM, B = V
//              MN-major from shared memory).  Issuing an instruction costs its thread about a
//              hundred cycles and threads of different warps issue concurrently, hence four warps.
// S is DOUBLE-BUFFERED per query tile: S_X(t+2) goes into the buffer P_X(t) leaves once its P.V
// product is complete, so S_X(t+1) is there when the softmax of tile t finishes.  TMEM (512
// columns): O_A, O_B (128 each, f32; one O of 256 at head_dim 256), S_{A,0}, S_{A,1}, S_{B,0},
// S_{B,1} (64 each).  Causality: a query tile only visits KV tiles up to its diagonal, the last
// two or three are masked element-wise; the query rows may sit behind an existing cache.
// In front of the kernel one launch makes the fp16 twins of q, K and V (from the f32 store, or
// from the int8 store's bytes and scales; an fp16 store is read in place) and, on request, the int8
// pool rows of the call's new positions; the attention kernel is its programmatic dependent.
// Every wait is bounded; a wait that runs out records an error bit, every other wait of the launch
// then gives up at once, the block frees its TMEM and returns.
#include <algorithm>

#include "tc_tcgen05.cuh"

namespace tc {

constexpr int kPfBM = 128;    // query rows per tile (two tiles per CTA)
constexpr int kPfStages = 4;  // K and V ring depth
constexpr float kPfLazyLog2 = 8.0f;

// Where the int8 mirror of the call's new K/V rows goes (the reference keeps such a pool beside its
// f32 store and rebuilds it before the first decode step, GPUComputeMoE.cu:3049-3063): rows
// [cachePos, cachePos + seqLen) of the cache become pool rows dstRow ..; null k8 = no mirror.
struct PrefillMirror {
    int8_t *k8, *v8;   // [rows][nKV][hd]
    float *ks, *vs;    // [rows][nKV]
    uint64_t dstRow;   // pool row of cache row cachePos
    uint64_t maxRows;  // rows the pool holds
};

// What the K/V rows of a call are read from: the f32 store (twins made here), the fp16 store (used in
// place: its layout is the twins'), or the int8 store (twins made here: byte x the row's scale).
struct PrefillKvSource {
    int kind;             // 0 f32, 1 fp16, 2 int8
    const void *k, *v;    // [rows][nKV][hd] of float / __half / int8_t
    const float *ks, *vs; // int8: [rows][nKV] scales
};

// f32 -> fp16 twins of q, K and V in ONE launch (the reference's kF32ToF16 x3,
// GpuElementwiseKernels.hpp:92-101; GPUComputeForward.cu:3957-3968), and -- the K/V rows being in
// registers anyway -- the int8 rows of the new positions (one scale per row and kv head, amax / 127,
// round-half-even: the arithmetic of kvQuantKernel, bit for bit).  q goes float4 by float4; a K/V
// row of one kv head goes to a warp, lane i holding dims 4 i .. 4 i + 3 (and 128 further on at head_dim 256).
// With an int8 source (k8 != nullptr) the K/V rows are bytes and a scale per row and kv head instead of
// floats, and there is no mirror to write.
// MAXV: float4 per lane and row, 1 up to head_dim 128, 2 at 256.
template <int MAXV>
__global__ void __launch_bounds__(256)
f32ToF16MirrorKernel(const float4 *__restrict__ q, const float4 *__restrict__ k, const float4 *__restrict__ v,
                     const uint32_t *__restrict__ k8, const uint32_t *__restrict__ v8, const float *__restrict__ ks8,
                     const float *__restrict__ vs8, uint2 *__restrict__ q16, uint2 *__restrict__ k16,
                     uint2 *__restrict__ v16, size_t nq4, size_t kvRowHeads, uint32_t nvec, size_t mirrorFrom,
                     PrefillMirror mir, uint32_t nKV, unsigned int *__restrict__ err,
                     unsigned int *__restrict__ workCounter) {
    // the attention launch that follows in the stream hands out its work items through this counter
    if (blockIdx.x == 0 && threadIdx.x == 0) *workCounter = 0u;
    gridDepLaunch();  // the attention launch may set itself up while this one drains
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = tid; i < nq4; i += stride) {
        const float4 x = __ldg(q + i);
        uint2 o;
        o.x = packHalf2(x.x, x.y);
        o.y = packHalf2(x.z, x.w);
        q16[i] = o;
    }
    const uint32_t lane = threadIdx.x & 31u;
    for (size_t rh = tid >> 5; rh < kvRowHeads; rh += stride >> 5) {
        // lane i holds float4 i and, at head_dim 256, float4 i + 32 of the row
        float4 kx[MAXV], vx[MAXV];
        bool active[MAXV];
#pragma unroll
        for (int u = 0; u < MAXV; ++u) {
            const uint32_t i4 = lane + 32u * u;
            active[u] = i4 < nvec;
            kx[u] = make_float4(0.f, 0.f, 0.f, 0.f), vx[u] = kx[u];
            if (!active[u]) continue;
            if (k8 != nullptr) {
                const uint32_t kb = __ldg(k8 + rh * nvec + i4), vb = __ldg(v8 + rh * nvec + i4);
                const float sk = __ldg(ks8 + rh), sv = __ldg(vs8 + rh);
                auto b = [](uint32_t w, int i) { return static_cast<float>(static_cast<int8_t>((w >> (8 * i)) & 0xffu)); };
                kx[u] = make_float4(b(kb, 0) * sk, b(kb, 1) * sk, b(kb, 2) * sk, b(kb, 3) * sk);
                vx[u] = make_float4(b(vb, 0) * sv, b(vb, 1) * sv, b(vb, 2) * sv, b(vb, 3) * sv);
            } else {
                kx[u] = __ldg(k + rh * nvec + i4);
                vx[u] = __ldg(v + rh * nvec + i4);
            }
            uint2 o;
            o.x = packHalf2(kx[u].x, kx[u].y);
            o.y = packHalf2(kx[u].z, kx[u].w);
            k16[rh * nvec + i4] = o;
            o.x = packHalf2(vx[u].x, vx[u].y);
            o.y = packHalf2(vx[u].z, vx[u].w);
            v16[rh * nvec + i4] = o;
        }
        if (mir.k8 == nullptr || rh < mirrorFrom) continue;  // warp-uniform
        const size_t dst = mir.dstRow * nKV + (rh - mirrorFrom);
        if (dst >= mir.maxRows * nKV) {
            if (lane == 0) atomicOr(err, kDevErrRowBound);
            continue;
        }
        auto amax4 = [](const float4 &x) { return fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))); };
        float mk = amax4(kx[0]), mv = amax4(vx[0]);
        if (MAXV > 1) mk = fmaxf(mk, amax4(kx[MAXV - 1])), mv = fmaxf(mv, amax4(vx[MAXV - 1]));
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
            mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
        }
        const float sk = mk > 0.0f ? __fdiv_rn(mk, 127.0f) : 1.0f;
        const float sv = mv > 0.0f ? __fdiv_rn(mv, 127.0f) : 1.0f;
        if (lane == 0) {
            mir.ks[dst] = sk;
            mir.vs[dst] = sv;
        }
        auto q8 = [](float x, float sc) -> uint32_t {
            int qv = __float2int_rn(__fdiv_rn(x, sc));
            qv = qv < -128 ? -128 : (qv > 127 ? 127 : qv);
            return static_cast<uint32_t>(qv) & 0xffu;
        };
#pragma unroll
        for (int u = 0; u < MAXV; ++u) {
            if (!active[u]) continue;
            const uint32_t i4 = lane + 32u * u;
            reinterpret_cast<uint32_t *>(mir.k8)[dst * nvec + i4] =
                    q8(kx[u].x, sk) | (q8(kx[u].y, sk) << 8) | (q8(kx[u].z, sk) << 16) | (q8(kx[u].w, sk) << 24);
            reinterpret_cast<uint32_t *>(mir.v8)[dst * nvec + i4] =
                    q8(vx[u].x, sv) | (q8(vx[u].y, sv) << 8) | (q8(vx[u].z, sv) << 16) | (q8(vx[u].w, sv) << 24);
        }
    }
}

struct PrefillF16Params {
    float *out;        // [seqLen][nHeads][128] f32
    uint32_t seqLen, nHeads, nKV, group;
    uint32_t cachePos;  // query row r sits at position cachePos + r and sees K/V rows [0, cachePos + r]
    uint32_t nQTiles;   // query blocks of itemRows rows
    uint32_t itemRows;  // 256: two query tiles per work item; 128: one (short calls, so that every SM gets an item)
    float scaleLog2;   // invSqrt * log2(e)
    unsigned int *err;
    unsigned int *workCounter;  // zero at launch; item gridDim.x + n goes to the n-th request
    uint32_t totalItems;        // nQTiles * nHeads (query block, head) pairs, heavy blocks first
    uint32_t out32;             // out is 32-byte aligned: rows can be written with 32-byte stores
#ifdef TC_TRACE
    unsigned long long *trace;  // [8 roles][64 steps][4 stamps] of block 0
#endif
};

#ifdef TC_TRACE
unsigned long long *g_pfTrace = nullptr;
__device__ __forceinline__ unsigned long long pfTime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define PF_BLK(k) do { if (p.trace) p.trace[8u * 64u * 4u + item * 8u + (k)] = pfTime(); } while (0)
#define PF_STAMP(role, step, k) do { if (p.trace && item == 0u && (step) < 64u) p.trace[((role) * 64u + (step)) * 4u + (k)] = pfTime(); } while (0)
#else
#define PF_STAMP(role, step, k) do { } while (0)
#define PF_BLK(k) do { } while (0)
#endif

// HD = head_dim (64, 128 or 256): a tile is HD / 64 halves of 64 columns (128 bytes, one swizzle span)
// each.  BN = tokens per KV tile: 64, or 32 at head_dim 256, where one query tile and its 256-column
// accumulator take the room two tiles take at head_dim 128 (a block then serves one query tile).
template <int HD, int BN>
struct PrefillF16Smem {
    static constexpr int kHalves = HD / 64;
    static constexpr int kQTiles = HD > 128 ? 1 : 2;   // query tiles a block holds
    static constexpr int kQHalf = kPfBM * 128;         // 16 KB: 128 rows x 64 fp16
    static constexpr int kKvHalf = BN * 128;           // BN rows x 64 fp16
    static constexpr int kQTile = kHalves * kQHalf;    // head_dim 128: 32 KB
    static constexpr int kKvTile = kHalves * kKvHalf;  // head_dim 128: 16 KB
    static constexpr int kQ = 0;                       // two query tiles
    static constexpr int kK01 = kQTiles * kQTile;      // K_0, K_1 (the products issued before the loop)
    static constexpr int kStage = kK01 + 2 * kKvTile;  // stage s: K slot, then V slot
    static constexpr int kStageBytes = 2 * kKvTile;
    static constexpr int kBars = kStage + kPfStages * kStageBytes;
    // qFull, k01Full, stage full + empty, sFull[2][2], pFull[2][2], pvDone[2], pvBuf[2][2], qFree[2], itemFull[4]
    static constexpr int kNumBars = 2 + 2 * kPfStages + 4 + 4 + 2 + 4 + 2 + 4;
    static constexpr int kTmemSlot = kBars + kNumBars * 8;
    static constexpr int kItemSlots = kTmemSlot + 16;  // four work item indices
    static constexpr int kTotal = kItemSlots + 16 + 1024;
};

__device__ __forceinline__ bool pfWait(uint64_t *bar, uint32_t parity, unsigned int *err, uint32_t bit) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbarTryWait(bar, parity)) return true;
        // somebody has already given up: what this thread waits for will not come either
        if ((*reinterpret_cast<volatile unsigned int *>(err) & (kDevErrFullWait | kDevErrEmptyWait | kDevErrMmaWait)) != 0u)
            return false;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    atomicOr(err, bit);
    return false;
}

// one 32-byte store (the address has to be 32-byte aligned)
__device__ __forceinline__ void stGlobalV8(float *dst, float a, float b, float c, float d, float e, float f, float g,
                                           float h) {
    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d),
                 "f"(e), "f"(f), "f"(g), "f"(h)
                 : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// A matrix descriptor whose start address is moved by `bytes` (the address field holds
// bytes >> 4 in its low 14 bits; shared memory is far smaller than their range, so the sum
// never carries out of the field).
__device__ __forceinline__ uint64_t descAdvance(uint64_t d, uint32_t bytes) { return d + (bytes >> 4); }

// What one work item (a 256-row query block of one head) covers.  Query tile X (0 = A, 1 = B) holds
// rows m0 + 128 X .. at positions cachePos + row; it sees KV tiles 0 .. nX - 1 (64 tokens each; the
// last two or three straddle its diagonal).  B may lie wholly past the sequence; a call with fewer
// 256-row items than SMs is cut into 128-row items instead, which have no tile B.
struct PfItem {
    uint32_t head, kvHead, m0, nA, nB, nTiles;
};
template <int BN>
__device__ __forceinline__ PfItem pfItem(const PrefillF16Params &p, uint32_t item) {
    PfItem it;
    const uint32_t qb = p.nQTiles - 1u - item / p.nHeads;  // heavy query blocks (long causal prefixes) first
    it.head = item % p.nHeads;
    it.kvHead = it.head / p.group;
    it.m0 = qb * p.itemRows;
    const bool activeB = p.itemRows > kPfBM && it.m0 + kPfBM < p.seqLen;
    it.nA = (p.cachePos + it.m0 + kPfBM + BN - 1u) / BN;
    it.nB = activeB ? (p.cachePos + it.m0 + 2u * kPfBM + BN - 1u) / BN : 0u;
    it.nTiles = activeB ? it.nB : it.nA;
    return it;
}

// 416 threads: warps 0-3 softmax of query tile A, warps 4-7 softmax of query tile B
// (rows 128 further down), warp 8 TMA producer and scheduler, warps 9 and 10 issue the score
// products of A and B, warps 11 and 12 their P.V products.
//
// One block per SM works through (query block, head) items: its first is blockIdx.x, the following
// ones come from a counter, so the heavy items start first and the light ones fill in behind them.
// The roles walk the item list independently and meet only at the mbarriers, which are never
// initialised again: every ring (K/V stages, score buffers, P.V commits) is indexed by a count that
// runs on from item to item.  So the next item's query tiles load as soon as this item's last score
// product has been issued, its first scores are in TMEM while the softmax threads still write this
// item's output, and tile A moves on while tile B finishes its two extra diagonal tiles.
constexpr int kPfThreads = 416;
template <int HD, int BN>
__global__ void __launch_bounds__(kPfThreads, 1)
prefillF16Kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const PrefillF16Params p) {
    using L = PrefillF16Smem<HD, BN>;
    constexpr int NC = BN / 32;  // 32-column chunks of a score row
    constexpr uint32_t NS = kPfStages;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kBars);
    uint64_t *qFull = bars, *k01Full = bars + 1, *stFull = bars + 2, *stEmpty = stFull + NS,
             *sFull = stEmpty + NS /* [x][b] */, *pFull = sFull + 4 /* [x][b] */, *pvDone = pFull + 4 /* [x] */,
             *pvBuf = pvDone + 2 /* [x][b] */, *qFree = pvBuf + 4 /* [x] */, *itemFull = qFree + 2 /* [4] */;
    uint32_t *tmemSlot = reinterpret_cast<uint32_t *>(smem + L::kTmemSlot);
    volatile uint32_t *itemSlots = reinterpret_cast<volatile uint32_t *>(smem + L::kItemSlots);  // [4]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;

    if (threadIdx.x == 0) {
        mbarInit(qFull, 1);
        mbarInit(k01Full, 1);
        for (uint32_t s = 0; s < NS; ++s) {
            mbarInit(&stFull[s], 1);
            mbarInit(&stEmpty[s], 4);  // all four MMA warps release a stage
        }
        for (int i = 0; i < 4; ++i) {
            mbarInit(&sFull[i], 1);
            mbarInit(&pFull[i], 4);  // one arrival per warp
            mbarInit(&pvBuf[i], 1);
            mbarInit(&itemFull[i], 1);
        }
        mbarInit(&pvDone[0], 1);
        mbarInit(&pvDone[1], 1);
        mbarInit(&qFree[0], 1);  // score warp X is done with the query tiles and K_0, K_1
        mbarInit(&qFree[1], 1);
        fenceBarrierInit();
        tmaPrefetchDesc(&tmQ);
        tmaPrefetchDesc(&tmK);
        tmaPrefetchDesc(&tmV);
    }
    if (warp == 0) {
        tmemAlloc(tmemSlot, 512);
        tmemRelinquish();
        tcFenceBefore();
    }
    __syncthreads();
    tcFenceAfter();
    const uint32_t tmemBase = *reinterpret_cast<volatile uint32_t *>(tmemSlot);
    // O of tile X at columns 128 X; S buffer b of tile X at 256 + 128 X + 64 b (its fp16
    // probabilities overwrite the first 32 of those columns)

    // The n-th item of this block: the producer publishes it in slot n % 4 (the end of the list as
    // an index past the last item); the other roles pick it up there.
    auto takeItem = [&](uint32_t n, uint32_t &item) -> bool {
        if (!pfWait(&itemFull[n & 3u], (n >> 2) & 1u, p.err, kDevErrFullWait)) return false;
        item = itemSlots[n & 3u];
        return item < p.totalItems;
    };

    if (warp == 8) {
        // ------------------------ TMA producer and scheduler ------------------------
        if (lane == 0) {
            uint32_t item = blockIdx.x, g = 0;  // g: K/V tiles requested so far, over all items
            gridDepWait();  // the twins and the work counter come from the launch in front
            itemSlots[0] = item;
            mbarArrive(&itemFull[0]);
            bool ok = true;
            for (uint32_t n = 0; ok && item < p.totalItems; ++n) {
                const PfItem it = pfItem<BN>(p, item);
                PF_BLK(0);
#ifdef TC_TRACE
                if (p.trace) { unsigned sm; asm("mov.u32 %0, %%smid;" : "=r"(sm)); p.trace[8u * 64u * 4u + item * 8u + 6] = sm; }
#endif
                // the query tiles and K_0, K_1 are free once both score warps have issued the last
                // product of the previous item that reads them, and those products are complete
                if (n > 0 && !(pfWait(&qFree[0], (n - 1u) & 1u, p.err, kDevErrEmptyWait) &&
                               pfWait(&qFree[1], (n - 1u) & 1u, p.err, kDevErrEmptyWait))) {
                    ok = false;
                    break;
                }
                mbarExpectTx(qFull, L::kQTiles * L::kQTile);
#pragma unroll
                for (int x = 0; x < L::kQTiles; ++x)
#pragma unroll
                    for (int h = 0; h < L::kHalves; ++h)
                        tmaLoad3D(smem + L::kQ + x * L::kQTile + h * L::kQHalf, &tmQ, qFull, 64 * h, it.head,
                                  it.m0 + x * kPfBM);
                // K_0 and K_1 feed the products issued ahead of the loop (nTiles >= 2 always)
                mbarExpectTx(k01Full, 2 * L::kKvTile);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint8_t *kd = smem + L::kK01 + j * L::kKvTile;
#pragma unroll
                    for (int h = 0; h < L::kHalves; ++h)
                        tmaLoad3D(kd + h * L::kKvHalf, &tmK, k01Full, 64 * h, it.kvHead, j * BN);
                }
                // The next item is drawn late -- with the third last tile request, some six tiles before
                // the consumers finish this item -- so that the blocks which finish first take the
                // heavier of the remaining items.
                const uint32_t drawAt = it.nTiles >= 3u ? it.nTiles - 3u : 0u;
                uint32_t drawn = 0, flags = 0;
                for (uint32_t j = 0; j < it.nTiles; ++j, ++g) {
                    if (j == drawAt) {
                        flags = *reinterpret_cast<volatile unsigned int *>(p.err);
                        drawn = gridDim.x + atomicAdd(p.workCounter, 1u);
                    }
                    const uint32_t s = g % NS;
                    if (g >= NS && !pfWait(&stEmpty[s], ((g / NS) - 1u) & 1u, p.err, kDevErrEmptyWait)) {
                        ok = false;
                        break;
                    }
                    uint8_t *kd = smem + L::kStage + s * L::kStageBytes, *vd = kd + L::kKvTile;
                    const bool withK = j + 2 < it.nTiles;
                    mbarExpectTx(&stFull[s], withK ? 2 * L::kKvTile : L::kKvTile);
#pragma unroll
                    for (int h = 0; h < L::kHalves; ++h) {
                        if (withK) tmaLoad3D(kd + h * L::kKvHalf, &tmK, &stFull[s], 64 * h, it.kvHead, (j + 2) * BN);
                        tmaLoad3D(vd + h * L::kKvHalf, &tmV, &stFull[s], 64 * h, it.kvHead, j * BN);
                    }
                }
                if (!ok) break;
                // a wait that ran out anywhere ends the launch: the flag is the caller's to read
                constexpr unsigned int kWaitBits = kDevErrFullWait | kDevErrEmptyWait | kDevErrMmaWait;
                const uint32_t next = (flags & kWaitBits) != 0u ? p.totalItems : drawn;
                itemSlots[(n + 1u) & 3u] = next;
                mbarArrive(&itemFull[(n + 1u) & 3u]);
                item = next;
            }
            // the last release of every stage has to have arrived before the block leaves
            for (uint32_t back = 0; ok && back < NS && back < g; ++back) {
                const uint32_t gg = g - 1u - back;
                ok = pfWait(&stEmpty[gg % NS], (gg / NS) & 1u, p.err, kDevErrEmptyWait);
            }
        }
    } else if (warp >= 9) {
        // ------------------------------- MMA issuers -------------------------------
        // Issuing one tcgen05.mma costs its thread about a hundred cycles whatever the shape, and
        // threads of different warps issue concurrently.  So the score products and the P.V products
        // of a query tile have an issuing warp each: warp 9 + X issues S_X(t) = Q_X K^T (M128 N64
        // K16 x8), warp 11 + X issues O_X += P_X(t) V (A from TMEM, B = V MN-major from shared
        // memory, K16 x4).  t counts the tiles of X over all items; tile t uses score buffer t % 2,
        // and S_X(t+2) goes into the buffer P_X(t) occupies: the score warp waits for the commit of
        // that P.V product (pvBuf) before it issues.
        // All 32 lanes run this warp-uniform code; only lane 0 executes the tcgen05 instructions.
        const uint32_t x = (warp - 9u) & 1u;
        const bool pvRole = warp >= 11u;
        const uint32_t issue = lane == 0 ? 1u : 0u;
        constexpr uint32_t idQK = umaInstrDescF16(kPfBM, BN, 0, 0);
        constexpr uint32_t idPV = umaInstrDescF16(kPfBM, HD, 0, 1);
        const uint64_t dQ = umaSmemDesc(smemAddr(smem + L::kQ + x * L::kQTile), 16, 1024);
        const uint64_t dK01 = umaSmemDesc(smemAddr(smem + L::kK01), 16, 1024);
        const uint64_t dKs = umaSmemDesc(smemAddr(smem + L::kStage), 16, 1024);
        const uint64_t dVs = umaSmemDesc(smemAddr(smem + L::kStage + L::kKvTile), L::kKvHalf, 1024);
        const uint32_t tO = tmemBase + 128u * x, tS0 = tmemBase + 256u + 128u * x;
        // score product of running tile tt from the K tile at descriptor dK; tt >= 2 first waits
        // until the P.V product of tile tt - 2 has left the buffer
        auto issueQK = [&](uint64_t dK, uint32_t tt) -> bool {
            if (tt >= 2u && !pfWait(&pvBuf[2u * x + (tt & 1u)], ((tt - 2u) >> 1) & 1u, p.err, kDevErrMmaWait)) return false;
            tcFenceAfter();
#pragma unroll
            for (uint32_t ks = 0; ks < HD / 16; ++ks) {
                // k step ks: dims 16 ks .. +15 = 32 bytes inside the (ks >> 2)-th 64-dim half
                umaMmaSSIf(issue, tS0 + 64u * (tt & 1u), descAdvance(dQ, (ks >> 2) * L::kQHalf + (ks & 3u) * 32u),
                           descAdvance(dK, (ks >> 2) * L::kKvHalf + (ks & 3u) * 32u), idQK, ks > 0 ? 1u : 0u);
            }
            umaCommitIf(issue, &sFull[2u * x + (tt & 1u)]);
            return true;
        };
        uint32_t g = 0, t = 0, item = 0;  // K/V tiles consumed, tiles of X done, over all items
        bool ok = true;
        for (uint32_t n = 0; ok && takeItem(n, item); ++n) {
            const PfItem it = pfItem<BN>(p, item);
            const uint32_t myTiles = x == 0 ? it.nA : it.nB;
            if (!pvRole) {
                if (myTiles != 0) {
                    ok = pfWait(qFull, n & 1u, p.err, kDevErrFullWait) && pfWait(k01Full, n & 1u, p.err, kDevErrFullWait);
                    ok = ok && issueQK(dK01, t) && issueQK(descAdvance(dK01, L::kKvTile), t + 1u);
                    if (myTiles <= 2u) umaCommitIf(issue, &qFree[x]);
                }
            }
            // Every stage is released by all four warps, also the ones past a tile's diagonal -- but
            // only after the stage has been filled: a warp with nothing to do must not run ahead and
            // hand in the release of a later round, or the barrier would complete without the warp
            // that still reads the stage.
            for (uint32_t j = 0; ok && j < it.nTiles; ++j, ++g) {
                const uint32_t s = g % NS;
                ok = pfWait(&stFull[s], (g / NS) & 1u, p.err, kDevErrFullWait);
                if (!ok) break;
                if (pvRole && j < myTiles) {
                    const uint32_t tt = t + j;
                    if (lane == 0) PF_STAMP(4u + x, j, 0);
                    ok = pfWait(&pFull[2u * x + (tt & 1u)], (tt >> 1) & 1u, p.err, kDevErrMmaWait);
                    if (lane == 0) PF_STAMP(4u + x, j, 1);
                    if (!ok) break;
                    tcFenceAfter();
                    const uint64_t dV = descAdvance(dVs, s * L::kStageBytes);
                    const uint32_t tP = tS0 + 64u * (tt & 1u);
#pragma unroll
                    for (uint32_t ks = 0; ks < BN / 16; ++ks)  // 16 tokens per step: 8 columns of fp16 P, 2 KB of V
                        umaMmaTSIf(issue, tO, tP + ks * 8u, descAdvance(dV, ks * 2048u), idPV, (j > 0 || ks > 0) ? 1u : 0u);
                    umaCommitIf(issue, &pvDone[x]);
                    umaCommitIf(issue, &pvBuf[2u * x + (tt & 1u)]);
                    if (lane == 0) PF_STAMP(4u + x, j, 2);
                } else if (!pvRole && j + 2 < myTiles) {
                    if (lane == 0) PF_STAMP(2u + x, j, 0);
                    ok = issueQK(descAdvance(dKs, s * L::kStageBytes), t + j + 2u);
                    if (!ok) break;
                    if (lane == 0) PF_STAMP(2u + x, j, 2);
                    // the item's last score product: the query tiles may be replaced once it is complete
                    if (j + 3u == myTiles) umaCommitIf(issue, &qFree[x]);
                }
                umaCommitIf(issue, &stEmpty[s]);
            }
            // A tile that is not there still hands in its phase of qFree, one per item -- but only
            // behind the item's last stage: the producer fills that stage after it has looked at the
            // previous phase, so this warp cannot complete two phases before the producer has seen
            // the first (a parity wait cannot tell those apart).
            if (!pvRole && myTiles == 0u && ok) umaCommitIf(issue, &qFree[x]);
            t += myTiles;
        }
        if (pvRole && ok) {
            // nobody waits for the last two buffer commits; they have to land before the block leaves
            for (uint32_t tt = t >= 2u ? t - 2u : 0u; tt < t; ++tt)
                if (!pfWait(&pvBuf[2u * x + (tt & 1u)], (tt >> 1) & 1u, p.err, kDevErrMmaWait)) break;
        }
    } else {
        // --------------------------------- softmax ---------------------------------
        const uint32_t x = warp >> 2;                         // which query tile this warpgroup owns
        const uint32_t row = (warp & 3u) * 32u + lane;        // row of that tile = TMEM lane
        const uint32_t laneBase = ((warp & 3u) * 32u) << 16;  // TMEM lane field
        const uint32_t rowInBlock = x * kPfBM + row;          // row inside the 256-row block
        const uint32_t tO = tmemBase + 128u * x;
        uint32_t t = 0, item = 0;  // tiles of X done over all items
        bool ok = true;
        for (uint32_t n = 0; ok && takeItem(n, item); ++n) {
            const PfItem it = pfItem<BN>(p, item);
            const uint32_t m0 = it.m0, head = it.head;
            const uint32_t rq = m0 + rowInBlock;  // query position
            const uint32_t myTiles = x == 0 ? it.nA : it.nB;
            if (myTiles == 0) continue;
            float m = kNegBig, l = 0.0f;
            for (uint32_t j = 0; j < myTiles; ++j) {
                const uint32_t tt = t + j, b = tt & 1u;
                const uint32_t tS = tmemBase + 256u + 128u * x + 64u * b;
                if (row == 0) PF_STAMP(x, j, 0);
                if (!pfWait(&sFull[2u * x + b], (tt >> 1) & 1u, p.err, kDevErrMmaWait)) {
                    ok = false;
                    break;
                }
                if (row == 0) PF_STAMP(x, j, 1);
                if (row == 0 && x == 0 && j == 0) PF_BLK(2);
                tcFenceAfter();
                uint32_t r[NC][32];  // the BN scores of this row
#pragma unroll
                for (int c = 0; c < NC; ++c) tmemLd32(tS + laneBase + 32u * c, r[c]);
                tmemLdWait();
                if (row == 0 && x == 0) PF_STAMP(6u, j, 0);
                if (BN * j + (BN - 1u) > p.cachePos + m0 + x * kPfBM) {
                    // causal edge (the tile reaches past the position of this tile's first row): token
                    // 64 j + c is visible iff it is not past the query position; relative to the block's
                    // first row that is 64 j - (cachePos + m0) + c <= rowInBlock
                    const int32_t first = static_cast<int32_t>(BN * j) - static_cast<int32_t>(p.cachePos + m0);
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (first + c * 32 + i > static_cast<int32_t>(rowInBlock)) r[c][i] = 0xff800000u;  // -inf
                }
                float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
                for (int c = 0; c < NC; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        mxa = max3(mxa, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                        mxb = max3(mxb, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                    }
                const float mx = fmaxf(mxa, mxb) * p.scaleLog2;  // scale > 0: max commutes with it
                const float mNew = mx > m + kPfLazyLog2 ? mx : m;
                const float alpha = fastExp2(m - mNew);
                const bool rescale = j > 0 && __any_sync(0xffffffffu, mNew != m);
                if (row == 0 && x == 0) PF_STAMP(6u, j, 1);
                // O may only be touched between two of its PV products: the previous one has to be
                // complete (the next one cannot start before this thread publishes P).  The last
                // step takes the wait in any case: a parity wait can only tell the current phase from
                // the one before it, and the final wait below must not find the barrier two behind.
                // (pvDone completes one phase per tile, so its parity follows the running count.)
                if (j > 0 && (rescale || j + 1u == myTiles)) {
                    if (!pfWait(&pvDone[x], (tt - 1u) & 1u, p.err, kDevErrMmaWait)) {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
                }
                if (rescale) {
#pragma unroll 1
                    for (uint32_t c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmemLd32(tO + laneBase + c * 32u, o);
                        tmemLdWait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmemSt32(tO + laneBase + c * 32u, o);
                    }
                    tmemStWait();
                }
                m = mNew;
                // probabilities as fp16 pairs over the first 32 columns of this S buffer: the A
                // operand of the PV product (every score of the row is already in registers)
                // Pairs of elements with packed f32x2 arithmetic (scale-and-shift, row sum).  Evaluating
                // part of the exponentials on the FMA pipe (round-to-integer trick + cubic) was measured
                // at 25 / 50 / 75 % of the pairs: 716 / 699 / 694 TFLOP/s against 732 with all of them on
                // the special-function unit; a second implementation (magic-constant integer split, cubic
                // with relative error 7.5e-5, exponent patched by an integer add, selected per pair at run
                // time) lost a fifth from 0 to 4 of every 4 pairs.  Exponentials of fp16 PAIRS
                // (ex2.approx.f16x2 on the rounded exponent, row sum over fp16 partial sums) pass the
                // parity tests but are slower too: 673 TFLOP/s.  Per 64-token step a softmax thread is busy
                // for 0.9 us, 0.8 of them in these two loops; more instructions cost time in proportion,
                // whichever pipe they run on.
                const float2 scale2 = make_float2(p.scaleLog2, p.scaleLog2), negM2 = make_float2(-m, -m);
                float psum = 0.0f;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    uint32_t h[16];
                    {
                        float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])),
                                                         scale2, negM2);
                            const float2 p2 = make_float2(fastExp2(x2.x), fastExp2(x2.y));
                            sum2 = __fadd2_rn(sum2, p2);
                            h[i] = packHalf2(p2.x, p2.y);
                        }
                        psum += sum2.x + sum2.y;
                    }
                    tmemSt16(tS + laneBase + c * 16u, h);
                    if (row == 0 && x == 0) PF_STAMP(6u, j, 2 + c);
                }
                l = l * alpha + psum;
                tmemStWait();
                tcFenceBefore();
                __syncwarp();
                if (lane == 0) mbarArrive(&pFull[2u * x + b]);
                if (row == 0) PF_STAMP(x, j, 2);
                if (row == 0 && j + 1u == myTiles) PF_BLK(3u + x);
            }
            if (!ok || !pfWait(&pvDone[x], (t + myTiles - 1u) & 1u, p.err, kDevErrMmaWait)) {
                ok = false;
                break;
            }
            tcFenceAfter();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float *orow = p.out + (static_cast<size_t>(rq) * p.nHeads + head) * HD;
#pragma unroll 1
            for (uint32_t c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmemLd32(tO + laneBase + c * 32u, o);
                tmemLdWait();
                if (rq < p.seqLen && !p.out32) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4 *>(orow + c * 32 + 4 * i) =
                                make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                            __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
                } else if (rq < p.seqLen) {
                    // 32 bytes per store: a thread owns its row, so a warp's store touches 32 rows, and
                    // whole sectors halve the number of transactions against 16-byte stores
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        stGlobalV8(orow + c * 32 + 8 * i, __uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv,
                                   __uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv,
                                   __uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv,
                                   __uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
                }
            }
            if (threadIdx.x == 0) PF_BLK(5);
            t += myTiles;
        }
    }
    tcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        tcFenceAfter();
        tmemDealloc(tmemBase, 512);
    }
}

static int f16Map(const void *base, uint32_t hd, uint32_t heads, uint32_t rows, uint32_t boxRows, CUtensorMap *out) {
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.rank = 3;
    key.elemBytes = 2;
    key.swizzle = 3;
    key.dims[0] = hd;
    key.dims[1] = heads;
    key.dims[2] = rows;
    key.strides[0] = hd * 2;
    key.strides[1] = static_cast<uint64_t>(heads) * hd * 2;
    key.box[0] = 64;  // 128 bytes: one swizzle span
    key.box[1] = 1;
    key.box[2] = boxRows;
    return getTensorMap(key, out);
}

static size_t prefillScratchBytes(uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV, uint32_t hd) {
    // fp16 twins: q [seqLen][nHeads][hd], k and v [cachePos + seqLen][nKV][hd]; each region 1 KB aligned;
    // then the work counter of the attention launch
    auto al = [](size_t x) { return (x + 1023) & ~size_t(1023); };
    return al(static_cast<size_t>(seqLen) * nHeads * hd * 2) +
           2 * al((static_cast<size_t>(cachePos) + seqLen) * nKV * hd * 2) + 1024;  // + the work counter
}

}  // namespace tc

#ifdef TC_TRACE
extern "C" void tc_debug_trace_prefill(unsigned long long *buf) { tc::g_pfTrace = buf; }
#endif

extern "C" {

int tc_attn_prefill_f16_scratch_bytes(uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV, uint32_t hd,
                                      size_t *bytes) {
    TC_REQUIRE(bytes != nullptr, TC_EINVAL, "tc_attn_prefill_f16_scratch_bytes: null output");
    TC_REQUIRE(hd == 64 || hd == 128 || hd == 256, TC_EUNSUPPORTED, "tc_attn_prefill_f16: head_dim %u (built for 64, 128 and 256)", hd);
    *bytes = tc::prefillScratchBytes(seqLen, cachePos, nHeads, nKV, hd);
    return TC_OK;
}

static int prefillF16Impl(const float *q, const tc::PrefillKvSource &src, float *out, void *scratch,
                          size_t scratchBytes, uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                          uint32_t hd, float invSqrt, const tc::PrefillMirror &mir, tc_stream stream) {
    using namespace tc;
    const void *kvK = src.k, *kvV = src.v;
    TC_REQUIRE(q && kvK && kvV && out && scratch, TC_EINVAL, "tc_attn_prefill_f16: null pointer");
    TC_REQUIRE(src.kind != 2 || (src.ks && src.vs), TC_EINVAL, "tc_attn_prefill_f16: null scale pointer");
    TC_REQUIRE(hd == 64 || hd == 128 || hd == 256, TC_EUNSUPPORTED, "tc_attn_prefill_f16: head_dim %u (built for 64, 128 and 256)", hd);
    TC_REQUIRE(nKV > 0 && nHeads % nKV == 0, TC_EINVAL, "tc_attn_prefill_f16: nHeads %u not a multiple of nKV %u",
               nHeads, nKV);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kvK) | reinterpret_cast<uintptr_t>(kvV) |
                 reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0,
               TC_EINVAL, "tc_attn_prefill_f16: pointers need 16-byte alignment");
    if (seqLen == 0) return TC_OK;
    TC_REQUIRE(static_cast<uint64_t>(cachePos) + seqLen < (1ull << 31), TC_EUNSUPPORTED,
               "tc_attn_prefill_f16: %u + %u rows", cachePos, seqLen);
    // an fp16 store is read in place: only q's twin and the counter live in the scratch
    const size_t need = src.kind == 1 ? prefillScratchBytes(seqLen, 0, nHeads, 0, hd)
                                      : prefillScratchBytes(seqLen, cachePos, nHeads, nKV, hd);
    TC_REQUIRE(scratchBytes >= need, TC_EWORKSPACE, "tc_attn_prefill_f16: scratch of %zu bytes, %zu needed",
               scratchBytes, need);
    TC_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 1023u) == 0, TC_EINVAL,
               "tc_attn_prefill_f16: scratch needs 1024-byte alignment");
    const int sms = numSMs();
    // two query tiles per item keep both softmax warpgroups of a block busy; a call too short to give
    // every SM such an item (a 512-row chunk of a prompt: 2 x nHeads items) is cut into one-tile items
    // (head_dim 256: a block holds one query tile, so its items are always one-tile items)
    const uint32_t itemRows =
            hd == 256 || static_cast<uint64_t>((seqLen + 2 * kPfBM - 1) / (2 * kPfBM)) * nHeads < static_cast<uint64_t>(sms)
                    ? kPfBM
                    : 2 * kPfBM;
    const uint32_t bn = hd == 256 ? 32u : 64u;  // tokens per KV tile
    const uint32_t nQTiles = (seqLen + itemRows - 1) / itemRows;
    TC_REQUIRE(static_cast<uint64_t>(nQTiles) * nHeads < (1ull << 31), TC_EUNSUPPORTED,
               "tc_attn_prefill_f16: grid too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto al = [](size_t x) { return (x + 1023) & ~size_t(1023); };
    const size_t qElems = static_cast<size_t>(seqLen) * nHeads * hd;
    const uint32_t kvRows = cachePos + seqLen;  // the cache rows this call attends over
    const size_t kvElems = static_cast<size_t>(kvRows) * nKV * hd;
    uint8_t *sc = static_cast<uint8_t *>(scratch);
    void *q16 = sc, *k16 = sc + al(qElems * 2), *v16 = sc + al(qElems * 2) + al(kvElems * 2);
    unsigned int *workCounter = reinterpret_cast<unsigned int *>(sc + al(qElems * 2) + 2 * al(kvElems * 2));
    if (src.kind == 1) {
        k16 = const_cast<void *>(kvK);
        v16 = const_cast<void *>(kvV);
        workCounter = reinterpret_cast<unsigned int *>(sc + al(qElems * 2));
    }
    unsigned int *err = devErrorWord();
    TC_REQUIRE(err != nullptr, TC_ECUDA, "tc_attn_prefill_f16: no device error word");
    {
        const size_t nq4 = qElems / 4, kvRowHeads = src.kind == 1 ? 0 : static_cast<size_t>(kvRows) * nKV;
        const size_t threads = std::max(nq4, kvRowHeads * 32);
        const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((threads + 255) / 256, static_cast<size_t>(sms) * 16));
        const bool i8 = src.kind == 2;
        auto conv = hd > 128 ? f32ToF16MirrorKernel<2> : f32ToF16MirrorKernel<1>;
        conv<<<blocks, 256, 0, st>>>(
                reinterpret_cast<const float4 *>(q), i8 ? nullptr : static_cast<const float4 *>(kvK),
                i8 ? nullptr : static_cast<const float4 *>(kvV), i8 ? static_cast<const uint32_t *>(kvK) : nullptr,
                i8 ? static_cast<const uint32_t *>(kvV) : nullptr, src.ks, src.vs, static_cast<uint2 *>(q16),
                static_cast<uint2 *>(k16), static_cast<uint2 *>(v16), nq4, kvRowHeads, hd / 4,
                static_cast<size_t>(cachePos) * nKV, mir, nKV, err, workCounter);
    }
    TC_CUDA_OK(cudaGetLastError());
    CUtensorMap tmQ, tmK, tmV;
    int rc = f16Map(q16, hd, nHeads, seqLen, kPfBM, &tmQ);
    if (rc != TC_OK) return rc;
    rc = f16Map(k16, hd, nKV, kvRows, bn, &tmK);
    if (rc != TC_OK) return rc;
    rc = f16Map(v16, hd, nKV, kvRows, bn, &tmV);
    if (rc != TC_OK) return rc;
    PrefillF16Params prm;
    prm.out = out;
    prm.seqLen = seqLen;
    prm.cachePos = cachePos;
    prm.nHeads = nHeads;
    prm.nKV = nKV;
    prm.group = nHeads / nKV;
    prm.nQTiles = nQTiles;
    prm.itemRows = itemRows;
    prm.scaleLog2 = invSqrt * kLog2e;
    prm.err = err;
    prm.workCounter = workCounter;
    prm.totalItems = nQTiles * nHeads;
    prm.out32 = (reinterpret_cast<uintptr_t>(out) & 31u) == 0 ? 1u : 0u;
#ifdef TC_TRACE
    prm.trace = tc::g_pfTrace;
#endif
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(prefillF16Kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        PrefillF16Smem<64, 64>::kTotal));
        TC_CUDA_OK(cudaFuncSetAttribute(prefillF16Kernel<128, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        PrefillF16Smem<128, 64>::kTotal));
        TC_CUDA_OK(cudaFuncSetAttribute(prefillF16Kernel<256, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        PrefillF16Smem<256, 32>::kTotal));
        attrDone[dev] = true;
    }
    const uint32_t grid = std::min<uint32_t>(prm.totalItems, static_cast<uint32_t>(sms));  // one block per SM
    // programmatic dependent launch: the blocks allocate TMEM and set up their barriers while the twins
    // launch drains; the producer waits for it before its first load (nothing else reads its outputs)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kPfThreads);
    cfg.dynamicSmemBytes = hd == 64 ? PrefillF16Smem<64, 64>::kTotal
                                    : (hd == 128 ? PrefillF16Smem<128, 64>::kTotal : PrefillF16Smem<256, 32>::kTotal);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (hd == 64)
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, prefillF16Kernel<64, 64>, tmQ, tmK, tmV, prm));
    else if (hd == 128)
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, prefillF16Kernel<128, 64>, tmQ, tmK, tmV, prm));
    else
        TC_CUDA_OK(cudaLaunchKernelEx(&cfg, prefillF16Kernel<256, 32>, tmQ, tmK, tmV, prm));
    return TC_OK;
}

int tc_attn_prefill_f16(const float *q, const float *kvK, const float *kvV, float *out, void *scratch,
                        size_t scratchBytes, uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                        uint32_t hd, float invSqrt, tc_stream stream) {
    tc::PrefillMirror none;
    memset(&none, 0, sizeof(none));
    const tc::PrefillKvSource src = {0, kvK, kvV, nullptr, nullptr};
    return prefillF16Impl(q, src, out, scratch, scratchBytes, seqLen, cachePos, nHeads, nKV, hd, invSqrt, none, stream);
}

int tc_attn_prefill_f16_kvhalf(const float *q, const void *kvK16, const void *kvV16, float *out, void *scratch,
                               size_t scratchBytes, uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                               uint32_t hd, float invSqrt, tc_stream stream) {
    tc::PrefillMirror none;
    memset(&none, 0, sizeof(none));
    const tc::PrefillKvSource src = {1, kvK16, kvV16, nullptr, nullptr};
    return prefillF16Impl(q, src, out, scratch, scratchBytes, seqLen, cachePos, nHeads, nKV, hd, invSqrt, none, stream);
}

int tc_attn_prefill_f16_i8(const float *q, const int8_t *k8, const int8_t *v8, const float *ks, const float *vs,
                           float *out, void *scratch, size_t scratchBytes, uint32_t seqLen, uint32_t cachePos,
                           uint32_t nHeads, uint32_t nKV, uint32_t hd, float invSqrt, tc_stream stream) {
    tc::PrefillMirror none;
    memset(&none, 0, sizeof(none));
    const tc::PrefillKvSource src = {2, k8, v8, ks, vs};
    return prefillF16Impl(q, src, out, scratch, scratchBytes, seqLen, cachePos, nHeads, nKV, hd, invSqrt, none, stream);
}

int tc_attn_prefill_f16_kv8(const float *q, const float *kvK, const float *kvV, float *out, void *scratch,
                            size_t scratchBytes, uint32_t seqLen, uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                            uint32_t hd, float invSqrt, int8_t *k8, int8_t *v8, float *ks, float *vs,
                            uint64_t kv8Row, uint64_t kv8MaxRows, tc_stream stream) {
    TC_REQUIRE(k8 && v8 && ks && vs, TC_EINVAL, "tc_attn_prefill_f16_kv8: null pool pointer");
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8)) & 3u) == 0, TC_EINVAL,
               "tc_attn_prefill_f16_kv8: k8/v8 need 4-byte alignment");
    if (kv8Row + seqLen > kv8MaxRows) {
        tc::setError("tc_attn_prefill_f16_kv8: rows [%llu, %llu) pass the pool's %llu rows", (unsigned long long) kv8Row,
                     (unsigned long long) kv8Row + seqLen, (unsigned long long) kv8MaxRows);
        return TC_ECONTEXT_FULL;
    }
    tc::PrefillMirror mir;
    mir.k8 = k8, mir.v8 = v8, mir.ks = ks, mir.vs = vs, mir.dstRow = kv8Row, mir.maxRows = kv8MaxRows;
    const tc::PrefillKvSource src = {0, kvK, kvV, nullptr, nullptr};
    return prefillF16Impl(q, src, out, scratch, scratchBytes, seqLen, cachePos, nHeads, nKV, hd, invSqrt, mir, stream);
}

}  // extern "C"
