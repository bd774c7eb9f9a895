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
// One CTA = one q head x 256 query rows = two 128-row query tiles A and B.  Warp roles:
//   warps 0-3 / 4-7  softmax of tile A / B: thread r owns query row r, reads its 128
//              scores from TMEM in one pass (tcgen05.ld), keeps (m, l), writes the fp16
//              probabilities over the first 64 columns of the same S region (tcgen05.st)
//              as the A operand of the PV product, rescales O in TMEM only when the row
//              maximum ran ahead by 2^8 (lazy rescale);
//   warp 8     TMA producer: both Q tiles once, then K / V tiles of 128 tokens into
//              two-stage rings (cp.async.bulk.tensor, 128-byte swizzle = the canonical UMMA
//              shared-memory layout, so no register pass touches the operands);
//   warp 9     MMA issuer: one thread issues tcgen05.mma -- S_X = Q_X K^T (M128 N128 K16
//              x8), O_X += P_X V (A from TMEM, B = V MN-major from shared memory) -- in the
//              order S_A, S_B, then per KV tile [O_A, S_A(next)], [O_B, S_B(next)], so the
//              tensor pipe works for one tile while the other tile's softmax runs;
//              tcgen05.commit onto mbarriers.
// Causality: a query tile only visits KV tiles up to its own diagonal tile, which is
// masked element-wise; heavy (late) query blocks are scheduled first.
// TMEM: S_A, S_B (128 columns each, f32; P aliases their first 64), O_A, O_B (128 each) = 512.
// Every wait is bounded; a wait that runs out records an error bit, the CTA drains and
// frees its TMEM before it returns.
#include <algorithm>

#include "tc_tcgen05.cuh"

namespace tc {

constexpr int kPfHD = 128;    // head_dim the kernel is built for
constexpr int kPfBM = 128;    // query rows per CTA
constexpr int kPfBN = 128;    // tokens per KV tile
constexpr int kPfStages = 2;  // K and V ring depth
constexpr float kPfLazyLog2 = 8.0f;

// f32 -> fp16 twins (the reference's kF32ToF16, GpuElementwiseKernels.hpp:92-101)
__global__ void __launch_bounds__(256)
f32ToF16Kernel(const float4 *__restrict__ x, uint2 *__restrict__ y, size_t n4) {
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (; i < n4; i += stride) {
        const float4 v = __ldg(x + i);
        uint2 o;
        o.x = packHalf2(v.x, v.y);
        o.y = packHalf2(v.z, v.w);
        y[i] = o;
    }
}

struct PrefillF16Params {
    float *out;        // [seqLen][nHeads][128] f32
    uint32_t seqLen, nHeads, nKV, group;
    uint32_t nQTiles;  // 256-row query blocks
    float scaleLog2;   // invSqrt * log2(e)
    unsigned int *err;
};

struct PrefillF16Smem {
    static constexpr int kTile = kPfBM * kPfHD * 2;          // 32 KB: one 128x128 fp16 tile (two 64-column halves)
    static constexpr int kQ = 0;                             // two query tiles
    static constexpr int kK = 2 * kTile;
    static constexpr int kV = kK + kPfStages * kTile;
    static constexpr int kBars = kV + kPfStages * kTile;
    static constexpr int kNumBars = 1 + 4 * kPfStages + 6;   // qFull, k/v full+empty, sFull[2], pFull[2], pvDone[2]
    static constexpr int kTmemSlot = kBars + kNumBars * 8;
    static constexpr int kTotal = kTmemSlot + 16 + 1024;
};

__device__ __forceinline__ bool pfWait(uint64_t *bar, uint32_t parity, unsigned int *err, uint32_t bit) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbarTryWait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    atomicOr(err, bit);
    return false;
}

// 320 threads: warps 0-3 softmax of query tile A, warps 4-7 softmax of query tile B
// (rows 128 further down), warp 8 TMA producer, warp 9 MMA issuer.
__global__ void __launch_bounds__(320, 1)
prefillF16Kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const PrefillF16Params p) {
    using L = PrefillF16Smem;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kBars);
    uint64_t *qFull = bars, *kFull = bars + 1, *kEmpty = bars + 3, *vFull = bars + 5, *vEmpty = bars + 7,
             *sFull = bars + 9, *pFull = bars + 11, *pvDone = bars + 13;
    uint32_t *tmemSlot = reinterpret_cast<uint32_t *>(smem + L::kTmemSlot);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // heavy query blocks (long causal prefixes) first
    const uint32_t qb = p.nQTiles - 1u - blockIdx.x / p.nHeads;  // 256-row query block
    const uint32_t head = blockIdx.x % p.nHeads;
    const uint32_t kvHead = head / p.group;
    const uint32_t m0 = qb * 2u * kPfBM;
    // query tile X (0 = A, 1 = B) sits on KV tile 2*qb + X; B may lie wholly past the sequence
    const bool activeB = m0 + kPfBM < p.seqLen;
    const uint32_t qtA = 2u * qb, qtB = qtA + 1u;
    const uint32_t nTiles = activeB ? qtB + 1u : qtA + 1u;

    if (threadIdx.x == 0) {
        mbarInit(qFull, 1);
        for (int s = 0; s < 2; ++s) {
            mbarInit(&kFull[s], 1);
            mbarInit(&kEmpty[s], 1);
            mbarInit(&vFull[s], 1);
            mbarInit(&vEmpty[s], 1);
            mbarInit(&sFull[s], 1);
            mbarInit(&pFull[s], 128);
            mbarInit(&pvDone[s], 1);
        }
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
    // S of tile X at columns 128X (its fp16 probabilities overwrite the first 64 of them), O at 256 + 128X

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            mbarExpectTx(qFull, 2 * L::kTile);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                tmaLoad3D(smem + L::kQ + x * L::kTile, &tmQ, qFull, 0, head, m0 + x * kPfBM);
                tmaLoad3D(smem + L::kQ + x * L::kTile + L::kTile / 2, &tmQ, qFull, 64, head, m0 + x * kPfBM);
            }
            for (uint32_t j = 0; j < nTiles; ++j) {
                const uint32_t b = j & 1u;
                if (j >= kPfStages && !pfWait(&kEmpty[b], ((j >> 1) - 1u) & 1u, p.err, kDevErrEmptyWait)) break;
                uint8_t *kd = smem + L::kK + b * L::kTile;
                mbarExpectTx(&kFull[b], L::kTile);
                tmaLoad3D(kd, &tmK, &kFull[b], 0, kvHead, j * kPfBN);
                tmaLoad3D(kd + L::kTile / 2, &tmK, &kFull[b], 64, kvHead, j * kPfBN);
                if (j >= kPfStages && !pfWait(&vEmpty[b], ((j >> 1) - 1u) & 1u, p.err, kDevErrEmptyWait)) break;
                uint8_t *vd = smem + L::kV + b * L::kTile;
                mbarExpectTx(&vFull[b], L::kTile);
                tmaLoad3D(vd, &tmV, &vFull[b], 0, kvHead, j * kPfBN);
                tmaLoad3D(vd + L::kTile / 2, &tmV, &vFull[b], 64, kvHead, j * kPfBN);
            }
        }
    } else if (warp == 9) {
        // ------------------------------- MMA issuer -------------------------------
        // Order: S_A(0), S_B(0), then per KV tile j: [P_A(j)] O_A += P_A V, S_A(j+1); [P_B(j)] O_B += P_B V,
        // S_B(j+1) -- while one tile's softmax runs, the tensor pipe works for the other tile.
        if (lane == 0) {
            constexpr uint32_t idQK = umaInstrDescF16(kPfBM, kPfBN, 0, 0);
            constexpr uint32_t idPV = umaInstrDescF16(kPfBM, kPfHD, 0, 1);
            auto tileOn = [&](uint32_t x, uint32_t j) { return x == 0 ? j <= qtA : (activeB && j <= qtB); };
            auto issueQK = [&](uint32_t x, uint32_t j) {
                const uint32_t qAddr = smemAddr(smem + L::kQ + x * L::kTile);
                const uint32_t kAddr = smemAddr(smem + L::kK + (j & 1u) * L::kTile);
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * (L::kTile / 2) + (ks & 3u) * 32u;
                    umaMmaSS(tmemBase + 128u * x, umaSmemDesc(qAddr + off, 16, 1024), umaSmemDesc(kAddr + off, 16, 1024),
                             idQK, ks > 0 ? 1u : 0u);
                }
                umaCommit(&sFull[x]);
            };
            bool ok = pfWait(qFull, 0, p.err, kDevErrFullWait) && pfWait(&kFull[0], 0, p.err, kDevErrFullWait);
            if (ok) {
                tcFenceAfter();
                issueQK(0, 0);
                if (tileOn(1, 0)) issueQK(1, 0);
                umaCommit(&kEmpty[0]);
            }
            for (uint32_t j = 0; ok && j < nTiles; ++j) {
                const uint32_t b = j & 1u;
                const bool more = j + 1 < nTiles;
                if (!pfWait(&vFull[b], (j >> 1) & 1u, p.err, kDevErrFullWait)) break;
                if (more && !pfWait(&kFull[b ^ 1u], ((j + 1) >> 1) & 1u, p.err, kDevErrFullWait)) break;
                const uint32_t vAddr = smemAddr(smem + L::kV + b * L::kTile);
                for (uint32_t x = 0; x < 2 && ok; ++x) {
                    if (!tileOn(x, j)) continue;
                    if (!pfWait(&pFull[x], j & 1u, p.err, kDevErrMmaWait)) {
                        ok = false;
                        break;
                    }
                    tcFenceAfter();
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks)
                        umaMmaTS(tmemBase + 256u + 128u * x, tmemBase + 128u * x + ks * 8u,
                                 umaSmemDesc(vAddr + ks * 2048u, L::kTile / 2, 1024), idPV, (j > 0 || ks > 0) ? 1u : 0u);
                    umaCommit(&pvDone[x]);
                    if (more && tileOn(x, j + 1)) issueQK(x, j + 1);  // overwrites P_x(j): issued after its PV
                }
                umaCommit(&vEmpty[b]);
                if (more) umaCommit(&kEmpty[b ^ 1u]);
            }
        }
    } else {
        // --------------------------------- softmax ---------------------------------
        const uint32_t x = warp >> 2;                         // which query tile this warpgroup owns
        const uint32_t row = (warp & 3u) * 32u + lane;        // row of that tile = TMEM lane
        const uint32_t laneBase = ((warp & 3u) * 32u) << 16;  // TMEM lane field
        const uint32_t rq = m0 + x * kPfBM + row;             // query position
        const uint32_t qt = x == 0 ? qtA : qtB;               // diagonal KV tile of this query tile
        const uint32_t tS = tmemBase + 128u * x, tO = tmemBase + 256u + 128u * x;
        float m = kNegBig, l = 0.0f;
        bool ok = x == 0 || activeB;
        const uint32_t myTiles = ok ? qt + 1u : 0u;
        for (uint32_t j = 0; j < myTiles; ++j) {
            if (!pfWait(&sFull[x], j & 1u, p.err, kDevErrMmaWait)) {
                ok = false;
                break;
            }
            tcFenceAfter();
            // the whole score row in registers: one TMEM pass per tile
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmemLd32(tS + laneBase + c * 32u, r[c]);
            tmemLdWait();
            if (j == qt) {
                // causal edge: column c of the diagonal tile is visible iff c <= row
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (static_cast<uint32_t>(c * 32 + i) > row) r[c][i] = 0xff800000u;  // -inf
            }
            float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    mxa = fmaxf(mxa, __uint_as_float(r[c][i]));
                    mxb = fmaxf(mxb, __uint_as_float(r[c][i + 1]));
                }
            const float mx = fmaxf(mxa, mxb) * p.scaleLog2;  // scale > 0: max commutes with it
            const float mNew = mx > m + kPfLazyLog2 ? mx : m;
            const float alpha = fastExp2(m - mNew);
            // O is stable once the previous tile's PV has completed
            if (j > 0) {
                if (!pfWait(&pvDone[x], (j - 1u) & 1u, p.err, kDevErrMmaWait)) {
                    ok = false;
                    break;
                }
                tcFenceAfter();
                if (__any_sync(0xffffffffu, mNew != m)) {
#pragma unroll 1
                    for (uint32_t c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tmemLd32(tO + laneBase + c * 32u, o);
                        tmemLdWait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmemSt32(tO + laneBase + c * 32u, o);
                    }
                    tmemStWait();
                }
            }
            m = mNew;
            // probabilities as fp16 pairs, written over the first 64 columns of this tile's S:
            // the A operand of the PV product (every score of the row is already in registers)
            float suma = 0.0f, sumb = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = fastExp2(fmaf(__uint_as_float(r[c][2 * i]), p.scaleLog2, -m));
                    const float p1 = fastExp2(fmaf(__uint_as_float(r[c][2 * i + 1]), p.scaleLog2, -m));
                    suma += p0;
                    sumb += p1;
                    h[i] = packHalf2(p0, p1);
                }
                tmemSt16(tS + laneBase + c * 16u, h);
            }
            l = l * alpha + (suma + sumb);
            tmemStWait();
            tcFenceBefore();
            mbarArrive(&pFull[x]);
        }
        if (ok && myTiles && pfWait(&pvDone[x], (myTiles - 1u) & 1u, p.err, kDevErrMmaWait)) {
            tcFenceAfter();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float *orow = p.out + (static_cast<size_t>(rq) * p.nHeads + head) * kPfHD;
#pragma unroll 1
            for (uint32_t c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmemLd32(tO + laneBase + c * 32u, o);
                tmemLdWait();
                if (rq < p.seqLen) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4 *>(orow + c * 32 + 4 * i) =
                                make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                            __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
                }
            }
        }
    }
    tcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        tcFenceAfter();
        tmemDealloc(tmemBase, 512);
    }
}

static int f16Map(const void *base, uint32_t heads, uint32_t rows, CUtensorMap *out) {
    TensorMapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.rank = 3;
    key.elemBytes = 2;
    key.swizzle = 3;
    key.dims[0] = kPfHD;
    key.dims[1] = heads;
    key.dims[2] = rows;
    key.strides[0] = kPfHD * 2;
    key.strides[1] = static_cast<uint64_t>(heads) * kPfHD * 2;
    key.box[0] = 64;  // 128 bytes: one swizzle span
    key.box[1] = 1;
    key.box[2] = kPfBM;
    return getTensorMap(key, out);
}

static size_t prefillScratchBytes(uint32_t seqLen, uint32_t nHeads, uint32_t nKV) {
    // fp16 twins: q [seqLen][nHeads][128], k and v [seqLen][nKV][128]; each region 1 KB aligned
    auto al = [](size_t x) { return (x + 1023) & ~size_t(1023); };
    return al(static_cast<size_t>(seqLen) * nHeads * kPfHD * 2) + 2 * al(static_cast<size_t>(seqLen) * nKV * kPfHD * 2);
}

}  // namespace tc

extern "C" {

int tc_attn_prefill_f16_scratch_bytes(uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd, size_t *bytes) {
    TC_REQUIRE(bytes != nullptr, TC_EINVAL, "tc_attn_prefill_f16_scratch_bytes: null output");
    TC_REQUIRE(hd == tc::kPfHD, TC_EUNSUPPORTED, "tc_attn_prefill_f16: head_dim %u (built for 128)", hd);
    *bytes = tc::prefillScratchBytes(seqLen, nHeads, nKV);
    return TC_OK;
}

int tc_attn_prefill_f16(const float *q, const float *kvK, const float *kvV, float *out, void *scratch,
                        size_t scratchBytes, uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd,
                        float invSqrt, tc_stream stream) {
    using namespace tc;
    TC_REQUIRE(q && kvK && kvV && out && scratch, TC_EINVAL, "tc_attn_prefill_f16: null pointer");
    TC_REQUIRE(hd == kPfHD, TC_EUNSUPPORTED, "tc_attn_prefill_f16: head_dim %u (built for 128)", hd);
    TC_REQUIRE(nKV > 0 && nHeads % nKV == 0, TC_EINVAL, "tc_attn_prefill_f16: nHeads %u not a multiple of nKV %u",
               nHeads, nKV);
    TC_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kvK) | reinterpret_cast<uintptr_t>(kvV) |
                 reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15u) == 0,
               TC_EINVAL, "tc_attn_prefill_f16: pointers need 16-byte alignment");
    if (seqLen == 0) return TC_OK;
    TC_REQUIRE(scratchBytes >= prefillScratchBytes(seqLen, nHeads, nKV), TC_EWORKSPACE,
               "tc_attn_prefill_f16: scratch of %zu bytes, %zu needed", scratchBytes,
               prefillScratchBytes(seqLen, nHeads, nKV));
    TC_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 1023u) == 0, TC_EINVAL,
               "tc_attn_prefill_f16: scratch needs 1024-byte alignment");
    const uint32_t nQTiles = (seqLen + 2 * kPfBM - 1) / (2 * kPfBM);  // 256-row query blocks
    TC_REQUIRE(static_cast<uint64_t>(nQTiles) * nHeads < (1ull << 31), TC_EUNSUPPORTED,
               "tc_attn_prefill_f16: grid too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto al = [](size_t x) { return (x + 1023) & ~size_t(1023); };
    const size_t qElems = static_cast<size_t>(seqLen) * nHeads * kPfHD;
    const size_t kvElems = static_cast<size_t>(seqLen) * nKV * kPfHD;
    uint8_t *sc = static_cast<uint8_t *>(scratch);
    void *q16 = sc, *k16 = sc + al(qElems * 2), *v16 = sc + al(qElems * 2) + al(kvElems * 2);
    const int sms = numSMs();
    auto conv = [&](const float *src, void *dst, size_t n) {
        const size_t n4 = n / 4;
        const uint32_t blocks = static_cast<uint32_t>(std::min<size_t>((n4 + 255) / 256, static_cast<size_t>(sms) * 8));
        f32ToF16Kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float4 *>(src), static_cast<uint2 *>(dst), n4);
    };
    conv(q, q16, qElems);
    conv(kvK, k16, kvElems);
    conv(kvV, v16, kvElems);
    TC_CUDA_OK(cudaGetLastError());
    CUtensorMap tmQ, tmK, tmV;
    int rc = f16Map(q16, nHeads, seqLen, &tmQ);
    if (rc != TC_OK) return rc;
    rc = f16Map(k16, nKV, seqLen, &tmK);
    if (rc != TC_OK) return rc;
    rc = f16Map(v16, nKV, seqLen, &tmV);
    if (rc != TC_OK) return rc;
    PrefillF16Params prm;
    prm.out = out;
    prm.seqLen = seqLen;
    prm.nHeads = nHeads;
    prm.nKV = nKV;
    prm.group = nHeads / nKV;
    prm.nQTiles = nQTiles;
    prm.scaleLog2 = invSqrt * kLog2e;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "tc_attn_prefill_f16: no device error word");
    static bool attrDone[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attrDone[dev]) {
        TC_CUDA_OK(cudaFuncSetAttribute(prefillF16Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        PrefillF16Smem::kTotal));
        attrDone[dev] = true;
    }
    prefillF16Kernel<<<nQTiles * nHeads, 320, PrefillF16Smem::kTotal, st>>>(tmQ, tmK, tmV, prm);
    TC_CUDA_OK(cudaGetLastError());
    return TC_OK;
}

}  // extern "C"
