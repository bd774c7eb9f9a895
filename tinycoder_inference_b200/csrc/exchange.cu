// exchange.cu -- the merge of a context-axis split across GPUs, with the exchange inside
// the kernel.
//
// New capability (the reference engine is single-device).  Every rank has run the split-KV
// decode kernel over ITS row range of one sequence and holds chunk partials (m, l, acc) per
// q head.  One launch per rank then does, for q head h (one block each):
//   1. merge the rank's own chunks into ONE partial (M, L, A[hd]) -- the rule of merge.cu,
//      left unnormalised;
//   2. store that partial into the exchange buffer of every rank (peer stores over NVLink,
//      about 1 KB per head and peer).  Every 16-byte store carries two 64-bit words, each a
//      float with the step number in its upper half, so the data is its own arrival flag
//      (a 64-bit word is written and read as one piece): no fence and no separate
//      flag store sit between a rank's arithmetic and its peers (system-scope fences and
//      release/acquire pairs cost several microseconds each here, more than the merge);
//   3. poll (bounded) this rank's own buffer until every 16-byte unit of every source rank
//      shows this step, then merge the `world` partials and write out[h].
// No collective library call, no second launch, nothing staged through the host: the data
// crosses NVLink once, as plain peer stores.
//
// Steps are told apart by an epoch per head that lives in the rank's own buffer and is
// advanced by the block that used it, so a captured graph can replay the launch unchanged.
// Partials are double-buffered by epoch parity: a rank can only be one step ahead of a peer
// (its step e+1 needs the peer's partial of step e+1, which the peer sends after it has
// finished reading step e).
//
// The same kernel can carry several ranks in one (cooperative) launch on one GPU -- the
// single-GPU tests run the full protocol that way; blocks that wait for one another must be
// co-resident, which a cooperative launch guarantees.
#include "decode_shared.cuh"

namespace tc {

constexpr uint32_t kMaxRanks = 16;
constexpr uint32_t kMaxViews = 8;
constexpr uint32_t kExMaxChunks = 1024;

// Layout of one rank's exchange buffer (uint32 / float words):
//   epoch[nHeads]                           this rank's step counter per head
//   data[2][kMaxRanks][nHeads][units][4]    per parity, source rank and head: 16-byte units
//                                           {value 2u, step, value 2u+1, step} over the
//                                           hd + 2 values A[0..hd), M, L
struct ExLayout {
    uint32_t nHeads, hd;
    __host__ __device__ size_t epochOff() const { return 0; }
    __host__ __device__ uint32_t units() const { return (hd + 2 + 1) / 2; }
    __host__ __device__ size_t dataOff(uint32_t par, uint32_t src, uint32_t h) const {
        const size_t start = (static_cast<size_t>(nHeads) + 3) & ~static_cast<size_t>(3);  // 16-byte aligned
        return start + ((static_cast<size_t>(par) * kMaxRanks + src) * nHeads + h) * units() * 4;
    }
    __host__ __device__ size_t totalWords() const { return dataOff(2, 0, 0); }
};

struct ExView {  // one rank
    const float *pAcc, *pM, *pL;
    float *out;
    float *peers[kMaxRanks];  // exchange buffers of all ranks, as seen from this rank
    uint32_t rank;
};

struct ExParams {
    ExView v[kMaxViews];
    uint32_t world, nHeads, numChunks, active, hd;
    unsigned int *err;
};

// A unit is two 64-bit words, each {value (low half), step (high half)}.  Loads and stores move a
// unit as a vector of two 64-bit ELEMENTS: the memory model treats a vector access as separate
// accesses of its elements, and an aligned 64-bit scalar element is single-copy atomic -- a value
// can therefore never be seen with another step's tag, which a vector of four 32-bit elements
// (the same bytes) would not promise.
__device__ __forceinline__ uint4 ldVolatileV4(const void *p) {
    unsigned long long a, b;
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4(static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32), static_cast<uint32_t>(b),
                      static_cast<uint32_t>(b >> 32));
}
__device__ __forceinline__ void stVolatileV4(void *p, uint4 v) {
    const unsigned long long a = (static_cast<unsigned long long>(v.y) << 32) | v.x;
    const unsigned long long b = (static_cast<unsigned long long>(v.w) << 32) | v.z;
    asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

template <int NV4>
__global__ void __launch_bounds__(256)
mergeExchangeKernel(const ExParams p) {
    constexpr int NW = 8;
    const uint32_t head = blockIdx.x;
    const ExView &me = p.v[blockIdx.y];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const ExLayout lay{p.nHeads, p.hd};
    const uint32_t nvec = p.hd >> 2;
    gridDepLaunch();
    gridDepWait();

    __shared__ float sw[kExMaxChunks], sl[kExMaxChunks];
    __shared__ float sred[NW];
    __shared__ float4 sacc[NW][NV4][32];
    __shared__ uint32_t sOk;

    // ---- 1. this rank's chunks -> one unnormalised partial ----
    // As in merge.cu the accumulator rows are requested before anything is consumed (their
    // addresses do not depend on the weights): the kernel is a chain of latencies, and a load
    // per loop iteration would pay one L2 round trip per chunk.
    const uint32_t active = p.active < p.numChunks ? p.active : p.numChunks;
    const uint64_t base = static_cast<uint64_t>(head) * p.numChunks;
    constexpr int kBatch = 16;
    float4 a[kBatch][NV4];
    auto loadBatch = [&](uint32_t c0) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const uint32_t c = c0 + u * NW;
            const uint32_t cc = c < active ? c : (active ? active - 1 : 0);  // always a valid address
            const float4 *pa = reinterpret_cast<const float4 *>(me.pAcc + (base + cc) * p.hd);
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const uint32_t i = lane + 32u * j;
                a[u][j] = pa[i < nvec ? i : 0];
            }
        }
    };
    if (active) loadBatch(warp);
    float M = kNegBig;
    for (uint32_t c = threadIdx.x; c < active; c += 256) {
        const float m = me.pM[base + c];
        const float lc = me.pL[base + c];
        sw[c] = m;
        sl[c] = lc;
        if (lc > 0.0f) M = fmaxf(M, m);
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
    __syncthreads();
    lsum = 0.0f;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) lsum += sred[w2];
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
                // an empty chunk's row may never have been written: select, never multiply
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
    if (warp == 0) {
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
            sacc[0][j][lane] = r;
        }
    }
    __syncthreads();

    // ---- 2. send it to every rank ----
    // the hd + 2 values as one array in shared memory: A (already there), then M and L
    float *vals = reinterpret_cast<float *>(&sacc[0][0][0]);  // [NV4 * 128] floats, hd of them used
    __shared__ float sML[2];
    __shared__ float spart[kMaxRanks][256 + 2];
    if (threadIdx.x == 0) {
        sML[0] = M;
        sML[1] = lsum;
        sOk = 1;
    }
    __syncthreads();
    unsigned int *myWords = reinterpret_cast<unsigned int *>(me.peers[me.rank]);
    const uint32_t epoch = myWords[lay.epochOff() + head];  // only this block ever touches it
    const uint32_t step = epoch + 1, par = epoch & 1u;
    const uint32_t units = lay.units(), nvals = p.hd + 2;
    auto value = [&](uint32_t i) -> uint32_t {
        return __float_as_uint(i < p.hd ? vals[i] : (i < nvals ? sML[i - p.hd] : 0.0f));
    };
    for (uint32_t r = warp; r < p.world; r += NW) {
        uint4 *dst = reinterpret_cast<uint4 *>(me.peers[r] + lay.dataOff(par, me.rank, head));
        for (uint32_t u = lane; u < units; u += 32) stVolatileV4(dst + u, make_uint4(value(2 * u), step, value(2 * u + 1), step));
    }

    // ---- 3. take in every rank's partial of this step as it lands, merge them ----
    for (uint32_t r = warp; r < p.world; r += NW) {
        const uint4 *src = reinterpret_cast<const uint4 *>(me.peers[me.rank] + lay.dataOff(par, r, head));
        const long long t0 = clock64();
        for (uint32_t u = lane; u < units; u += 32) {
            uint4 v = ldVolatileV4(src + u);
            while (v.y != step || v.w != step) {
                if (clock64() - t0 > (1ll << 31)) {  // about a second: give up, say so, keep the context alive
                    atomicOr(p.err, kDevErrMergeWait);
                    sOk = 0;
                    break;
                }
                v = ldVolatileV4(src + u);
            }
            spart[r][2 * u] = __uint_as_float(v.x);
            if (2 * u + 1 < 258) spart[r][2 * u + 1] = __uint_as_float(v.z);
        }
    }
    __syncthreads();
    if (warp == 0 && sOk) {
        float Mx = kNegBig;
        for (uint32_t r = 0; r < p.world; ++r)
            if (spart[r][p.hd + 1] > 0.0f) Mx = fmaxf(Mx, spart[r][p.hd]);
        float L = 0.0f;
        float4 o[NV4];
#pragma unroll
        for (int j = 0; j < NV4; ++j) o[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < p.world; ++r) {
            const float lr = spart[r][p.hd + 1];
            if (!(lr > 0.0f)) continue;
            const float w = exp2f((spart[r][p.hd] - Mx) * kLog2e);
            L = fmaf(w, lr, L);
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const uint32_t i = lane + 32u * j;
                if (i < nvec) {
                    const float *v = &spart[r][4 * i];
                    o[j].x = fmaf(w, v[0], o[j].x);
                    o[j].y = fmaf(w, v[1], o[j].y);
                    o[j].z = fmaf(w, v[2], o[j].z);
                    o[j].w = fmaf(w, v[3], o[j].w);
                }
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        float4 *op = reinterpret_cast<float4 *>(me.out + static_cast<uint64_t>(head) * p.hd);
#pragma unroll
        for (int j = 0; j < NV4; ++j) {
            const uint32_t i = lane + 32u * j;
            if (i < nvec) op[i] = make_float4(o[j].x * inv, o[j].y * inv, o[j].z * inv, o[j].w * inv);
        }
    }
    if (threadIdx.x == 0) myWords[lay.epochOff() + head] = step;
}

static int checkShape(const char *who, uint32_t nHeads, uint32_t hd, uint32_t world) {
    TC_REQUIRE(hd >= 32 && hd <= 256 && (hd % 32u) == 0, TC_EUNSUPPORTED, "%s: hd=%u", who, hd);
    TC_REQUIRE(nHeads >= 1 && nHeads <= 65535, TC_EINVAL, "%s: %u heads", who, nHeads);
    TC_REQUIRE(world >= 1 && world <= kMaxRanks, TC_EUNSUPPORTED, "%s: %u ranks (max %u)", who, world, kMaxRanks);
    return TC_OK;
}

static int launchExchange(const ExParams &prm, uint32_t views, bool cooperative, bool pdl, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(prm.nHeads, views);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cooperative) {
        attr[n].id = cudaLaunchAttributeCooperative;
        attr[n].val.cooperative = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    if (prm.hd <= 128) TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergeExchangeKernel<1>, prm));
    else TC_CUDA_OK(cudaLaunchKernelEx(&cfg, mergeExchangeKernel<2>, prm));
    return TC_OK;
}

}  // namespace tc

extern "C" {

int tc_attn_exchange_bytes(uint32_t nHeads, uint32_t hd, uint32_t world, size_t *bytes) {
    TC_REQUIRE(bytes != nullptr, TC_EINVAL, "tc_attn_exchange_bytes: null output");
    const int rc = tc::checkShape("tc_attn_exchange_bytes", nHeads, hd, world);
    if (rc != TC_OK) return rc;
    *bytes = tc::ExLayout{nHeads, hd}.totalWords() * 4;
    return TC_OK;
}

int tc_attn_merge_exchange(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t nHeads,
                           uint32_t numChunks, uint32_t activeChunks, uint32_t hd, const tc_peer_group *g,
                           uint32_t flags, tc_stream stream) {
    using namespace tc;
    TC_REQUIRE(pAcc && pM && pL && out && g, TC_EINVAL, "tc_attn_merge_exchange: null pointer");
    int rc = checkShape("tc_attn_merge_exchange", nHeads, hd, g->world);
    if (rc != TC_OK) return rc;
    TC_REQUIRE(g->rank < g->world, TC_EINVAL, "tc_attn_merge_exchange: rank %u of %u", g->rank, g->world);
    TC_REQUIRE(numChunks >= 1 && activeChunks <= kExMaxChunks, TC_EUNSUPPORTED,
               "tc_attn_merge_exchange: %u active chunks (max %u)", activeChunks, kExMaxChunks);
    ExParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.v[0].pAcc = pAcc;
    prm.v[0].pM = pM;
    prm.v[0].pL = pL;
    prm.v[0].out = out;
    prm.v[0].rank = g->rank;
    for (uint32_t r = 0; r < g->world; ++r) {
        TC_REQUIRE(g->buffers[r] != nullptr && (reinterpret_cast<uintptr_t>(g->buffers[r]) & 15u) == 0, TC_EINVAL,
                   "tc_attn_merge_exchange: buffer of rank %u is null or not 16-byte aligned", r);
        prm.v[0].peers[r] = static_cast<float *>(g->buffers[r]);
    }
    prm.world = g->world;
    prm.nHeads = nHeads;
    prm.numChunks = numChunks;
    prm.active = activeChunks;
    prm.hd = hd;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "tc_attn_merge_exchange: no device error word");
    return launchExchange(prm, 1, false, (flags & TC_DECODE_PDL) != 0, static_cast<cudaStream_t>(stream));
}

int tc_attn_merge_exchange_local(const float *const *pAcc, const float *const *pM, const float *const *pL,
                                 float *const *out, void *const *buffers, uint32_t ranks, uint32_t nHeads,
                                 uint32_t numChunks, uint32_t activeChunks, uint32_t hd, tc_stream stream) {
    using namespace tc;
    TC_REQUIRE(pAcc && pM && pL && out && buffers, TC_EINVAL, "tc_attn_merge_exchange_local: null pointer");
    int rc = checkShape("tc_attn_merge_exchange_local", nHeads, hd, ranks);
    if (rc != TC_OK) return rc;
    TC_REQUIRE(ranks <= kMaxViews, TC_EUNSUPPORTED, "tc_attn_merge_exchange_local: %u ranks in one launch (max %u)",
               ranks, kMaxViews);
    TC_REQUIRE(numChunks >= 1 && activeChunks <= kExMaxChunks, TC_EUNSUPPORTED,
               "tc_attn_merge_exchange_local: %u active chunks", activeChunks);
    // every block must be resident: the cooperative launch refuses a grid that is not
    ExParams prm;
    memset(&prm, 0, sizeof(prm));
    for (uint32_t v = 0; v < ranks; ++v) {
        TC_REQUIRE(pAcc[v] && pM[v] && pL[v] && out[v] && buffers[v], TC_EINVAL,
                   "tc_attn_merge_exchange_local: null pointer for rank %u", v);
        prm.v[v].pAcc = pAcc[v];
        prm.v[v].pM = pM[v];
        prm.v[v].pL = pL[v];
        prm.v[v].out = out[v];
        prm.v[v].rank = v;
        for (uint32_t r = 0; r < ranks; ++r) prm.v[v].peers[r] = static_cast<float *>(buffers[r]);
    }
    prm.world = ranks;
    prm.nHeads = nHeads;
    prm.numChunks = numChunks;
    prm.active = activeChunks;
    prm.hd = hd;
    prm.err = devErrorWord();
    TC_REQUIRE(prm.err != nullptr, TC_ECUDA, "tc_attn_merge_exchange_local: no device error word");
    return launchExchange(prm, ranks, true, false, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
