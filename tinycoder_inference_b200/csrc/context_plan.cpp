// context_plan.cpp -- window / KV-precision planner and KV pool geometry (host only).
//
// Same decision as the reference's planContext (src/cpp/core/ContextPlan.cpp:
// 80-246): the budget is free VRAM minus a fixed session overhead and a 256 MiB
// margin (or free RAM minus 2 GiB without a GPU), minus the weights; the ladder
// f32 store + int8 decode mirror -> f32 store -> int8 store is walked in that
// order and the first rung that holds the request wins, otherwise the rung with
// the largest fit; fits are floored to 256 tokens, capped at the model's limit
// (4096 when unknown); auto asks for 2048; below 1024 tokens nothing is granted.
// The byte accounting (kvStoreBytesPerToken / kvBytesPerToken, :58-78) is exact
// integer arithmetic and must reproduce the reference's known answers.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cmath>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/tc_attn.h"

namespace {

constexpr uint64_t kMiB = 1024ull * 1024ull;
constexpr uint64_t kSafetyMargin = 256ull * kMiB;   // ContextPlan.cpp:24
constexpr uint64_t kRamSlack = 2048ull * kMiB;      // ContextPlan.cpp:38
constexpr uint32_t kFloorSeqLen = 1024;             // ContextPlan.cpp:27
constexpr uint32_t kAutoSeqLen = 2048;              // ContextPlan.cpp:31
constexpr uint32_t kFallbackModelMax = 4096;        // ContextPlan.cpp:34
constexpr uint64_t kDefaultOverhead = 1408ull * kMiB;  // include/ContextPlan.hpp:58

uint64_t minus(uint64_t a, uint64_t b) { return a > b ? a - b : 0; }

struct Rung {
    uint32_t kv;
    bool mirror;
    uint32_t fit;
};

const char *kvName(const Rung &r) { return r.kv == TC_KV_I8 ? "int8 K/V" : "f32 K/V"; }

}  // namespace

extern "C" {

void tc_context_request_init(tc_context_request *r) {
    if (!r) return;
    std::memset(r, 0, sizeof(*r));
    r->gpuFixedOverhead = kDefaultOverhead;
}

uint64_t tc_kv_store_bytes_per_token(const tc_context_request *r, uint32_t kv, uint32_t mirror) {
    const uint64_t heads = r->numKVHeads, hd = r->headDim;
    const bool i8 = kv == TC_KV_I8;
    uint64_t bytes = 2ull * heads * hd * (i8 ? 1ull : 4ull);        // K and V
    if (i8) bytes += 2ull * heads * 4ull;                            // one f32 scale per (token, head)
    if (!i8 && mirror) bytes += 2ull * heads * (hd + 4ull);          // int8 decode mirror + its scales
    return bytes;
}

uint64_t tc_kv_bytes_per_token(const tc_context_request *r, uint32_t kv, uint32_t mirror) {
    // cos + sin rows are charged once for the whole model, not per layer
    return static_cast<uint64_t>(r->numAttentionLayers) * tc_kv_store_bytes_per_token(r, kv, mirror) +
           4ull * static_cast<uint64_t>(r->ropeDims);
}

int tc_context_plan_compute(const tc_context_request *r, tc_context_plan *plan) {
    if (!r || !plan) return TC_EINVAL;
    std::memset(plan, 0, sizeof(*plan));
    const uint32_t ceiling = r->modelMax ? r->modelMax : kFallbackModelMax;
    const bool gpu = r->freeVram != 0;
    const uint64_t base = gpu ? minus(minus(r->freeVram, r->gpuFixedOverhead), kSafetyMargin)
                              : minus(r->availableRam, kRamSlack);
    const uint64_t budget = minus(base, gpu ? r->weightBytes : 0);

    // ladder, in preference order
    Rung rungs[3];
    int n = 0;
    auto push = [&](uint32_t kv, bool mirror) {
        if (r->forceKvSet && kv != r->forceKv) return;
        const uint64_t per = tc_kv_bytes_per_token(r, kv, mirror ? 1u : 0u);
        uint64_t fit = ceiling;
        if (per != 0) {
            fit = (budget / per) / 256ull * 256ull;
            if (fit > ceiling) fit = ceiling;
        }
        rungs[n++] = Rung{kv, mirror, static_cast<uint32_t>(fit)};
    };
    if (gpu) {
        if (r->int8KvSupported) push(TC_KV_F32, true);
        push(TC_KV_F32, false);
        if (r->int8KvSupported) push(TC_KV_I8, false);
    } else {
        push(TC_KV_F32, false);  // the host cache is f32 only
    }
    uint32_t best = 0;
    for (int i = 0; i < n; ++i) best = rungs[i].fit > best ? rungs[i].fit : best;

    const bool clamped = r->requested > ceiling;
    const uint32_t want = r->requested ? (r->requested < ceiling ? r->requested : ceiling)
                                       : (kAutoSeqLen < best ? kAutoSeqLen : best);
    std::string why;
    plan->kvOnGpu = gpu ? 1u : 0u;
    if (want < kFloorSeqLen || best < kFloorSeqLen) {
        if (r->requested != 0 && r->requested < kFloorSeqLen)
            why = "requested " + std::to_string(r->requested) + ", below the " + std::to_string(kFloorSeqLen) +
                  "-token floor";
        else
            why = "not even " + std::to_string(kFloorSeqLen) + " tokens fit";
        if (!gpu) why += "; no GPU, RAM path";
        if (!r->modelMax) why += "; model max unknown, assuming 4096";
        if (r->forceKvSet && !gpu)
            why += r->forceKv == TC_KV_I8 ? "; an int8 K/V store needs the GPU" : "; f32 K/V pinned by the caller";
        std::snprintf(plan->reason, sizeof(plan->reason), "%s", why.c_str());
        return TC_OK;
    }
    const Rung *chosen = nullptr, *widest = nullptr;
    for (int i = 0; i < n && !chosen; ++i)
        if (rungs[i].fit >= want) chosen = &rungs[i];
    for (int i = 0; i < n && !widest; ++i)
        if (rungs[i].fit == best) widest = &rungs[i];
    const bool reduced = chosen == nullptr;
    if (reduced) chosen = widest;

    plan->kv = chosen->kv;
    plan->kvMirror = chosen->mirror ? 1u : 0u;
    plan->seqLen = want < chosen->fit ? want : chosen->fit;
    plan->maxAllowed = best;  // the ladder's best, whatever rung serves this request
    plan->reduced = reduced ? 1u : 0u;
    plan->kvBytes = static_cast<uint64_t>(plan->seqLen) * tc_kv_bytes_per_token(r, plan->kv, plan->kvMirror);

    if (r->requested) {
        why = "requested " + std::to_string(r->requested);
        if (clamped) why += ", clamped to model max " + std::to_string(ceiling);
    } else {
        why = "auto";
        if (best > plan->seqLen)
            why += "; memory allows up to " + std::to_string(best) + " at " + kvName(*widest) +
                   (widest->mirror ? " + mirror" : "");
    }
    if (reduced)
        why += std::string(", limited by ") + (gpu ? "VRAM" : "RAM") + ": " + std::to_string(chosen->fit) +
               " tokens fit";
    if (!gpu) why += "; no GPU, RAM path";
    if (!r->modelMax) why += "; model max unknown, assuming 4096";
    std::snprintf(plan->reason, sizeof(plan->reason), "%s", why.c_str());
    return TC_OK;
}

int tc_context_plan_compute_sharded(const tc_context_request *r, uint32_t headParts, uint32_t ctxParts,
                                    tc_context_shard_plan *out) {
    if (!r || !out || headParts == 0 || ctxParts == 0) return TC_EINVAL;
    std::memset(out, 0, sizeof(*out));
    out->headParts = headParts;
    out->ctxParts = ctxParts;
    // one GPU's view: its share of the kv heads, and -- for an explicit request -- its share of the rows
    tc_context_request g = *r;
    g.numKVHeads = (r->numKVHeads + headParts - 1) / headParts;
    out->kvHeadsPerGpu = g.numKVHeads;
    auto share = [&](uint32_t rows) -> uint32_t {
        const uint64_t per = (static_cast<uint64_t>(rows) + ctxParts - 1) / ctxParts;
        return static_cast<uint32_t>((per + 255ull) / 256ull * 256ull);
    };
    const bool split = ctxParts > 1 && r->requested != 0;   // an auto window (2048 rows) is not worth a context split
    if (split) {
        g.requested = share(r->requested);
        if (r->modelMax) g.modelMax = share(r->modelMax);
    }
    const int rc = tc_context_plan_compute(&g, &out->plan);
    if (rc != TC_OK) return rc;
    tc_context_plan &p = out->plan;
    const uint64_t ceiling = r->modelMax ? r->modelMax : 4096u;
    if (split) {
        // back to whole-window rows; a GPU's rows stay what the ladder granted it
        out->rowsPerGpu = p.seqLen;
        uint64_t whole = static_cast<uint64_t>(p.seqLen) * ctxParts;
        const uint64_t want = r->requested < ceiling ? r->requested : ceiling;
        if (whole > want) whole = want;
        p.seqLen = static_cast<uint32_t>(whole);
        uint64_t mx = static_cast<uint64_t>(p.maxAllowed) * ctxParts;
        p.maxAllowed = static_cast<uint32_t>(mx < ceiling ? mx : ceiling);
    } else {
        out->rowsPerGpu = (p.seqLen + 255u) / 256u * 256u;
        if (ctxParts > 1) {
            uint64_t mx = static_cast<uint64_t>(p.maxAllowed) * ctxParts;
            p.maxAllowed = static_cast<uint32_t>(mx < ceiling ? mx : ceiling);
        }
    }
    return TC_OK;
}

uint64_t tc_context_overhead_bytes(uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t window, uint32_t headParts,
                                   uint32_t ctxParts, int kvStoreI8, uint32_t prefillChunk, uint64_t runtimeReserve) {
    if (headParts == 0 || ctxParts == 0 || nKV == 0) return runtimeReserve;
    const uint64_t kvLocal = (nKV + headParts - 1) / headParts;
    const uint64_t qLocal = kvLocal * (nHeads / nKV);
    const uint64_t rows = ((static_cast<uint64_t>(window) + ctxParts - 1) / ctxParts + 255ull) / 256ull * 256ull;
    uint64_t total = runtimeReserve;
    total += qLocal * 512ull * (hd + 2ull) * 4ull;                       // split-KV partials: acc, m, l at 512 chunk slots
    if (ctxParts > 1) {
        size_t ex = 0;
        if (tc_attn_exchange_bytes(static_cast<uint32_t>(qLocal), hd, ctxParts, &ex) == TC_OK) total += ex;
        total += qLocal * 64ull * (hd + 2ull) * 4ull;                    // the context split's own 64-slot partial block
    }
    if (!kvStoreI8 && prefillChunk != 0 && (hd == 64 || hd == 128 || hd == 256)) {
        size_t tw = 0;                                                   // fp16 twins: q of a chunk, K/V of the GPU's rows
        const uint32_t chunk = prefillChunk < rows ? prefillChunk : static_cast<uint32_t>(rows);
        if (tc_attn_prefill_f16_scratch_bytes(chunk, static_cast<uint32_t>(rows) - chunk, static_cast<uint32_t>(qLocal),
                                              static_cast<uint32_t>(kvLocal), hd, &tw) == TC_OK)
            total += tw;
    }
    return total;
}

uint64_t tc_probe_free_vram_bytes(void) {
    size_t f = 0, t = 0;
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) {
        (void) cudaGetLastError();
        return 0;
    }
    return static_cast<uint64_t>(f);
}

uint64_t tc_probe_total_vram_bytes(void) {
    size_t f = 0, t = 0;
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) {
        (void) cudaGetLastError();
        return 0;
    }
    return static_cast<uint64_t>(t);
}

int tc_split_geometry(uint32_t maxSeqLen, uint32_t nHeads, uint32_t hd, uint32_t *chunkSize,
                      uint32_t *numChunks) {
    if (!chunkSize || !numChunks) return TC_EINVAL;
    // default 16 (32 for the 12-head x 128 shape), raised so that at most 512
    // chunks cover the window (GPUComputeUpload.cu:318-334)
    uint32_t c = (nHeads == 12 && hd == 128) ? 32u : 16u;
    const uint32_t floorChunk = ((maxSeqLen + 511u) / 512u + 31u) / 32u * 32u;
    if (floorChunk > c) c = floorChunk;
    uint32_t n = (maxSeqLen + c - 1) / c;
    if (n == 0) n = 1;
    *chunkSize = c;
    *numChunks = n;
    return n <= 512u ? TC_OK : TC_EUNSUPPORTED;
}

int tc_kv_pool_geometry_compute(uint32_t maxSeqLen, uint32_t nLayersOnGpu, uint32_t fullAttentionInterval,
                                uint32_t nHeads, uint32_t nKV, uint32_t hd, int kvHalf, int kvStoreI8,
                                int kvMirror, tc_kv_pool_geometry *g) {
    if (!g || nKV == 0 || hd == 0) return TC_EINVAL;
    std::memset(g, 0, sizeof(*g));
    const uint64_t elem = kvHalf ? 2ull : 4ull;
    g->kvLayerStride = static_cast<uint64_t>(maxSeqLen) * nKV * hd * elem;
    // hybrid models keep K/V only on every interval-th layer (GPUComputeUpload.cu:1262-1273)
    g->kvSlots = nLayersOnGpu;
    if (fullAttentionInterval > 1u) g->kvSlots = (nLayersOnGpu + fullAttentionInterval - 1u) / fullAttentionInterval;
    g->kvAllocBytes = kvStoreI8 ? 0ull : static_cast<uint64_t>(g->kvSlots) * g->kvLayerStride;
    if (kvStoreI8 || kvMirror) {
        // 16 spare rows: a decode token may land at index maxSeq when the prompt
        // already fills the window (GPUComputeUpload.cu:1304-1308)
        const uint64_t cap = static_cast<uint64_t>(maxSeqLen) + 16ull;
        g->kv8LayerStride = cap * nKV * hd;
        g->kv8ScaleStride = cap * nKV * sizeof(float);
        g->kv8AllocBytes = static_cast<uint64_t>(g->kvSlots) * g->kv8LayerStride;
        g->kv8ScaleAllocBytes = static_cast<uint64_t>(g->kvSlots) * g->kv8ScaleStride;
    }
    const int rc = tc_split_geometry(maxSeqLen, nHeads, hd, &g->attnChunk, &g->attnChunks);
    // partials are sized for ONE token (GPUComputeUpload.cu:346-365)
    g->partialAccBytes = static_cast<uint64_t>(nHeads) * g->attnChunks * hd * sizeof(float);
    g->partialMLBytes = static_cast<uint64_t>(nHeads) * g->attnChunks * sizeof(float);
    return rc;
}

// Rotation tables (host).  Plain float arithmetic in the reference's order, so the tables are
// the ones the engine uploads (GPUComputeUpload.cu:1149-1163 and 1178-1203).
int tc_rope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t headDim, float theta) {
    if (!cosT || !sinT || headDim < 2 || (headDim % 2u) != 0) return TC_EINVAL;
    const uint32_t pairs = headDim / 2;
    std::vector<float> freq(pairs);
    for (uint32_t j = 0; j < pairs; ++j)
        freq[j] = 1.0f / std::pow(theta, static_cast<float>(2 * j) / static_cast<float>(headDim));
    for (uint32_t p = 0; p < rows; ++p)
        for (uint32_t j = 0; j < pairs; ++j) {
            const float ang = static_cast<float>(p) * freq[j];
            cosT[static_cast<size_t>(p) * pairs + j] = std::cos(ang);
            sinT[static_cast<size_t>(p) * pairs + j] = std::sin(ang);
        }
    return TC_OK;
}

int tc_mrope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t nDims, float thetaBase) {
    if (!cosT || !sinT || nDims < 2 || (nDims % 2u) != 0) return TC_EINVAL;
    const uint32_t half = nDims / 2;
    const float thetaScale = std::pow(thetaBase, -2.0f / static_cast<float>(nDims));
    for (uint32_t p = 0; p < rows; ++p) {
        float theta = 1.0f;
        for (uint32_t j = 0; j < half; ++j) {
            cosT[static_cast<size_t>(p) * half + j] = std::cos(static_cast<float>(p) * theta);
            sinT[static_cast<size_t>(p) * half + j] = std::sin(static_cast<float>(p) * theta);
            theta *= thetaScale;
        }
    }
    return TC_OK;
}

}  // extern "C"
