// ref_shim.cpp -- C entry points around the reference project's OWN object code.
// TEST INFRASTRUCTURE ONLY (same rule as tc_oracle.c): nothing that ships may
// link or load what this builds.
//
// oracle/Makefile compiles three reference sources where they lie
// (src/cpp/core/ContextPlan.cpp, ThreadPool.cpp, SIMDMatMulVecAVX512.cpp) and
// links them with this file into oracle/_ref/libtc_ref.so.  The shim adds no
// arithmetic of its own to the planner: ref_plan_context() forwards to
// tinycoder::detail::planContext.  For CPU attention the engine's member
// function Model::attentionFused cannot be compiled outside the engine (its
// header needs an array library that the reference fetches at configure time),
// so its task loop is driven here with the engine's own thread pool
// (ThreadPool::parallelFor2D over seqLen x nKVHeads, as
// src/cpp/core/ModelPrimitives.cpp:258 does) and the engine's own AVX-512 leaf
// kernels (dotProductFMA_AVX512 / accumulateFMA_AVX512,
// src/cpp/core/SIMDMatMulVecAVX512.cpp:46-75); the loop body follows
// ModelPrimitives.cpp:262-342.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <algorithm>

#include "ContextPlan.hpp"
#include "ThreadPool.hpp"

namespace tinycoder::simd {
    void accumulateFMA_AVX512(float *local, const float *blockOut, float alpha, uint32_t n);
    float dotProductFMA_AVX512(const float *hidden, const float *blockOut, uint32_t n);
}// namespace tinycoder::simd

extern "C" {

struct orc_context_request {
    uint32_t requested, modelMax, numLayers, numAttentionLayers, numKVHeads, headDim, ropeDims;
    uint32_t int8KvSupported, forceKv, forceKvSet;
    uint64_t weightBytes, freeVram, availableRam, gpuFixedOverhead;
};
struct orc_context_plan {
    uint32_t seqLen, maxAllowed, kv, kvMirror, kvOnGpu, reduced;
    uint64_t kvBytes;
    char reason[256];
};

static tinycoder::detail::ContextRequest toRef(const orc_context_request *r) {
    tinycoder::detail::ContextRequest q;
    q.requested = r->requested;
    q.modelMax = r->modelMax;
    q.numLayers = r->numLayers;
    q.numAttentionLayers = r->numAttentionLayers;
    q.numKVHeads = r->numKVHeads;
    q.headDim = r->headDim;
    q.ropeDims = r->ropeDims;
    q.int8KvSupported = r->int8KvSupported != 0;
    q.forceKv = r->forceKv ? tinycoder::detail::KvPrecision::I8 : tinycoder::detail::KvPrecision::F32;
    q.forceKvSet = r->forceKvSet != 0;
    q.weightBytes = r->weightBytes;
    q.freeVram = r->freeVram;
    q.availableRam = r->availableRam;
    q.gpuFixedOverhead = r->gpuFixedOverhead;
    return q;
}

uint64_t ref_default_gpu_fixed_overhead(void) {
    return tinycoder::detail::ContextRequest{}.gpuFixedOverhead;
}

uint64_t ref_kv_bytes_per_token(const orc_context_request *r, int i8, int mirror) {
    return tinycoder::detail::kvBytesPerToken(
            toRef(r), i8 ? tinycoder::detail::KvPrecision::I8 : tinycoder::detail::KvPrecision::F32,
            mirror != 0);
}

uint64_t ref_kv_store_bytes_per_token(const orc_context_request *r, int i8, int mirror) {
    return tinycoder::detail::kvStoreBytesPerToken(
            toRef(r), i8 ? tinycoder::detail::KvPrecision::I8 : tinycoder::detail::KvPrecision::F32,
            mirror != 0);
}

void ref_plan_context(const orc_context_request *r, orc_context_plan *out) {
    const auto p = tinycoder::detail::planContext(toRef(r));
    std::memset(out, 0, sizeof(*out));
    out->seqLen = p.seqLen;
    out->maxAllowed = p.maxAllowed;
    out->kv = p.kv == tinycoder::detail::KvPrecision::I8 ? 1u : 0u;
    out->kvMirror = p.kvMirror ? 1u : 0u;
    out->kvOnGpu = p.kvOnGpu ? 1u : 0u;
    out->reduced = p.reason.find("limited by") != std::string::npos ? 1u : 0u;
    out->kvBytes = p.kvBytes;
    std::strncpy(out->reason, p.reason.c_str(), sizeof(out->reason) - 1);
}

int ref_cpu_has_avx512(void) {
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
}

// Threads the engine would start (ThreadPool::recommendedThreadCount, or the
// caller's count when > 0).  Returns the pool size in use.
uint32_t ref_pool_init(uint32_t threads) {
    auto &pool = tinycoder::ThreadPool::instance();
    if (!pool.isInitialized()) {
        pool.initialize(threads ? threads : tinycoder::ThreadPool::recommendedThreadCount());
    }
    return static_cast<uint32_t>(pool.numThreads());
}

// flatten != 0: "all-cores" variant -- `batch` independent decode sequences
// (each with its own q / cache / output, seqLen rows each) are flattened into
// one (batch*seqLen) x nKVHeads task grid.  flatten == 0 with batch > 1 runs
// the sequences one after another, as the single-session engine would.
void ref_attention_fused(const float *q, const float *kCache, const float *vCache, float *output,
                         uint32_t batch, uint64_t qStride, uint64_t kvStride, const uint32_t *cachePosArr,
                         uint32_t seqLen, uint32_t nHeads, uint32_t nKVHeads, uint32_t headDim,
                         int flatten) {
    using tinycoder::simd::accumulateFMA_AVX512;
    using tinycoder::simd::dotProductFMA_AVX512;
    const uint32_t nGroups = nHeads / nKVHeads;
    const float invSqrtHeadDim = 1.0f / std::sqrt(static_cast<float>(headDim));
    constexpr float LOG2E = 1.4426950408889634f;
    constexpr uint32_t BLOCK = 32;
    auto task = [&](uint32_t bs, uint32_t g) {
        const uint32_t b = bs / seqLen, s = bs % seqLen;
        const float *qb = q + b * qStride;
        const float *kc = kCache + b * kvStride;
        const float *vc = vCache + b * kvStride;
        float *ob = output + b * qStride;
        const uint64_t csEnd = static_cast<uint64_t>(cachePosArr[b]) + s;
        for (uint32_t h = 0; h < nGroups; ++h) {
            const uint32_t qHead = g * nGroups + h;
            const float *qPtr = qb + (static_cast<uint64_t>(s) * nHeads + qHead) * headDim;
            float o[256];
            for (uint32_t d = 0; d < headDim; ++d) o[d] = 0.0f;
            float m = -std::numeric_limits<float>::infinity();
            float l = 0.0f;
            uint64_t cs = 0;
            for (; cs + BLOCK <= csEnd + 1; cs += BLOCK) {
                float scores[BLOCK];
                for (uint32_t i = 0; i < BLOCK; ++i) {
                    scores[i] = dotProductFMA_AVX512(qPtr, kc + ((cs + i) * nKVHeads + g) * headDim, headDim) *
                                invSqrtHeadDim;
                }
                float blockMax = scores[0];
                for (uint32_t i = 1; i < BLOCK; ++i) blockMax = std::max(blockMax, scores[i]);
                const float mNew = std::max(m, blockMax);
                const float alpha = std::exp2f((m - mNew) * LOG2E);
                if (alpha != 1.0f) accumulateFMA_AVX512(o, o, alpha - 1.0f, headDim);
                l *= alpha;
                for (uint32_t i = 0; i < BLOCK; ++i) {
                    const float p = std::exp2f((scores[i] - mNew) * LOG2E);
                    l += p;
                    accumulateFMA_AVX512(o, vc + ((cs + i) * nKVHeads + g) * headDim, p, headDim);
                }
                m = mNew;
            }
            for (; cs <= csEnd; ++cs) {
                const float score =
                        dotProductFMA_AVX512(qPtr, kc + (cs * nKVHeads + g) * headDim, headDim) * invSqrtHeadDim;
                if (score > m) {
                    const float alpha = std::exp2f((m - score) * LOG2E);
                    if (alpha != 1.0f) accumulateFMA_AVX512(o, o, alpha - 1.0f, headDim);
                    l *= alpha;
                    m = score;
                }
                const float p = std::exp2f((score - m) * LOG2E);
                l += p;
                accumulateFMA_AVX512(o, vc + (cs * nKVHeads + g) * headDim, p, headDim);
            }
            const float invL = 1.0f / l;
            float *outPtr = ob + (static_cast<uint64_t>(s) * nHeads + qHead) * headDim;
            for (uint32_t d = 0; d < headDim; ++d) outPtr[d] = o[d] * invL;
        }
    };
    auto &pool = tinycoder::ThreadPool::current();
    if (flatten) {
        pool.parallelFor2D(batch * seqLen, nKVHeads, task);
    } else {
        for (uint32_t b = 0; b < batch; ++b) {
            pool.parallelFor2D(seqLen, nKVHeads,
                               [&](uint32_t s, uint32_t g) { task(b * seqLen + s, g); });
        }
    }
}

}// extern "C"
