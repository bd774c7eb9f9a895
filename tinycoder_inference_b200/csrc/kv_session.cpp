// kv_session.cpp -- the host-side bookkeeping of the attention block: which kernels run for a
// (slot, position, row count) given the KV mode the context plan chose, the per-slot row count
// of the int8 pool, the window guard and the cache reset.
//
// Mirrors the attention block of GPUModel's per-layer loop
// (src/cpp/core/cuda/forward/GPUComputeMoE.cu:3013-3200 for the gated models,
// GPUComputeForward.cu:3778-4040 for the dense ones), GPUModel::forward's window guard
// (GPUComputeForward.cu:3362-3372) and GPUModel::clearKVCache (:5175-5222).  The session owns
// no device memory: the pools, scales and partial buffers stay with the caller, laid out as
// tc_kv_pool_geometry_compute says, exactly as GPUModel lays them out.  Not thread-safe, one
// stream per session -- the reference's contract (one caller at a time under the adapter mutex).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/tc_attn.h"

struct tc_kv_session {
    tc_kv_session_config c;
    tc_kv_pool_geometry g;
    std::vector<uint32_t> rows8;  // kv8Rows_: rows of each slot's int8 pool that are current
    uint32_t kvPos = 0;           // kvPos_
    bool contextFull = false;     // contextFull_
    float invSqrt = 0.0f;
    size_t elem = 4;
};

namespace {

inline uint8_t *slotPtr(void *base, uint64_t stride, uint32_t slot) {
    return static_cast<uint8_t *>(base) + stride * slot;
}

}  // namespace

extern "C" {

int tc_kv_session_create(const tc_kv_session_config *cfg, tc_kv_session **out) {
    if (!cfg || !out) return TC_EINVAL;
    *out = nullptr;
    if (cfg->nKV == 0 || cfg->nHeads == 0 || cfg->nHeads % cfg->nKV != 0 || cfg->hd == 0 || cfg->slots == 0 ||
        cfg->maxSeqLen == 0)
        return TC_EINVAL;
    const bool int8Pool = cfg->kvStoreI8 || cfg->kvMirror;
    if (cfg->kvStoreI8 && (cfg->kvMirror || cfg->kvHalf)) return TC_EINVAL;  // the store is either int8 or f32/fp16
    if (!cfg->kvStoreI8 && (!cfg->kvK || !cfg->kvV)) return TC_EINVAL;
    if (int8Pool && (!cfg->kvK8 || !cfg->kvV8 || !cfg->kvK8Scale || !cfg->kvV8Scale)) return TC_EINVAL;
    if ((cfg->ropeCos == nullptr) != (cfg->ropeSin == nullptr)) return TC_EINVAL;
    // The int8 paths attend over rows as the caller hands them in (already rotated, as the gated
    // models do it in their own Q/K norm + rotation kernel): rotation tables together with an int8
    // pool would rotate the prefill rows and not the decode rows.
    if (int8Pool && cfg->ropeCos != nullptr) return TC_EUNSUPPORTED;
    // The decode pool is rebuilt from f32 rows; an fp16 store has none to rebuild it from.
    if (cfg->kvHalf && cfg->kvMirror) return TC_EUNSUPPORTED;
    tc_kv_session *s = new (std::nothrow) tc_kv_session();
    if (!s) return TC_EINVAL;
    s->c = *cfg;
    // one slot per attention layer: interval 1 over `slots` layers gives the strides of the pools
    const int rc = tc_kv_pool_geometry_compute(cfg->maxSeqLen, cfg->slots, 1, cfg->nHeads, cfg->nKV, cfg->hd,
                                               cfg->kvHalf, cfg->kvStoreI8, cfg->kvMirror, &s->g);
    if (rc != TC_OK) {
        delete s;
        return rc;
    }
    s->rows8.assign(cfg->slots, 0u);
    s->invSqrt = 1.0f / std::sqrt(static_cast<float>(cfg->hd));
    s->elem = cfg->kvHalf ? 2 : 4;
    *out = s;
    return TC_OK;
}

void tc_kv_session_destroy(tc_kv_session *s) { delete s; }

// GPUModel::clearKVCache: zero the f32 / fp16 cache, forget every int8 row, position 0.
int tc_kv_session_clear(tc_kv_session *s, tc_stream stream) {
    if (!s) return TC_EINVAL;
    s->contextFull = false;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!s->c.kvStoreI8) {
        const size_t bytes = static_cast<size_t>(s->g.kvLayerStride) * s->c.slots;
        if (cudaMemsetAsync(s->c.kvK, 0, bytes, st) != cudaSuccess) return TC_ECUDA;
        if (cudaMemsetAsync(s->c.kvV, 0, bytes, st) != cudaSuccess) return TC_ECUDA;
    }
    s->kvPos = 0;
    // the pool itself needs no memset: the next decode rebuilds exactly rows [0, pos)
    std::fill(s->rows8.begin(), s->rows8.end(), 0u);
    return cudaStreamSynchronize(st) == cudaSuccess ? TC_OK : TC_ECUDA;
}

// GPUModel::forward's guard: a request that would grow the position past the window is refused
// before any kernel writes; the refusal is a state of its own, not a fault.
int tc_kv_session_begin(tc_kv_session *s, uint32_t newTokens, uint32_t *pos) {
    if (!s || !pos) return TC_EINVAL;
    if (static_cast<uint64_t>(s->kvPos) + newTokens > s->c.maxSeqLen) {
        s->contextFull = true;
        return TC_ECONTEXT_FULL;
    }
    *pos = s->kvPos;
    return TC_OK;
}

int tc_kv_session_commit(tc_kv_session *s, uint32_t newTokens) {
    if (!s) return TC_EINVAL;
    if (static_cast<uint64_t>(s->kvPos) + newTokens > s->c.maxSeqLen) return TC_ECONTEXT_FULL;
    s->kvPos += newTokens;
    return TC_OK;
}

uint32_t tc_kv_session_pos(const tc_kv_session *s) { return s ? s->kvPos : 0; }
int tc_kv_session_context_full(const tc_kv_session *s) { return s && s->contextFull ? 1 : 0; }
uint32_t tc_kv_session_rows8(const tc_kv_session *s, uint32_t slot) {
    return (s && slot < s->rows8.size()) ? s->rows8[slot] : 0;
}

int tc_kv_session_attend(tc_kv_session *s, uint32_t slot, float *q, const float *kSrc, const float *vSrc,
                         float *attnOut, uint32_t seqLen, uint32_t pos, const uint32_t *devPos, int graphCapture,
                         tc_stream stream) {
    if (!s || !q || !kSrc || !vSrc || !attnOut) return TC_EINVAL;
    if (slot >= s->c.slots) return TC_EINVAL;
    if (seqLen == 0) return TC_OK;
    const tc_kv_session_config &c = s->c;
    if (static_cast<uint64_t>(pos) + seqLen > c.maxSeqLen) {
        s->contextFull = true;
        return TC_ECONTEXT_FULL;
    }
    const uint32_t nH = c.nHeads, nKV = c.nKV, hd = c.hd;
    const bool int8Pool = c.kvStoreI8 || c.kvMirror;
    const uint64_t rows8Cap = static_cast<uint64_t>(c.maxSeqLen) + 16;
    int8_t *k8 = nullptr, *v8 = nullptr;
    float *ks = nullptr, *vs = nullptr;
    if (int8Pool) {
        k8 = c.kvK8 + s->g.kv8LayerStride * slot;
        v8 = c.kvV8 + s->g.kv8LayerStride * slot;
        ks = c.kvK8Scale + (s->g.kv8ScaleStride / sizeof(float)) * slot;
        vs = c.kvV8Scale + (s->g.kv8ScaleStride / sizeof(float)) * slot;
    }
    void *kvK = nullptr, *kvV = nullptr;
    if (!c.kvStoreI8) {
        kvK = slotPtr(c.kvK, s->g.kvLayerStride, slot);
        kvV = slotPtr(c.kvV, s->g.kvLayerStride, slot);
    }
    int rc;

    // ---- decode over the int8 pool (kv8Decode) ----
    // One row, not under graph capture (the row counts below are host state the replay could
    // not update), position known on the host.
    if (int8Pool && seqLen == 1 && !graphCapture && devPos == nullptr) {
        uint32_t &rows8 = s->rows8[slot];
        if (!c.kvStoreI8) {
            if (rows8 < pos) {
                // rows a prefill left in the f32 cache but not in the pool: [rows8, pos)
                if (c.kvHalf) return TC_EUNSUPPORTED;  // the mirror is rebuilt from f32 rows
                rc = tc_kv_quantize_i8(static_cast<const float *>(kvK), static_cast<const float *>(kvV), k8, v8, ks,
                                       vs, pos - rows8, nKV, hd, rows8, rows8, nullptr, rows8Cap, stream);
                if (rc != TC_OK) return rc;
                rows8 = pos;
            }
            // The reference leaves the f32 row of a token decoded through the pool unwritten;
            // writing it costs one row and keeps a later multi-row call (which reads the f32
            // cache) looking at the whole history.  The attention of this call does not read it.
            rc = tc_kv_append(kSrc, vSrc, kvK, kvV, c.kvHalf, 1, nKV, hd, pos, nullptr, c.maxSeqLen, stream);
            if (rc != TC_OK) return rc;
        }
        // the decode launch quantises the new row into the pool itself (one launch instead of two)
        tc_decode_i8_batch d;
        memset(&d, 0, sizeof(d));
        d.q = q, d.out = attnOut;
        d.k8 = k8, d.v8 = v8, d.ks = ks, d.vs = vs;
        d.pAcc = c.pAcc, d.pM = c.pM, d.pL = c.pL;
        d.totalRows = rows8Cap;
        d.batch = 1, d.nHeads = nH, d.nKV = nKV, d.hd = hd;
        d.maxLen = pos + 1u;
        d.numChunks = c.numChunks;
        d.invSqrt = s->invSqrt;
        d.appendK = kSrc, d.appendV = vSrc;
        rc = tc_attn_decode_i8_batch(&d, stream);
        if (rc == TC_OK) rows8 = pos + 1u;
        return rc;
    }

    // ---- int8 as the store: quantise the rows straight into the pool, attend over it ----
    if (c.kvStoreI8) {
        rc = tc_kv_quantize_i8(kSrc, vSrc, k8, v8, ks, vs, seqLen, nKV, hd, pos, 0, devPos, rows8Cap, stream);
        if (rc != TC_OK) return rc;
        s->rows8[slot] = pos + seqLen;
        // a multi-row call with scratch for the twins (bytes x row scale) takes the tensor-core prefill
        if (seqLen > 1 && devPos == nullptr && !graphCapture && (hd == 64 || hd == 128 || hd == 256) && c.prefillScratch != nullptr) {
            size_t need = 0;
            if (tc_attn_prefill_f16_scratch_bytes(seqLen, pos, nH, nKV, hd, &need) == TC_OK && need <= c.prefillScratchBytes)
                return tc_attn_prefill_f16_i8(q, k8, v8, ks, vs, attnOut, c.prefillScratch, c.prefillScratchBytes, seqLen,
                                              pos, nH, nKV, hd, s->invSqrt, stream);
        }
        return tc_attn_prefill_i8(q, k8, v8, ks, vs, attnOut, seqLen, nH, nKV, hd, pos, devPos, rows8Cap, s->invSqrt,
                                  stream);
    }

    // ---- f32 / fp16 store ----
    if (c.ropeCos != nullptr)
        rc = tc_kv_append_rope(q, kSrc, vSrc, kvK, kvV, c.kvHalf, seqLen, nH, nKV, hd, pos, pos, devPos, c.ropeCos,
                               c.ropeSin, c.maxSeqLen, stream);
    else
        rc = tc_kv_append(kSrc, vSrc, kvK, kvV, c.kvHalf, seqLen, nKV, hd, pos, devPos, c.maxSeqLen, stream);
    if (rc != TC_OK) return rc;
    // (no int8 bookkeeping here: the next decode's rebuild converts exactly the rows the pool lacks)
    if (seqLen == 1) {
        // A launch whose position lives on the device (the form a captured graph replays) is sized
        // for the whole window: the host position is only the value at capture time, the grid and
        // the chunk length must cover every position a replay can reach (the reference's *Pos
        // decode launches its fixed attnChunk_ x attnChunks_ grid for the same reason).
        const uint32_t hostBound = devPos != nullptr ? c.maxSeqLen - 1u : pos;
        return tc_attn_decode_kv(q, kvK, kvV, attnOut, c.pAcc, c.pM, c.pL, 1, nH, nKV, hd, hostBound, devPos,
                                 c.maxSeqLen, c.numChunks, 0, s->invSqrt, c.kvHalf, nullptr, stream);
    }
    // every multi-row call on the f32 cache -- the first chunk of a prompt and the chunks behind it
    // (ModelForward.cpp:115-127 cuts prompts into 512-token calls) -- takes the tensor-core prefill
    // when the caller's scratch holds the fp16 twins of the rows it attends over
    if (devPos == nullptr && !graphCapture && c.kvHalf && (hd == 64 || hd == 128 || hd == 256) && c.prefillScratch != nullptr) {
        // the fp16 store is read in place: the scratch only has to hold q's twin
        size_t need = 0;
        if (tc_attn_prefill_f16_scratch_bytes(seqLen, 0, nH, 0, hd, &need) == TC_OK && need <= c.prefillScratchBytes)
            return tc_attn_prefill_f16_kvhalf(q, kvK, kvV, attnOut, c.prefillScratch, c.prefillScratchBytes, seqLen, pos,
                                              nH, nKV, hd, s->invSqrt, stream);
    }
    if (devPos == nullptr && !graphCapture && !c.kvHalf && (hd == 64 || hd == 128 || hd == 256) && c.prefillScratch != nullptr) {
        size_t need = 0;
        if (tc_attn_prefill_f16_scratch_bytes(seqLen, pos, nH, nKV, hd, &need) == TC_OK && need <= c.prefillScratchBytes) {
            // With a decode pool that is current up to this call's first row, the launch that makes
            // the fp16 twins writes the pool's rows of the new positions too: the mirror stays
            // current through the chunks of a prompt and the first decode step has nothing to rebuild.
            if (c.kvMirror && s->rows8[slot] == pos) {
                rc = tc_attn_prefill_f16_kv8(q, static_cast<const float *>(kvK), static_cast<const float *>(kvV),
                                             attnOut, c.prefillScratch, c.prefillScratchBytes, seqLen, pos, nH, nKV, hd,
                                             s->invSqrt, k8, v8, ks, vs, pos, rows8Cap, stream);
                if (rc == TC_OK) s->rows8[slot] = pos + seqLen;
                return rc;
            }
            return tc_attn_prefill_f16(q, static_cast<const float *>(kvK), static_cast<const float *>(kvV), attnOut,
                                       c.prefillScratch, c.prefillScratchBytes, seqLen, pos, nH, nKV, hd, s->invSqrt,
                                       stream);
        }
    }
    return tc_attn_prefill_kv(q, kvK, kvV, attnOut, seqLen, nH, nKV, hd, pos, devPos, c.maxSeqLen, s->invSqrt,
                              c.kvHalf, stream);
}

}  // extern "C"
