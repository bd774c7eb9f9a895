// decode_shared.cuh -- pieces shared by the split-KV decode kernels (int8 store and
// f32/fp16 cache): the bounded mbarrier wait, the chunk plan, the merge launcher.
#pragma once

#include "tc_common.cuh"

namespace tc {

int launchMerge(const float *pAcc, const float *pM, const float *pL, float *out, uint32_t seqLen,
                uint32_t nHeads, uint32_t numChunks, uint32_t activeHost, uint32_t hd, const uint32_t *devLens,
                uint32_t lenAdd, uint32_t chunkTokens, uint8_t *q81, bool pdl, cudaStream_t st,
                uint32_t chunksPerRank = 0, uint64_t rankStride = 0);

// int8 decode on tcgen05 (decode_i8_tc.cu): head_dim 128, heads mode; arguments already validated
int decodeI8Tc(const tc_decode_i8_batch *d, uint32_t lenHost, uint32_t lenAdd, cudaStream_t st);

// fp16-cache twins of the f32 decode / causal kernels (decode_kv16.cu); arguments already validated
int decodeKv16(const float *q, const void *kvK, const void *kvV, float *attnOut, float *pAcc, float *pM, float *pL,
               uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t pos, const uint32_t *devPos, uint64_t totalRows,
               uint32_t numChunks, float invSqrt, uint8_t *q81Out, cudaStream_t st);
int prefillKv16(const float *q, const void *kvK, const void *kvV, float *out, uint32_t seqLen, uint32_t nHeads,
                uint32_t nKV, uint32_t hd, uint32_t cachePos, const uint32_t *devPos, uint64_t totalRows,
                float invSqrt, cudaStream_t st);

#ifdef __CUDACC__
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

#endif

// rowsPerStage = (token, kv-head) rows one pipeline stage holds; a CTA streams
// hpc kv heads, so a stage covers rowsPerStage / hpc tokens.
struct DecodePlan {
    uint32_t hpc, headGroups, chunkTokens, chunksPerSeq, tileTokens;
};

// One wave of CTAs over the SMs when every sequence has the same (host-known) length: a second
// wave only adds a tail (measured, 8 sequences of 32768 rows: 48.5 us per layer with one wave,
// 53.3 with two, 56.7 with three).  Lengths that live on the device may be ragged: chunks are cut
// by the longest sequence, short sequences leave most of theirs empty, and four waves of small
// chunks let the hardware scheduler even things out (64 sequences in [512, 32768]: 182 us with
// four waves, 186 with two, 324 with one).
inline DecodePlan planDecode(uint32_t batch, uint32_t nKV, uint32_t maxLen, uint32_t slots, uint32_t rowsPerStage,
                             bool uniformLengths = true, uint32_t maxHpc = 4) {
    DecodePlan pl;
    pl.hpc = (nKV % 4u == 0 && maxHpc >= 4u) ? 4u : ((nKV % 2u == 0 && maxHpc >= 2u) ? 2u : 1u);
    pl.headGroups = nKV / pl.hpc;
    pl.tileTokens = rowsPerStage / pl.hpc;
    const uint32_t tilesMax = (maxLen + pl.tileTokens - 1) / pl.tileTokens;
    const uint32_t sms = static_cast<uint32_t>(numSMs());
    // (four waves of blocks that stream four kv heads each; a block that streams fewer kv heads gets
    // proportionally more of them, so that a block covers the same token range: 64 ragged sequences
    // with one kv head per block: 204 us at 4 waves, 184 at 8 and 16, 206 at 32)
    const uint32_t waves = (batch > 1 && !uniformLengths) ? 4u * (4u / pl.hpc) : 1u;
    uint32_t want = (sms * waves) / (batch * pl.headGroups);
    want = want < 1u ? 1u : want;
    // ragged batches: never cut a sequence finer than about 24 stages per block -- with few sequences per
    // GPU the wave rule alone leaves blocks of a few tiles whose set-up costs more than their work
    if (waves > 1u && want > (tilesMax + 23u) / 24u) want = (tilesMax + 23u) / 24u;
    want = want > slots ? slots : want;
    want = want > tilesMax ? tilesMax : want;
    want = want < 1u ? 1u : want;
    const uint32_t tilesPerChunk = (tilesMax + want - 1) / want;
    pl.chunkTokens = tilesPerChunk * pl.tileTokens;
    pl.chunksPerSeq = (tilesMax + tilesPerChunk - 1) / tilesPerChunk;
    if (pl.chunksPerSeq == 0) pl.chunksPerSeq = 1;
    return pl;
}


}  // namespace tc
