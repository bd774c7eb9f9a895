/*
 * tc_attn.h -- C ABI of the B200 attention / KV-cache library (libtc_attn.so).
 *
 * These entry points are the call shapes of the reference engine's GPU
 * attention block: the kernels and host launchers that
 * tinycoder::gpu::GPUModel (include/GPUCompute.hpp:195-331) invokes with raw
 * device pointers inside its per-layer loops.  Each declaration names the
 * reference launch it replaces (path inside the reference project, line range).
 *
 * Conventions (the reference's own, kept):
 *   - every pointer is a DEVICE pointer owned by the caller unless the comment
 *     says HOST; the library never allocates device memory and never
 *     synchronises (the reference forbids allocation inside launches for CUDA
 *     graph capture, include/gpu/GpuAttentionKernels.hpp:1133-1135);
 *   - the stream is explicit (`tc_stream` is a cudaStream_t);
 *   - layouts are row-major, token-major: q/out [seq][nHeads][hd] f32;
 *     K/V cache [row][nKV][hd]; int8 pool [row][nKV][hd] int8 with scales
 *     [row][nKV] f32; partials partAcc [seq][nHeads][numChunks][hd],
 *     partM/partL [seq][nHeads][numChunks] (include/GPUCompute.hpp:1203-1204);
 *   - the GQA map is kvHead = qHead / (nHeads / nKV)
 *     (include/gpu/GpuAttentionKernels.hpp:226);
 *   - a position may arrive as a host value or as a device scalar (`devPos`,
 *     read at kernel time so that a captured graph can be replayed; the
 *     reference's *Pos kernel twins, GpuAttentionKernels.hpp:355-363);
 *   - functions return 0 on success or a TC_E* code; they never throw, abort
 *     or fall back to a CPU path.  tc_last_error() gives the message of the
 *     calling thread's last failure.
 *   - not thread-safe per (stream, workspace) pair, re-entrant across distinct
 *     pairs (one host thread per GPU may drive its own device).
 */
#ifndef TC_ATTN_H
#define TC_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *tc_stream; /* cudaStream_t */

enum {
    TC_OK = 0,
    TC_EINVAL = 1,        /* bad shape / pointer / alignment */
    TC_ECONTEXT_FULL = 2, /* the write would pass the window: nothing was launched
                             (GPUComputeForward.cu:3366-3372, ModelForward.cpp:57-63) */
    TC_ECUDA = 3,         /* a CUDA runtime / driver call failed */
    TC_EUNSUPPORTED = 4,  /* shape outside what the kernels are built for */
    TC_EWORKSPACE = 5,    /* caller's partial buffers are too small */
    TC_EDEVICE = 6        /* a kernel recorded a device-side error (bounded wait ran out) */
};

const char *tc_strerror(int code);
const char *tc_last_error(void);
/* Reads and clears the device-side error word of the current device
 * (synchronises the given stream).  0 = no kernel reported anything.  Bits:
 * 1 / 2 / 4 / 16 a bounded wait ran out (TMA stage, free stage, tensor-core commit,
 * partials of another rank), 8 TMEM allocation, 32 a KV writer read a
 * device-side position outside its pool and skipped the store. */
int tc_device_status(tc_stream stream, uint32_t *flags);

/* ------------------------------------------------------------------------- */
/* KV append                                                                   */
/* ------------------------------------------------------------------------- */

/* Replaces kQ35StoreKV (include/gpu/GpuQwen35Kernels.hpp:497-516; launch
 * src/cpp/core/cuda/forward/GPUComputeMoE.cu:3132): rows cachePos+s of kDst/vDst
 * receive kSrc/vSrc [seqLen][nKV*hd] verbatim.  devPos (nullable) overrides
 * cachePos.  kvHalf != 0 stores fp16 (the KV16 cache of
 * include/gpu/GpuElementwiseKernels.hpp:64-89).  maxRows bounds the write:
 * cachePos + seqLen > maxRows returns TC_ECONTEXT_FULL with a host position;
 * with devPos the kernel checks each row, skips a store that would land outside
 * and raises bit 32 of the device error word (the reference's *Pos kernels write
 * unchecked). */
int tc_kv_append(const float *kSrc, const float *vSrc, void *kDst, void *vDst,
                 int kvHalf, uint32_t seqLen, uint32_t nKV, uint32_t hd,
                 uint32_t cachePos, const uint32_t *devPos, uint32_t maxRows,
                 tc_stream stream);

/* Replaces kStoreKVRope / kStoreKVRopePos and, with q != NULL, the fused
 * kRoPEQStoreKV / kRoPEQStoreKVPos (include/gpu/GpuElementwiseKernels.hpp:452-483;
 * include/gpu/GpuAttentionKernels.hpp:389-533; launches
 * GPUComputeForward.cu:3878-3895): V verbatim, K rotated NEOX-style with the
 * angle row ropePos+s, into row cachePos+s; q [seqLen][nHeads][hd] rotated in
 * place.  cosT/sinT: [rows][hd/2] f32.  devPos (nullable) replaces both
 * cachePos and ropePos. */
int tc_kv_append_rope(float *q, const float *kSrc, const float *vSrc, void *kDst,
                      void *vDst, int kvHalf, uint32_t seqLen, uint32_t nHeads,
                      uint32_t nKV, uint32_t hd, uint32_t cachePos,
                      uint32_t ropePos, const uint32_t *devPos,
                      const float *cosT, const float *sinT, uint32_t maxRows,
                      tc_stream stream);

/* Replaces kRoPEQ / kRoPEQPos (include/gpu/GpuElementwiseKernels.hpp:425-448;
 * include/gpu/GpuAttentionKernels.hpp:364-387). */
int tc_rope_q(float *q, const float *cosT, const float *sinT, uint32_t seqLen,
              uint32_t nHeads, uint32_t hd, uint32_t pos, const uint32_t *devPos,
              tc_stream stream);

/* Replaces kQ35QuantKV8 (include/gpu/GpuQwen35Kernels.hpp:586-637; launches
 * GPUComputeMoE.cu:3056-3063, 3103-3105): quantise rows srcTokenBase+t of the
 * f32 k/v [row][nKV][hd] into rows dstTokenBase+t of the int8 pool, one f32
 * scale per (row, kv head): scale = amax/127 (1 when amax == 0),
 * q = clamp(lrintf(x/scale), -128, 127).  Bit-exact with the reference.
 * devDstBase (nullable) overrides dstTokenBase at kernel time; a row it sends
 * past maxRows (!= 0) is not stored and raises bit 32 of the device error word. */
int tc_kv_quantize_i8(const float *k, const float *v, int8_t *k8, int8_t *v8,
                      float *ks, float *vs, uint32_t tokens, uint32_t nKV,
                      uint32_t hd, uint64_t dstTokenBase, uint64_t srcTokenBase,
                      const uint32_t *devDstBase, uint64_t maxRows,
                      tc_stream stream);

/* The same quantiser for a batch of sequences that live in ONE pool (batched serving,
 * the layout tc_attn_decode_i8_batch reads): k/v [batch][nKV][hd] hold the new token
 * of every sequence; sequence b's row goes to
 *   (rowBase ? rowBase[b] : b * rowsPerSeq) + (lens ? lens[b] + lenAdd : pos).
 * lens / rowBase are device arrays (nullable).  With lens counting the new token
 * already (as tc_attn_decode_i8_batch wants it) pass lenAdd = -1.  One launch. */
int tc_kv_quantize_i8_batch(const float *k, const float *v, int8_t *k8, int8_t *v8,
                            float *ks, float *vs, uint32_t batch, uint32_t nKV,
                            uint32_t hd, uint64_t rowsPerSeq, const uint64_t *rowBase,
                            uint32_t pos, const uint32_t *lens, int32_t lenAdd,
                            uint64_t totalRows, tc_stream stream);

/* ------------------------------------------------------------------------- */
/* decode attention                                                            */
/* ------------------------------------------------------------------------- */

/* Bytes of partial storage for one decode call: fills the three sizes (in
 * bytes) the caller must give pAcc / pM / pL for `batch` sequences and
 * `numChunks` chunk slots (the reference sizes them in
 * src/cpp/core/cuda/forward/GPUComputeUpload.cu:354-365 for one token). */
int tc_attn_workspace_bytes(uint32_t batch, uint32_t nHeads, uint32_t hd,
                            uint32_t numChunks, size_t *accBytes,
                            size_t *mBytes, size_t *lBytes);

/* Chunk grid the library would pick for a window: the reference's
 * attnChunk_/attnChunks_ rule (GPUComputeUpload.cu:318-334; at most 512 chunks,
 * chunk a multiple of 32).  The decode entry points accept any numChunks >= 1;
 * they use at most numChunks chunk slots and choose their own tiling inside. */
int tc_split_geometry(uint32_t maxSeqLen, uint32_t nHeads, uint32_t hd,
                      uint32_t *chunkSize, uint32_t *numChunks);

/* Replaces kQ35WarpAttention8Split + kAttnCombinePartial, and the eager
 * kQ35WarpAttention8 (include/gpu/GpuQwen35Kernels.hpp:519-581, 641-692;
 * launches GPUComputeMoE.cu:3073-3090): one query token, attention over rows
 * [0, cachePos] of an int8 store, out [nHeads][hd] f32.  devPos (nullable)
 * overrides cachePos at kernel time (then cachePos is the host's upper bound
 * and sizes the grid).  pAcc/pM/pL hold numChunks chunk slots per head;
 * chunkSize is the caller's chunk (a hint: the kernel tiles the range itself).
 * totalRows = rows allocated in the pool (>= cachePos+1). */
int tc_attn_decode_i8(const float *q, const int8_t *k8, const int8_t *v8,
                      const float *ks, const float *vs, float *out, float *pAcc,
                      float *pM, float *pL, uint32_t nHeads, uint32_t nKV,
                      uint32_t hd, uint32_t cachePos, const uint32_t *devPos,
                      uint64_t totalRows, uint32_t numChunks, uint32_t chunkSize,
                      float invSqrt, tc_stream stream);

/* Batched form of the above for `batch` independent sequences that live in ONE
 * int8 pool (the serving mix: one decode step of many sessions).  Sequence b
 * occupies pool rows [rowBase[b], rowBase[b] + lens[b]); rowBase == NULL means
 * b * rowsPerSeq.  lens / rowBase are DEVICE arrays (uint32 / uint64); maxLen is
 * the host's upper bound on lens[] and sizes the grid; lens == NULL means every
 * sequence is exactly maxLen rows long.  q/out: [batch][nHeads][hd].
 * partialsOnly != 0 skips the merge and leaves (m, l, acc) per chunk in
 * pAcc/pM/pL -- the form a context-axis split across GPUs exchanges;
 * *chunksUsed (HOST, nullable) receives the chunk slots written per head. */
typedef struct tc_decode_i8_batch {
    const float *q;
    float *out;
    const int8_t *k8, *v8;
    const float *ks, *vs;
    float *pAcc, *pM, *pL;
    const uint32_t *lens;    /* device [batch] */
    const uint64_t *rowBase; /* device [batch] or NULL */
    uint64_t rowsPerSeq;
    uint64_t totalRows;
    uint32_t batch, nHeads, nKV, hd;
    uint32_t maxLen;
    uint32_t numChunks;
    float invSqrt;
    int partialsOnly;
    uint32_t *chunksUsed; /* HOST out, nullable */
    /* flags & TC_DECODE_PDL: launch with programmatic dependent launch, i.e. the
     * kernels may begin while the kernels ahead of them in the stream drain.
     * Whatever a kernel in flight may still write is read only after those
     * kernels have completed: q, the lengths, and every K/V row >= prefetchRows.
     * Rows [0, prefetchRows) of each sequence -- rows no kernel in flight writes,
     * e.g. everything before the token being appended -- are streamed in early,
     * but only with host lengths (lens == NULL: every sequence is maxLen rows
     * long) and rowBase == NULL.  flags == 0 keeps plain stream order. */
    uint32_t flags;
    uint32_t prefetchRows;
    /* Optional hint (NULL = none): the int8 pools the NEXT decode call on this stream
     * will read with the same geometry and lengths -- the next layer's slot.  Once a
     * block has requested its own last tile it asks the memory system to pull the
     * same rows of these pools into L2 (cp.async.bulk.prefetch.tensor), so DRAM keeps
     * streaming while this call's blocks fold their partials and the merge runs,
     * instead of idling until the next call's blocks start.  Nothing is read or
     * written through these pointers by the SMs.  Ignored when a call's rows
     * (batch * maxLen * nKV * hd * 2 bytes) exceed 48 MB: they would not stay in L2. */
    const int8_t *nextK8, *nextV8;
    /* Optional (NULL = merge in a second launch): batch * nKV arrival counters in DEVICE memory,
     * zero before the first call (the kernel leaves them zero).  With them the split-KV kernel
     * merges its own partials (head_dim 128, at most 8 q heads per kv head): every block
     * publishes its chunk partial and takes a ticket, the block that draws the last ticket of
     * a (sequence, kv head) folds all chunks and writes the output -- no block waits for
     * another, and the merge launch with its hand-off disappears.  Calls that may run
     * concurrently (different streams) need counters of their own. */
    uint32_t *mergeTickets;
    /* Optional (NULL = the rows are in the pool already): the new token's K and V rows, f32
     * [batch][nKV][hd].  The launch then quantises them into row len - 1 of every sequence --
     * the bytes and scales tc_kv_quantize_i8_batch writes -- before that row is read: the blocks
     * that hold a sequence's last tile do it once the kernels ahead in the stream have completed,
     * so the separate quantise launch between two layers' attention disappears.  k8 / v8 / ks / vs
     * are written through in this case.  A device length that puts the row outside totalRows
     * skips the store and sets the row-bound bit of tc_device_status. */
    const float *appendK, *appendV;
} tc_decode_i8_batch;

enum { TC_DECODE_PDL = 1u };

int tc_attn_decode_i8_batch(const tc_decode_i8_batch *d, tc_stream stream);

/* No counterpart in the reference.  The same int8 decode as tc_attn_decode_i8 for
 * callers that cannot provide scratch memory because they cannot allocate any: a
 * host that only passes device pointers from a memory plan fixed at load time, or a
 * latency-critical serving loop that is not allowed to touch the device allocator
 * once it is running.  The split-KV partials live in an array built into the library's device
 * image -- about 5.3 MB on every GPU that loads the library, held until the
 * process exits -- so the call takes only inputs and the output and performs no
 * cudaMalloc / cudaFree / allocating library call.
 * Limits: nHeads <= 64 and hd == 128 (TC_EWORKSPACE otherwise); host position only.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture.
 * All calls share the one array, which keeps the last call's partials: nothing in
 * it needs clearing between calls, but two calls that overlap on the GPU (different
 * streams) race on it -- serialise them. */
int tc_attn_decode_i8_noalloc(const float *q, const int8_t *k8, const int8_t *v8,
                              const float *ks, const float *vs, float *out,
                              uint32_t nHeads, uint32_t nKV, uint32_t hd,
                              uint32_t cachePos, uint64_t totalRows, float invSqrt,
                              tc_stream stream);

/* Replaces launchDecodeAttentionSplit (include/gpu/GpuAttentionKernels.hpp:
 * 1129-1230; launch GPUComputeForward.cu:3897-3902): split-KV decode over an
 * f32 (kvHalf == 0) or fp16 (kvHalf != 0) cache, seqLen query rows (the
 * reference only calls it with seqLen == 1), row s attends [0, pos + s].
 * q81Out (nullable): the merge also emits the Q8_1 blocks of the output
 * (40-byte slots per 32 values, GpuAttentionKernels.hpp:1068-1096).
 * With devPos != NULL the position is read on the device at run time and `pos`
 * is an UPPER BOUND of it: the grid and the chunk length are sized from pos + 1,
 * so a launch captured in a CUDA graph and replayed at growing positions passes
 * the last position of the window (maxSeqLen - 1), as the reference's *Pos
 * launch covers its whole attnChunk x attnChunks grid.  Rows past a bound that
 * was too small are not attended. */
int tc_attn_decode_kv(const float *q, const void *kvK, const void *kvV,
                      float *attnOut, float *pAcc, float *pM, float *pL,
                      uint32_t seqLen, uint32_t nHeads, uint32_t nKV, uint32_t hd,
                      uint32_t pos, const uint32_t *devPos, uint64_t totalRows,
                      uint32_t numChunks, uint32_t chunkSize, float invSqrt,
                      int kvHalf, uint8_t *q81Out, tc_stream stream);

/* Replaces kAttnCombinePartial / kAttnCombinePartialW4
 * (include/gpu/GpuAttentionKernels.hpp:909-946, 1003-1098): merge numChunks
 * partials per (token, head): M = max m_c, w_c = exp2((m_c-M)*log2e), chunks
 * with l_c <= 0 skipped, out = sum w_c acc_c / sum w_c l_c.  Also the merge
 * step of a context split across GPUs (numChunks = gathered partials). */
int tc_attn_merge_partials(const float *pAcc, const float *pM, const float *pL,
                           float *out, uint32_t seqLen, uint32_t nHeads,
                           uint32_t numChunks, uint32_t hd, uint8_t *q81Out,
                           tc_stream stream);

/* The merge step of a context-axis split across GPUs (new capability: the reference is
 * single-device).  `gathered` holds, rank after rank, the block every rank produced with
 * partialsOnly: [acc [nHeads][chunksPerRank][hd] | m [nHeads][chunksPerRank] |
 * l [nHeads][chunksPerRank]] (one all-gather of the rank's contiguous workspace).  Slots a
 * rank did not write must hold l == 0.  Same rule as tc_attn_merge_partials; out [nHeads][hd]. */
int tc_attn_merge_gathered(const float *gathered, float *out, uint32_t nHeads,
                           uint32_t ranks, uint32_t chunksPerRank, uint32_t hd,
                           tc_stream stream);

/* The same merge with the exchange inside the kernel (no collective library call).
 * Every rank owns an exchange buffer of tc_attn_exchange_bytes() bytes that all ranks
 * can store into (peer-mapped device memory: CUDA IPC, a symmetric-memory allocation,
 * or plain device memory when all "ranks" share a GPU), zeroed once before first use;
 * buffers[r] is rank r's buffer as addressed from the calling rank.  One launch per
 * rank and step: it merges the rank's own chunk partials (layout [nHeads][numChunks],
 * the first activeChunks slots written) into one partial per head, stores it into
 * every rank's buffer, waits -- at most about a second, after which
 * tc_device_status reports it -- for the partials of all ranks and writes out
 * [nHeads][hd].  Every rank must issue the same sequence of calls on its buffer.
 * flags & TC_DECODE_PDL as for tc_attn_decode_i8_batch. */
typedef struct tc_peer_group {
    void *buffers[16];
    uint32_t world, rank;
} tc_peer_group;

int tc_attn_exchange_bytes(uint32_t nHeads, uint32_t hd, uint32_t world, size_t *bytes);

int tc_attn_merge_exchange(const float *pAcc, const float *pM, const float *pL, float *out,
                           uint32_t nHeads, uint32_t numChunks, uint32_t activeChunks,
                           uint32_t hd, const tc_peer_group *g, uint32_t flags,
                           tc_stream stream);

/* All `ranks` of the protocol in ONE cooperative launch on one GPU (arrays of `ranks`
 * host pointers): for hosts that keep several context shards on one device, and for
 * testing the protocol without a second GPU.  Blocks of the launch wait for one
 * another, hence cooperative: the call fails if the grid cannot be resident at once. */
int tc_attn_merge_exchange_local(const float *const *pAcc, const float *const *pM,
                                 const float *const *pL, float *const *out,
                                 void *const *buffers, uint32_t ranks, uint32_t nHeads,
                                 uint32_t numChunks, uint32_t activeChunks, uint32_t hd,
                                 tc_stream stream);

/* ------------------------------------------------------------------------- */
/* prefill attention                                                           */
/* ------------------------------------------------------------------------- */

/* Scratch bytes tc_attn_prefill_f16 needs (fp16 twins of q and of the K/V
 * rows [0, cachePos + seqLen); the reference keeps attnQ16 / attnKV16 for the
 * same purpose, GPUComputeForward.cu:3952-3968; plus the counter the blocks
 * of the attention launch draw their work from).  The scratch belongs to one
 * call at a time: calls that share it have to be ordered on one stream. */
int tc_attn_prefill_f16_scratch_bytes(uint32_t seqLen, uint32_t cachePos,
                                      uint32_t nHeads, uint32_t nKV,
                                      uint32_t hd, size_t *bytes);

/* Replaces the materialised dense prefill: kF32ToF16 x3, cuBLAS QK^T,
 * kAttnSoftmaxCausal, cuBLAS PV (GPUComputeForward.cu:3937-4026;
 * include/gpu/GpuAttentionKernels.hpp:323-353): causal attention of seqLen
 * query rows at positions cachePos .. cachePos + seqLen - 1 over cache rows
 * [0, cachePos + seqLen), fp16 operands, f32 accumulation, f32 softmax,
 * probabilities rounded to fp16.  head_dim 64, 128 or 256 (TC_EUNSUPPORTED
 * otherwise: tc_attn_prefill_kv takes those shapes).  q f32 [seqLen][nHeads][hd]; kvK/kvV the f32
 * cache from row 0 (the new rows already appended); out f32.  No seqLen cap
 * (the reference stops at 512 because it materialises the score matrix), and
 * no cachePos == 0 condition: the reference takes this path only for the
 * first chunk of a prompt (GPUComputeForward.cu:3828-3835) and sends the
 * other 512-token chunks its caller cuts (ModelForward.cpp:115-127) through
 * the scalar kernel; here every chunk runs on the tensor cores. */
int tc_attn_prefill_f16(const float *q, const float *kvK, const float *kvV,
                        float *out, void *scratch, size_t scratchBytes,
                        uint32_t seqLen, uint32_t cachePos, uint32_t nHeads,
                        uint32_t nKV, uint32_t hd, float invSqrt,
                        tc_stream stream);

/* The same call for an engine that keeps an int8 decode pool beside its f32
 * store (kv8Rows_ and its rebuild before the first decode step,
 * GPUComputeMoE.cu:3049-3063; include/GPUCompute.hpp:869-872): the launch that makes the fp16 twins has
 * every K/V row in registers and also writes the int8 rows of the call's new
 * positions -- cache rows [cachePos, cachePos + seqLen) become pool rows
 * [kv8Row, kv8Row + seqLen), bit-identical to tc_kv_quantize_i8 on those
 * rows -- so no second pass over the cache is needed.  TC_ECONTEXT_FULL when
 * the rows pass kv8MaxRows. */
int tc_attn_prefill_f16_kv8(const float *q, const float *kvK, const float *kvV,
                            float *out, void *scratch, size_t scratchBytes,
                            uint32_t seqLen, uint32_t cachePos,
                            uint32_t nHeads, uint32_t nKV, uint32_t hd,
                            float invSqrt, int8_t *k8, int8_t *v8, float *ks,
                            float *vs, uint64_t kv8Row, uint64_t kv8MaxRows,
                            tc_stream stream);

/* The same kernel over the other two stores (tolerance of the fp16 prefill in
 * both cases: q and the probabilities are rounded to fp16):
 *  - _kvhalf: the fp16 store (kWarpAttention<HD, __half>,
 *    include/gpu/GpuAttentionKernels.hpp:211-272) is read in place -- its layout
 *    is the one the twins have -- so the scratch holds only q's twin
 *    (tc_attn_prefill_f16_scratch_bytes with nKV = 0 says how much);
 *  - _i8: the int8 store (kQ35WarpAttention8Prefill / kQ35PrefillAttnSharedKV8,
 *    include/gpu/GpuQwen35Kernels.hpp:2306-2435): the twins are byte x row scale,
 *    scratch as for the f32 store.  The rows [0, cachePos + seqLen) have to be
 *    in the pool already (tc_kv_quantize_i8 first). */
int tc_attn_prefill_f16_kvhalf(const float *q, const void *kvK16,
                               const void *kvV16, float *out, void *scratch,
                               size_t scratchBytes, uint32_t seqLen,
                               uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                               uint32_t hd, float invSqrt, tc_stream stream);
int tc_attn_prefill_f16_i8(const float *q, const int8_t *k8, const int8_t *v8,
                           const float *ks, const float *vs, float *out,
                           void *scratch, size_t scratchBytes, uint32_t seqLen,
                           uint32_t cachePos, uint32_t nHeads, uint32_t nKV,
                           uint32_t hd, float invSqrt, tc_stream stream);

/* Replaces kWarpAttention / kWarpAttentionPos and kQ35WarpAttention
 * (include/gpu/GpuAttentionKernels.hpp:211-272, 537-599;
 * include/gpu/GpuQwen35Kernels.hpp:2437-2492): causal attention of seqLen query
 * rows, row s over cache rows [0, cachePos + s], f32 or fp16 cache, f32 math. */
int tc_attn_prefill_kv(const float *q, const void *kvK, const void *kvV,
                       float *out, uint32_t seqLen, uint32_t nHeads,
                       uint32_t nKV, uint32_t hd, uint32_t cachePos,
                       const uint32_t *devPos, uint64_t totalRows, float invSqrt,
                       int kvHalf, tc_stream stream);

/* Replaces kQ35WarpAttention8Prefill / kQ35PrefillAttnSharedKV8
 * (include/gpu/GpuQwen35Kernels.hpp:2306-2435; launches GPUComputeMoE.cu:
 * 3110-3130): causal attention of seqLen query rows over an int8 store. */
int tc_attn_prefill_i8(const float *q, const int8_t *k8, const int8_t *v8,
                       const float *ks, const float *vs, float *out,
                       uint32_t seqLen, uint32_t nHeads, uint32_t nKV,
                       uint32_t hd, uint32_t cachePos, const uint32_t *devPos,
                       uint64_t totalRows, float invSqrt, tc_stream stream);

/* ------------------------------------------------------------------------- */
/* the step in front of attention: Q/K RMSNorm + rotation, rotation tables      */
/* ------------------------------------------------------------------------- */

/* Replaces kQ35QNormRoPE + kQ35KNormRoPE (include/gpu/GpuQwen35Kernels.hpp:55-137;
 * launched at src/cpp/core/cuda/forward/GPUComputeForward.cu:1330-1337) in one
 * launch: per (token, head) slice rms = rsqrt(mean(x^2) + 1e-6), y = x*rms*w, the
 * first nDims elements rotated NEOX-style (pairs j, j + nDims/2) by table row
 * pos + s (devPos: position read on the device), the rest copied.  Q: rows
 * qIn[s][h] of stride qInStride floats (2*hd in the gated models: q then gate)
 * -> qOut[s][nHeads][hd], out of place.  K: [s][nKV][hd] in place.  Either side
 * may be NULL.  cosT/sinT [tableRows][nDims/2].  Bit-identical to the reference
 * kernels (same summation order, same intrinsics). */
int tc_qk_norm_rope(const float *qIn, uint32_t qInStride, float *qOut, float *k,
                    const float *wq, const float *wk, uint32_t hd, uint32_t nDims,
                    uint32_t nHeads, uint32_t nKV, uint32_t seqLen, uint32_t pos,
                    const uint32_t *devPos, const float *cosT, const float *sinT,
                    uint32_t tableRows, tc_stream stream);

/* HOST functions: the rotation tables the engine uploads once.
 * tc_rope_tables: [rows][headDim/2], angle = float(p) / powf(theta, 2j/headDim)
 *   (src/cpp/core/cuda/forward/GPUComputeUpload.cu:1149-1163; CPU twin
 *   src/cpp/core/ModelPrimitives.cpp:112-127).
 * tc_mrope_tables: [rows][nDims/2], angle = float(p) * t_j with t_0 = 1 and
 *   t_{j+1} = t_j * powf(thetaBase, -2/nDims), the product taken in float
 *   (GPUComputeUpload.cu:1178-1203). */
int tc_rope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t headDim, float theta);
int tc_mrope_tables(float *cosT, float *sinT, uint32_t rows, uint32_t nDims, float thetaBase);

/* ------------------------------------------------------------------------- */
/* attention-output epilogues                                                  */
/* ------------------------------------------------------------------------- */

/* Replaces kQ35SigmoidGate (include/gpu/GpuQwen35Kernels.hpp:479-493):
 * attnOut[s][h][e] *= sigmoid(qGate[s][h][hd + e]), qGate rows [nHeads][2*hd]. */
int tc_attn_sigmoid_gate(float *attnOut, const float *qGate, uint32_t seqLen,
                         uint32_t nHeads, uint32_t hd, tc_stream stream);

/* ------------------------------------------------------------------------- */
/* context planner (host only, no CUDA)                                        */
/* ------------------------------------------------------------------------- */

enum { TC_KV_F32 = 0, TC_KV_I8 = 1 };

/* POD mirror of tinycoder::detail::ContextRequest (include/ContextPlan.hpp:21-61). */
typedef struct tc_context_request {
    uint32_t requested;          /* 0 = auto (2048) */
    uint32_t modelMax;           /* 0 = unknown (4096 assumed) */
    uint32_t numLayers;
    uint32_t numAttentionLayers; /* layers that own K/V slots */
    uint32_t numKVHeads;
    uint32_t headDim;
    uint32_t ropeDims;           /* cos/sin row width */
    uint32_t int8KvSupported;
    uint32_t forceKv;            /* TC_KV_F32 / TC_KV_I8, honoured when forceKvSet */
    uint32_t forceKvSet;
    uint64_t weightBytes;
    uint64_t freeVram;           /* 0 = no usable GPU */
    uint64_t availableRam;
    uint64_t gpuFixedOverhead;   /* tc_context_request_init sets the default */
} tc_context_request;

/* POD mirror of tinycoder::detail::ContextPlan (include/ContextPlan.hpp:65-72);
 * `reason` is the sentence the engine prints. */
typedef struct tc_context_plan {
    uint32_t seqLen;     /* granted window; 0 = nothing fits */
    uint32_t maxAllowed; /* largest fit of the whole ladder */
    uint32_t kv;         /* TC_KV_F32 / TC_KV_I8 */
    uint32_t kvMirror;   /* f32 store + int8 decode mirror */
    uint32_t kvOnGpu;
    uint32_t reduced;    /* the request was cut to what memory holds */
    uint64_t kvBytes;
    char reason[256];
} tc_context_plan;

void tc_context_request_init(tc_context_request *r);
/* kvBytesPerToken / kvStoreBytesPerToken (src/cpp/core/ContextPlan.cpp:58-78). */
uint64_t tc_kv_bytes_per_token(const tc_context_request *r, uint32_t kv, uint32_t mirror);
uint64_t tc_kv_store_bytes_per_token(const tc_context_request *r, uint32_t kv, uint32_t mirror);
/* planContext (src/cpp/core/ContextPlan.cpp:80-246). */
int tc_context_plan_compute(const tc_context_request *r, tc_context_plan *plan);

/* No counterpart in the reference (it plans for one device).  The same ladder for a KV cache
 * that is partitioned over headParts x ctxParts GPUs: every GPU stores the K/V rows of
 * ceil(numKVHeads / headParts) kv heads and of a 1 / ctxParts share of the window (the two
 * partitions of tc_attn_merge_exchange and of the kv-head split).  The request describes ONE
 * GPU (its free memory, the weight bytes it holds, its fixed overhead); the plan is the one
 * every GPU can honour.  plan.seqLen / maxAllowed are whole-window rows, plan.kvBytes and the
 * fields below are per GPU.  headParts == ctxParts == 1 gives tc_context_plan_compute's plan
 * bit for bit.  A context range shorter than the planner's 1024-row floor is refused like a
 * window shorter than it. */
typedef struct tc_context_shard_plan {
    tc_context_plan plan;
    uint32_t headParts, ctxParts;
    uint32_t kvHeadsPerGpu;
    uint32_t rowsPerGpu;         /* ceil(seqLen / ctxParts), rounded up to 256 rows */
} tc_context_shard_plan;
int tc_context_plan_compute_sharded(const tc_context_request *r, uint32_t headParts, uint32_t ctxParts,
                                    tc_context_shard_plan *out);

/* What this library itself needs next to weights and KV on one GPU, for gpuFixedOverhead (the
 * reference's 1408 MiB default, include/ContextPlan.hpp:58, was measured on its 11 GB cards with
 * its own scratch): the split-KV partial buffers of tc_attn_workspace_bytes at the 512-slot
 * capacity, the exchange buffers of a context split, the fp16 twins of the tensor-core prefill
 * for `prefillChunk`-row calls over the GPU's rows (f32 / fp16 store only), plus
 * `runtimeReserve` bytes for the CUDA context and the caller's allocator slack. */
uint64_t tc_context_overhead_bytes(uint32_t nHeads, uint32_t nKV, uint32_t hd, uint32_t window, uint32_t headParts,
                                   uint32_t ctxParts, int kvStoreI8, uint32_t prefillChunk, uint64_t runtimeReserve);
/* probeFreeVramBytes / probeTotalVramBytes (src/cpp/core/ContextPlan.cpp:248-272)
 * for the current device; 0 when there is none. */
uint64_t tc_probe_free_vram_bytes(void);
uint64_t tc_probe_total_vram_bytes(void);

/* KV pool geometry of one session (src/cpp/core/cuda/forward/GPUComputeUpload.cu:
 * 1254-1323; include/GPUCompute.hpp:844-899): byte sizes the engine allocates. */
typedef struct tc_kv_pool_geometry {
    uint64_t kvLayerStride;   /* bytes of ONE layer's K (or V): maxSeq*nKV*hd*elem */
    uint32_t kvSlots;         /* layers that own a slot */
    uint64_t kvAllocBytes;    /* per K and per V; 0 when int8 is the store */
    uint64_t kv8LayerStride;  /* int8 elements per slot: (maxSeq+16)*nKV*hd */
    uint64_t kv8ScaleStride;  /* bytes of scales per slot: (maxSeq+16)*nKV*4 */
    uint64_t kv8AllocBytes;   /* per K8 and per V8; 0 when no int8 pool */
    uint64_t kv8ScaleAllocBytes;
    uint32_t attnChunk, attnChunks;
    uint64_t partialAccBytes, partialMLBytes;
} tc_kv_pool_geometry;

int tc_kv_pool_geometry_compute(uint32_t maxSeqLen, uint32_t nLayersOnGpu,
                                uint32_t fullAttentionInterval, uint32_t nHeads,
                                uint32_t nKV, uint32_t hd, int kvHalf,
                                int kvStoreI8, int kvMirror,
                                tc_kv_pool_geometry *g);

/* ------------------------------------------------------------------------- */
/* the attention block's host bookkeeping                                       */
/* ------------------------------------------------------------------------- */

/* What GPUModel keeps around its attention kernels
 * (src/cpp/core/cuda/forward/GPUComputeMoE.cu:3013-3200; GPUComputeForward.cu:3778-4040,
 * 3362-3372, 5175-5222; include/GPUCompute.hpp:844-899): the KV mode chosen by
 * the context plan, the per-slot row count of the int8 pool (kv8Rows_), the
 * position and the window guard.  A session owns NO device memory: every buffer
 * below belongs to the caller and is laid out as tc_kv_pool_geometry_compute
 * says ([slot][row][nKV][hd]; int8 pools and scales have maxSeqLen + 16 rows per
 * slot).  One caller and one stream at a time per session. */
typedef struct tc_kv_session tc_kv_session;

typedef struct tc_kv_session_config {
    uint32_t nHeads, nKV, hd;
    uint32_t maxSeqLen;          /* the window (tc_context_plan.seqLen) */
    uint32_t slots;              /* layers that own K/V */
    int kvStoreI8;               /* plan.kv == int8: int8 rows ARE the store, no f32 cache */
    int kvMirror;                /* plan.kvMirror: f32 store + int8 pool for decode */
    int kvHalf;                  /* fp16 store (dense models, opt-in) */
    void *kvK, *kvV;             /* NULL when kvStoreI8 */
    int8_t *kvK8, *kvV8;         /* NULL without an int8 pool */
    float *kvK8Scale, *kvV8Scale;
    float *pAcc, *pM, *pL;       /* split-KV partials for one token */
    uint32_t numChunks;
    const float *ropeCos, *ropeSin; /* dense models: K (and q, in place) rotated in the store; NULL = verbatim */
    void *prefillScratch;        /* optional: lets a fresh prompt on the f32 cache use tc_attn_prefill_f16 */
    size_t prefillScratchBytes;
} tc_kv_session_config;

int tc_kv_session_create(const tc_kv_session_config *cfg, tc_kv_session **out);
void tc_kv_session_destroy(tc_kv_session *s);

/* GPUModel::clearKVCache: f32 / fp16 cache zeroed, every slot's int8 row count
 * and the position reset, "context full" cleared; synchronises the stream. */
int tc_kv_session_clear(tc_kv_session *s, tc_stream stream);

/* GPUModel::forward's window guard: TC_ECONTEXT_FULL (and the sticky flag) when
 * position + newTokens passes the window, before anything is written; else
 * *pos = the position the new rows start at.  tc_kv_session_commit advances the
 * position after the layers have run (kvPos_ += tokens). */
int tc_kv_session_begin(tc_kv_session *s, uint32_t newTokens, uint32_t *pos);
int tc_kv_session_commit(tc_kv_session *s, uint32_t newTokens);
uint32_t tc_kv_session_pos(const tc_kv_session *s);
int tc_kv_session_context_full(const tc_kv_session *s);
uint32_t tc_kv_session_rows8(const tc_kv_session *s, uint32_t slot);

/* One layer's attention block: store the seqLen new K/V rows of `slot` at `pos`
 * and attend.  q [seqLen][nHeads][hd] (rotated in place when the session has
 * rotation tables), kSrc/vSrc [seqLen][nKV][hd] f32, attnOut [seqLen][nHeads][hd].
 *   - one row, int8 pool present, not under graph capture, host position: the
 *     pool first receives the rows a prefill left only in the f32 cache
 *     ([rows8, pos)), then the new row, and the int8 decode kernel runs;
 *   - int8 store, several rows or graph capture: quantise into the pool, causal
 *     attention over it (devPos allowed);
 *   - f32 / fp16 store: append (with rotation if configured), then split-KV
 *     decode (one row) or causal attention (several; a fresh prompt takes the
 *     tensor-core prefill when scratch was given).
 * graphCapture != 0 says the call is being captured: nothing that depends on
 * host-side row counts is chosen. */
int tc_kv_session_attend(tc_kv_session *s, uint32_t slot, float *q, const float *kSrc,
                         const float *vSrc, float *attnOut, uint32_t seqLen, uint32_t pos,
                         const uint32_t *devPos, int graphCapture, tc_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* TC_ATTN_H */
