"""Thin torch-tensor front of the C ABI (one function per entry point).

torch is used for device memory and streams only; every call goes through
libtc_attn.so.  Tensors must live on the current CUDA device and be contiguous.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import capi
from .capi import check, lib


def _ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensor required"
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status(raise_on_flags=True) -> int:
    """Reads and clears the device error word; raises when a kernel reported anything
    (raise_on_flags=False returns the bits instead)."""
    flags = C.c_uint32(0)
    rc = lib.tc_device_status(_stream(), C.byref(flags))
    if rc != capi.TC_EDEVICE or raise_on_flags:
        check(rc)
    return flags.value


# ---- KV writers ---------------------------------------------------------------

def kv_quantize_i8(k, v, k8, v8, ks, vs, tokens, nKV, hd, dst_base=0, src_base=0, dev_dst_base=None,
                   max_rows=None):
    """k, v f32 [rows][nKV][hd] -> rows dst_base.. of the int8 pool k8/v8 + scales ks/vs."""
    if max_rows is None:
        max_rows = k8.numel() // (nKV * hd)
    check(lib.tc_kv_quantize_i8(_ptr(k), _ptr(v), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), tokens, nKV, hd,
                                dst_base, src_base, _ptr(dev_dst_base), max_rows, _stream()))


def kv_quantize_i8_batch(k, v, k8, v8, ks, vs, batch, nKV, hd, rows_per_seq=0, row_base=None, pos=0, lens=None,
                         len_add=0, total_rows=None):
    """The new token of every sequence of a batch into one pool, one launch."""
    total = k8.numel() // (nKV * hd) if total_rows is None else total_rows
    check(lib.tc_kv_quantize_i8_batch(_ptr(k), _ptr(v), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), batch, nKV, hd,
                                      rows_per_seq, _ptr(row_base), pos, _ptr(lens), len_add, total, _stream()))


def kv_append(kSrc, vSrc, kDst, vDst, seqLen, nKV, hd, cachePos, dev_pos=None, max_rows=None):
    half = kDst.dtype == torch.float16
    if max_rows is None:
        max_rows = kDst.numel() // (nKV * hd)
    check(lib.tc_kv_append(_ptr(kSrc), _ptr(vSrc), _ptr(kDst), _ptr(vDst), int(half), seqLen, nKV, hd, cachePos,
                           _ptr(dev_pos), max_rows, _stream()))


def kv_append_rope(q, kSrc, vSrc, kDst, vDst, seqLen, nHeads, nKV, hd, cachePos, ropePos, cosT, sinT,
                   dev_pos=None):
    half = kDst.dtype == torch.float16
    max_rows = kDst.numel() // (nKV * hd)
    check(lib.tc_kv_append_rope(_ptr(q), _ptr(kSrc), _ptr(vSrc), _ptr(kDst), _ptr(vDst), int(half), seqLen,
                                nHeads, nKV, hd, cachePos, ropePos, _ptr(dev_pos), _ptr(cosT), _ptr(sinT),
                                max_rows, _stream()))


def qk_norm_rope(qIn, qOut, k, wq, wk, hd, nDims, nHeads, nKV, seqLen, pos, cosT, sinT, dev_pos=None,
                 q_in_stride=None):
    """Per-head RMSNorm of q (out of place, rows of stride q_in_stride) and k (in place) + partial rotation."""
    stride = (2 * hd if q_in_stride is None else q_in_stride) if qIn is not None else 0
    rows = cosT.numel() // max(1, nDims // 2)
    check(lib.tc_qk_norm_rope(_ptr(qIn), stride, _ptr(qOut), _ptr(k), _ptr(wq), _ptr(wk), hd, nDims, nHeads, nKV,
                              seqLen, pos, _ptr(dev_pos), _ptr(cosT), _ptr(sinT), rows, _stream()))


def rope_tables(rows, headDim, theta):
    """Host: the engine's NEOX tables [rows][headDim/2] (numpy float32 pair)."""
    import numpy as np
    c = np.zeros((rows, headDim // 2), np.float32)
    s = np.zeros_like(c)
    check(lib.tc_rope_tables(c.ctypes.data, s.ctypes.data, rows, headDim, theta))
    return c, s


def mrope_tables(rows, nDims, thetaBase):
    import numpy as np
    c = np.zeros((rows, nDims // 2), np.float32)
    s = np.zeros_like(c)
    check(lib.tc_mrope_tables(c.ctypes.data, s.ctypes.data, rows, nDims, thetaBase))
    return c, s


def rope_q(q, cosT, sinT, seqLen, nHeads, hd, pos, dev_pos=None):
    check(lib.tc_rope_q(_ptr(q), _ptr(cosT), _ptr(sinT), seqLen, nHeads, hd, pos, _ptr(dev_pos), _stream()))


# ---- decode -------------------------------------------------------------------

def workspace(batch, nHeads, hd, numChunks, device=None):
    a, m, l = C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(lib.tc_attn_workspace_bytes(batch, nHeads, hd, numChunks, C.byref(a), C.byref(m), C.byref(l)))
    dev = device or torch.device("cuda", torch.cuda.current_device())
    return (torch.empty(a.value // 4, dtype=torch.float32, device=dev),
            torch.empty(m.value // 4, dtype=torch.float32, device=dev),
            torch.empty(l.value // 4, dtype=torch.float32, device=dev))


def split_geometry(maxSeqLen, nHeads, hd):
    a, b = C.c_uint32(), C.c_uint32()
    rc = lib.tc_split_geometry(maxSeqLen, nHeads, hd, C.byref(a), C.byref(b))
    check(rc)
    return a.value, b.value


def decode_i8(q, k8, v8, ks, vs, out, ws, nHeads, nKV, hd, cachePos, numChunks, chunkSize=0, invSqrt=None,
              dev_pos=None):
    """One query token over rows [0, cachePos] of an int8 store."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    total_rows = k8.numel() // (nKV * hd)
    pAcc, pM, pL = ws
    check(lib.tc_attn_decode_i8(_ptr(q), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), _ptr(out), _ptr(pAcc),
                                _ptr(pM), _ptr(pL), nHeads, nKV, hd, cachePos, _ptr(dev_pos), total_rows,
                                numChunks, chunkSize, invSqrt, _stream()))


def decode_i8_noalloc(q, k8, v8, ks, vs, out, nHeads, nKV, hd, cachePos, invSqrt=None):
    """tc_attn_decode_i8 without caller scratch: the partials live in an array inside the
    library (for callers that cannot allocate device memory)."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    total_rows = k8.numel() // (nKV * hd)
    check(lib.tc_attn_decode_i8_noalloc(_ptr(q), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), _ptr(out), nHeads, nKV,
                                        hd, cachePos, total_rows, invSqrt, _stream()))


def decode_i8_batch(q, k8, v8, ks, vs, out, ws, lens, batch, nHeads, nKV, hd, maxLen, numChunks,
                    rows_per_seq=0, row_base=None, invSqrt=None, partials_only=False, pdl=False,
                    prefetch_rows=0, next_kv=None, tickets=None, append=None):
    """`batch` sequences in one pool; returns the chunk slots used per head.
    lens=None: every sequence is maxLen rows long (host length).
    append=(k, v): f32 [batch][nKV][hd] rows of the new token, quantised into row len - 1 of every
    sequence by the launch itself."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    pAcc, pM, pL = ws
    used = C.c_uint32(0)
    d = capi.DecodeI8Batch()
    d.q, d.out = q.data_ptr(), out.data_ptr()
    d.k8, d.v8, d.ks, d.vs = k8.data_ptr(), v8.data_ptr(), ks.data_ptr(), vs.data_ptr()
    d.pAcc, d.pM, d.pL = pAcc.data_ptr(), pM.data_ptr(), pL.data_ptr()
    d.lens = lens.data_ptr() if lens is not None else None
    d.flags = capi.TC_DECODE_PDL if pdl else 0
    d.prefetchRows = prefetch_rows
    if next_kv is not None:
        d.nextK8, d.nextV8 = next_kv[0].data_ptr(), next_kv[1].data_ptr()
    if tickets is not None:      # zeroed uint32 [batch * nKV]: the kernel merges its own partials
        assert tickets.dtype == torch.int32 and tickets.numel() >= batch * nKV
        d.mergeTickets = tickets.data_ptr()
    if append is not None:
        d.appendK, d.appendV = append[0].data_ptr(), append[1].data_ptr()
    d.rowBase = row_base.data_ptr() if row_base is not None else None
    d.rowsPerSeq = rows_per_seq
    d.totalRows = k8.numel() // (nKV * hd)
    d.batch, d.nHeads, d.nKV, d.hd = batch, nHeads, nKV, hd
    d.maxLen, d.numChunks = maxLen, numChunks
    d.invSqrt = invSqrt
    d.partialsOnly = int(partials_only)
    d.chunksUsed = C.pointer(used)
    check(lib.tc_attn_decode_i8_batch(C.byref(d), _stream()))
    return used.value


def decode_kv(q, kvK, kvV, out, ws, seqLen, nHeads, nKV, hd, pos, numChunks, chunkSize=0, invSqrt=None,
              dev_pos=None, q81=None):
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    half = kvK.dtype == torch.float16
    total_rows = kvK.numel() // (nKV * hd)
    pAcc, pM, pL = ws
    check(lib.tc_attn_decode_kv(_ptr(q), _ptr(kvK), _ptr(kvV), _ptr(out), _ptr(pAcc), _ptr(pM), _ptr(pL),
                                seqLen, nHeads, nKV, hd, pos, _ptr(dev_pos), total_rows, numChunks, chunkSize,
                                invSqrt, int(half), _ptr(q81), _stream()))


def merge_partials(pAcc, pM, pL, out, seqLen, nHeads, numChunks, hd, q81=None):
    check(lib.tc_attn_merge_partials(_ptr(pAcc), _ptr(pM), _ptr(pL), _ptr(out), seqLen, nHeads, numChunks, hd,
                                     _ptr(q81), _stream()))


def merge_gathered(gathered, out, nHeads, ranks, chunksPerRank, hd):
    """Merge the all-gathered [acc | m | l] blocks of `ranks` context shards."""
    check(lib.tc_attn_merge_gathered(_ptr(gathered), _ptr(out), nHeads, ranks, chunksPerRank, hd, _stream()))


def exchange_bytes(nHeads, hd, world):
    n = C.c_size_t(0)
    check(lib.tc_attn_exchange_bytes(nHeads, hd, world, C.byref(n)))
    return n.value


def merge_exchange(ws, out, nHeads, numChunks, activeChunks, hd, buffer_ptrs, rank, pdl=False):
    """Merge this rank's chunk partials, exchange with the peers inside the kernel, write out.
    buffer_ptrs: device addresses of every rank's exchange buffer as seen from this rank."""
    g = capi.PeerGroup()
    for r, ptr in enumerate(buffer_ptrs):
        g.buffers[r] = ptr
    g.world, g.rank = len(buffer_ptrs), rank
    pAcc, pM, pL = ws
    check(lib.tc_attn_merge_exchange(_ptr(pAcc), _ptr(pM), _ptr(pL), _ptr(out), nHeads, numChunks, activeChunks, hd,
                                     C.byref(g), capi.TC_DECODE_PDL if pdl else 0, _stream()))


def merge_exchange_local(wss, outs, buffers, nHeads, numChunks, activeChunks, hd):
    """All ranks of the exchange protocol in one cooperative launch on this GPU."""
    n = len(wss)
    arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() for t in ts])  # noqa: E731
    check(lib.tc_attn_merge_exchange_local(arr([w[0] for w in wss]), arr([w[1] for w in wss]),
                                           arr([w[2] for w in wss]), arr(outs), arr(buffers), n, nHeads, numChunks,
                                           activeChunks, hd, _stream()))


# ---- prefill ------------------------------------------------------------------

def prefill_f16_scratch_bytes(seqLen, nHeads, nKV, hd, cachePos=0) -> int:
    b = C.c_size_t()
    check(lib.tc_attn_prefill_f16_scratch_bytes(seqLen, cachePos, nHeads, nKV, hd, C.byref(b)))
    return b.value


def prefill_f16(q, kvK, kvV, out, scratch, seqLen, nHeads, nKV, hd, invSqrt=None, cachePos=0, kv8=None, kv8_row=None):
    """seqLen query rows at positions cachePos.. over cache rows [0, cachePos + seqLen) of kvK / kvV.
    kv8 = (k8, v8, ks, vs): also write the int8 rows of the new positions into that pool, from row
    kv8_row (default cachePos) on."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    if kv8 is not None:
        k8, v8, ks, vs = kv8
        check(lib.tc_attn_prefill_f16_kv8(_ptr(q), _ptr(kvK), _ptr(kvV), _ptr(out), _ptr(scratch),
                                          scratch.numel() * scratch.element_size(), seqLen, cachePos, nHeads, nKV, hd,
                                          invSqrt, _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs),
                                          cachePos if kv8_row is None else kv8_row, ks.numel() // nKV, _stream()))
        return
    check(lib.tc_attn_prefill_f16(_ptr(q), _ptr(kvK), _ptr(kvV), _ptr(out), _ptr(scratch),
                                  scratch.numel() * scratch.element_size(), seqLen, cachePos, nHeads, nKV, hd,
                                  invSqrt, _stream()))


def prefill_f16_kvhalf(q, kvK16, kvV16, out, scratch, seqLen, nHeads, nKV, hd, invSqrt=None, cachePos=0):
    """The tcgen05 prefill over an fp16 store (read in place; the scratch holds q's twin only)."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    check(lib.tc_attn_prefill_f16_kvhalf(_ptr(q), _ptr(kvK16), _ptr(kvV16), _ptr(out), _ptr(scratch),
                                         scratch.numel() * scratch.element_size(), seqLen, cachePos, nHeads, nKV, hd,
                                         invSqrt, _stream()))


def prefill_f16_i8(q, k8, v8, ks, vs, out, scratch, seqLen, nHeads, nKV, hd, invSqrt=None, cachePos=0):
    """The tcgen05 prefill over an int8 store whose rows [0, cachePos + seqLen) are written."""
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    check(lib.tc_attn_prefill_f16_i8(_ptr(q), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), _ptr(out), _ptr(scratch),
                                     scratch.numel() * scratch.element_size(), seqLen, cachePos, nHeads, nKV, hd,
                                     invSqrt, _stream()))


def prefill_kv(q, kvK, kvV, out, seqLen, nHeads, nKV, hd, cachePos, invSqrt=None, dev_pos=None):
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    half = kvK.dtype == torch.float16
    total_rows = kvK.numel() // (nKV * hd)
    check(lib.tc_attn_prefill_kv(_ptr(q), _ptr(kvK), _ptr(kvV), _ptr(out), seqLen, nHeads, nKV, hd, cachePos,
                                 _ptr(dev_pos), total_rows, invSqrt, int(half), _stream()))


def prefill_i8(q, k8, v8, ks, vs, out, seqLen, nHeads, nKV, hd, cachePos, invSqrt=None, dev_pos=None):
    if invSqrt is None:
        invSqrt = 1.0 / math.sqrt(hd)
    total_rows = k8.numel() // (nKV * hd)
    check(lib.tc_attn_prefill_i8(_ptr(q), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs), _ptr(out), seqLen, nHeads,
                                 nKV, hd, cachePos, _ptr(dev_pos), total_rows, invSqrt, _stream()))


def sigmoid_gate(attnOut, qGate, seqLen, nHeads, hd):
    check(lib.tc_attn_sigmoid_gate(_ptr(attnOut), _ptr(qGate), seqLen, nHeads, hd, _stream()))


# ---- planner (host) -------------------------------------------------------------

def context_request(**kw) -> capi.ContextRequest:
    r = capi.ContextRequest()
    lib.tc_context_request_init(C.byref(r))
    for k, v in kw.items():
        setattr(r, k, int(v))
    return r


def plan_context(req: capi.ContextRequest) -> dict:
    p = capi.ContextPlan()
    check(lib.tc_context_plan_compute(C.byref(req), C.byref(p)))
    return p.as_dict()


def plan_context_sharded(req: capi.ContextRequest, head_parts: int, ctx_parts: int) -> dict:
    """The plan every GPU of a head_parts x ctx_parts partition can honour (req describes one GPU)."""
    p = capi.ContextShardPlan()
    check(lib.tc_context_plan_compute_sharded(C.byref(req), head_parts, ctx_parts, C.byref(p)))
    d = p.plan.as_dict()
    d.update(headParts=p.headParts, ctxParts=p.ctxParts, kvHeadsPerGpu=p.kvHeadsPerGpu, rowsPerGpu=p.rowsPerGpu)
    return d


def context_overhead_bytes(nHeads, nKV, hd, window, head_parts=1, ctx_parts=1, kv_store_i8=True, prefill_chunk=512,
                           runtime_reserve=512 << 20) -> int:
    return int(lib.tc_context_overhead_bytes(nHeads, nKV, hd, window, head_parts, ctx_parts, int(kv_store_i8),
                                             prefill_chunk, runtime_reserve))


def kv_bytes_per_token(req, kv, mirror) -> int:
    return int(lib.tc_kv_bytes_per_token(C.byref(req), int(kv), int(mirror)))


def kv_store_bytes_per_token(req, kv, mirror) -> int:
    return int(lib.tc_kv_store_bytes_per_token(C.byref(req), int(kv), int(mirror)))


def kv_pool_geometry(maxSeqLen, nLayersOnGpu, fullAttentionInterval, nHeads, nKV, hd, kvHalf=False,
                     kvStoreI8=False, kvMirror=False) -> capi.KvPoolGeometry:
    g = capi.KvPoolGeometry()
    check(lib.tc_kv_pool_geometry_compute(maxSeqLen, nLayersOnGpu, fullAttentionInterval, nHeads, nKV, hd,
                                          int(kvHalf), int(kvStoreI8), int(kvMirror), C.byref(g)))
    return g


# ---- the attention block's host bookkeeping ----------------------------------------

class KvSession:
    """tc_kv_session over torch-allocated pools (what GPUModel holds around its attention
    kernels): mode = "f32" | "f32+i8" (f32 store, int8 decode pool) | "i8" (int8 store) | "f16"."""

    def __init__(self, nHeads, nKV, hd, max_seq, slots, mode="f32", rope=None, prefill_scratch_rows=0, chunks=None):
        self.nH, self.nKV, self.hd, self.max_seq, self.slots, self.mode = nHeads, nKV, hd, max_seq, slots, mode
        store_i8, mirror, half = mode == "i8", mode == "f32+i8", mode == "f16"
        g = kv_pool_geometry(max_seq, slots, 1, nHeads, nKV, hd, half, store_i8, mirror)
        self.geom = g
        dev = "cuda"
        cfg = capi.KvSessionConfig()
        cfg.nHeads, cfg.nKV, cfg.hd, cfg.maxSeqLen, cfg.slots = nHeads, nKV, hd, max_seq, slots
        cfg.kvStoreI8, cfg.kvMirror, cfg.kvHalf = int(store_i8), int(mirror), int(half)
        self._keep = []
        if not store_i8:
            dt = torch.float16 if half else torch.float32
            self.kvK = torch.zeros((slots, max_seq, nKV, hd), dtype=dt, device=dev)
            self.kvV = torch.zeros_like(self.kvK)
            cfg.kvK, cfg.kvV = self.kvK.data_ptr(), self.kvV.data_ptr()
        if store_i8 or mirror:
            # stale bytes on purpose: the bookkeeping, not a memset, keeps old rows out
            self.k8 = torch.full((slots, max_seq + 16, nKV, hd), 77, dtype=torch.int8, device=dev)
            self.v8 = torch.full_like(self.k8, -55)
            self.ks = torch.full((slots, max_seq + 16, nKV), float("nan"), device=dev)
            self.vs = torch.full_like(self.ks, float("nan"))
            cfg.kvK8, cfg.kvV8 = self.k8.data_ptr(), self.v8.data_ptr()
            cfg.kvK8Scale, cfg.kvV8Scale = self.ks.data_ptr(), self.vs.data_ptr()
        self.chunks = chunks or g.attnChunks
        self.ws = workspace(1, nHeads, hd, self.chunks)
        cfg.pAcc, cfg.pM, cfg.pL = (w.data_ptr() for w in self.ws)
        cfg.numChunks = self.chunks
        if rope is not None:
            self._keep += list(rope)
            cfg.ropeCos, cfg.ropeSin = rope[0].data_ptr(), rope[1].data_ptr()
        if prefill_scratch_rows:
            # room for the fp16 twins of `prefill_scratch_rows` query rows over the whole window
            n = prefill_f16_scratch_bytes(prefill_scratch_rows, nHeads, nKV, hd, cachePos=max(0, max_seq - prefill_scratch_rows))
            buf = torch.empty(n + 1024, dtype=torch.uint8, device=dev)
            off = (-buf.data_ptr()) % 1024
            self._keep.append(buf)
            cfg.prefillScratch, cfg.prefillScratchBytes = buf.data_ptr() + off, n
        self.cfg = cfg
        h = C.c_void_p()
        check(lib.tc_kv_session_create(C.byref(cfg), C.byref(h)))
        self.h = h

    def __del__(self):
        if getattr(self, "h", None):
            lib.tc_kv_session_destroy(self.h)
            self.h = None

    def clear(self):
        check(lib.tc_kv_session_clear(self.h, _stream()))

    def begin(self, n):
        pos = C.c_uint32(0)
        check(lib.tc_kv_session_begin(self.h, n, C.byref(pos)))
        return pos.value

    def commit(self, n):
        check(lib.tc_kv_session_commit(self.h, n))

    @property
    def pos(self):
        return lib.tc_kv_session_pos(self.h)

    @property
    def context_full(self):
        return bool(lib.tc_kv_session_context_full(self.h))

    def rows8(self, slot):
        return lib.tc_kv_session_rows8(self.h, slot)

    def attend(self, slot, q, k, v, out, pos, dev_pos=None, graph_capture=False):
        seqLen = q.shape[0]
        check(lib.tc_kv_session_attend(self.h, slot, _ptr(q), _ptr(k), _ptr(v), _ptr(out), seqLen, pos, _ptr(dev_pos),
                                       int(graph_capture), _stream()))
