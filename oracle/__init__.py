"""ctypes binding of the CPU checker (oracle/tc_oracle.c, oracle/ref_shim.cpp).

TEST INFRASTRUCTURE ONLY.  Importable from tests/, from the smoke check and from
the bench's CPU-baseline / reference arm; the shipped package never imports it.

All arrays are C-contiguous numpy arrays; functions return new arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtc_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libtc_ref.so")


def build(ref: bool = True) -> None:
    """Compile the restatement (always) and the reference-built library (when
    the reference checkout is present; otherwise a prebuilt one is kept)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    if ref:
        subprocess.run(["make", "-s", "-C", _HERE, "ref"], check=True)


def _load():
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "tc_oracle.c")
    ):
        build(ref=False)
    return C.CDLL(_LIB_PATH)


_lib = _load()

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_i8p = C.POINTER(C.c_int8)
_u8p = C.POINTER(C.c_uint8)
_u32p = C.POINTER(C.c_uint32)


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


class ContextRequest(C.Structure):
    _fields_ = [
        ("requested", C.c_uint32),
        ("modelMax", C.c_uint32),
        ("numLayers", C.c_uint32),
        ("numAttentionLayers", C.c_uint32),
        ("numKVHeads", C.c_uint32),
        ("headDim", C.c_uint32),
        ("ropeDims", C.c_uint32),
        ("int8KvSupported", C.c_uint32),
        ("forceKv", C.c_uint32),
        ("forceKvSet", C.c_uint32),
        ("weightBytes", C.c_uint64),
        ("freeVram", C.c_uint64),
        ("availableRam", C.c_uint64),
        ("gpuFixedOverhead", C.c_uint64),
    ]


class ContextPlan(C.Structure):
    _fields_ = [
        ("seqLen", C.c_uint32),
        ("maxAllowed", C.c_uint32),
        ("kv", C.c_uint32),
        ("kvMirror", C.c_uint32),
        ("kvOnGpu", C.c_uint32),
        ("reduced", C.c_uint32),
        ("kvBytes", C.c_uint64),
        ("reason", C.c_char * 256),
    ]

    def as_dict(self):
        return {
            "seqLen": self.seqLen,
            "maxAllowed": self.maxAllowed,
            "kv": self.kv,
            "kvMirror": self.kvMirror,
            "kvOnGpu": self.kvOnGpu,
            "reduced": self.reduced,
            "kvBytes": self.kvBytes,
            "reason": self.reason.decode(),
        }


DEFAULT_GPU_FIXED_OVERHEAD = 1408 << 20  # include/ContextPlan.hpp:58


def make_request(**kw) -> ContextRequest:
    r = ContextRequest()
    r.gpuFixedOverhead = DEFAULT_GPU_FIXED_OVERHEAD
    for k, v in kw.items():
        setattr(r, k, int(v))
    return r


# ---- quantiser ---------------------------------------------------------------

def quant_kv8(k, v, nKV, hd, dst_base=0, src_base=0, tokens=None, out=None):
    """kQ35QuantKV8.  k, v: f32 [rows][nKV][hd].  Returns (k8, v8, ks, vs) sized
    dst_base + tokens rows unless `out` (k8, v8, ks, vs) is given to append into."""
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    if tokens is None:
        tokens = k.size // (nKV * hd) - src_base
    if out is None:
        rows = dst_base + tokens
        k8 = np.zeros((rows, nKV, hd), np.int8)
        v8 = np.zeros((rows, nKV, hd), np.int8)
        ks = np.zeros((rows, nKV), np.float32)
        vs = np.zeros((rows, nKV), np.float32)
    else:
        k8, v8, ks, vs = out
    _lib.orc_quant_kv8(_p(k, _f32p), _p(v, _f32p), _p(k8, _i8p), _p(v8, _i8p), _p(ks, _f32p),
                       _p(vs, _f32p), C.c_uint32(tokens), C.c_uint32(nKV), C.c_uint32(hd),
                       C.c_uint64(dst_base), C.c_uint64(src_base))
    return k8, v8, ks, vs


# ---- int8 attention ----------------------------------------------------------

def decode_i8_split(q, k8, v8, ks, vs, nHeads, nKV, hd, cachePos, numChunks, chunkSize, invSqrt):
    q = _c(q, np.float32)
    acc = np.zeros((nHeads, numChunks, hd), np.float32)
    m = np.zeros((nHeads, numChunks), np.float32)
    l = np.zeros((nHeads, numChunks), np.float32)
    _lib.orc_decode_i8_split(_p(q, _f32p), _p(k8, _i8p), _p(v8, _i8p), _p(ks, _f32p), _p(vs, _f32p),
                             _p(acc, _f32p), _p(m, _f32p), _p(l, _f32p), C.c_uint32(nHeads),
                             C.c_uint32(nKV), C.c_uint32(cachePos), C.c_uint32(numChunks),
                             C.c_uint32(chunkSize), C.c_uint32(hd), C.c_float(invSqrt))
    return acc, m, l


def attention_i8(q, k8, v8, ks, vs, seqLen, nHeads, nKV, hd, cachePos, invSqrt):
    q = _c(q, np.float32)
    out = np.zeros((seqLen, nHeads, hd), np.float32)
    _lib.orc_attention_i8(_p(q, _f32p), _p(k8, _i8p), _p(v8, _i8p), _p(ks, _f32p), _p(vs, _f32p),
                          _p(out, _f32p), C.c_uint32(seqLen), C.c_uint32(nHeads), C.c_uint32(nKV),
                          C.c_uint32(cachePos), C.c_uint32(hd), C.c_float(invSqrt))
    return out


def combine_partials(acc, m, l, seqLen, nHeads, numChunks, hd):
    acc = _c(acc, np.float32)
    m = _c(m, np.float32)
    l = _c(l, np.float32)
    out = np.zeros((seqLen, nHeads, hd), np.float32)
    _lib.orc_combine_partials(_p(acc, _f32p), _p(m, _f32p), _p(l, _f32p), _p(out, _f32p),
                              C.c_uint32(seqLen), C.c_uint32(nHeads), C.c_uint32(numChunks),
                              C.c_uint32(hd))
    return out


# ---- f32 / fp16 KV attention -------------------------------------------------

def _kv_ptr(a):
    return C.c_void_p(a.ctypes.data)


def decode_kv_split(q, kc, vc, seqLen, nHeads, nKV, hd, cachePos, numChunks, chunkSize, invSqrt):
    """kWarpAttentionSplit.  kc/vc: float32 or float16 arrays [rows][nKV][hd]."""
    q = _c(q, np.float32)
    half = kc.dtype == np.float16
    acc = np.zeros((seqLen, nHeads, numChunks, hd), np.float32)
    m = np.zeros((seqLen, nHeads, numChunks), np.float32)
    l = np.zeros((seqLen, nHeads, numChunks), np.float32)
    _lib.orc_decode_kv_split(_p(q, _f32p), _kv_ptr(kc), _kv_ptr(vc), C.c_int(int(half)), _p(acc, _f32p),
                             _p(m, _f32p), _p(l, _f32p), C.c_uint32(seqLen), C.c_uint32(nHeads),
                             C.c_uint32(nKV), C.c_uint32(cachePos), C.c_uint32(numChunks),
                             C.c_uint32(chunkSize), C.c_uint32(hd), C.c_float(invSqrt))
    return acc, m, l


def attention_kv(q, kc, vc, seqLen, nHeads, nKV, hd, cachePos, invSqrt):
    """kWarpAttention (unsplit causal)."""
    q = _c(q, np.float32)
    half = kc.dtype == np.float16
    out = np.zeros((seqLen, nHeads, hd), np.float32)
    _lib.orc_attention_kv(_p(q, _f32p), _kv_ptr(kc), _kv_ptr(vc), C.c_int(int(half)), _p(out, _f32p),
                          C.c_uint32(seqLen), C.c_uint32(nHeads), C.c_uint32(nKV), C.c_uint32(cachePos),
                          C.c_uint32(hd), C.c_float(invSqrt))
    return out


def attention_fused_cpu(q, kc, vc, seqLen, cachePos, nHeads, nKV, hd):
    """Model::attentionFused (CPU engine)."""
    q = _c(q, np.float32)
    kc = _c(kc, np.float32)
    vc = _c(vc, np.float32)
    out = np.zeros((seqLen, nHeads, hd), np.float32)
    _lib.orc_attention_fused_cpu(_p(q, _f32p), _p(kc, _f32p), _p(vc, _f32p), _p(out, _f32p),
                                 C.c_uint32(seqLen), C.c_uint32(cachePos), C.c_uint32(nHeads),
                                 C.c_uint32(nKV), C.c_uint32(hd))
    return out


def attention_f64(q, kc, vc, ks, vs, seqLen, nHeads, nKV, hd, cachePos, scale):
    """Double-precision causal attention.  kc/vc dtype selects f32 / fp16 / int8."""
    q = _c(q, np.float32)
    kind = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.int8): 2}[kc.dtype]
    out = np.zeros((seqLen, nHeads, hd), np.float64)
    ksp = _p(ks, _f32p) if ks is not None else None
    vsp = _p(vs, _f32p) if vs is not None else None
    _lib.orc_attention_f64(_p(q, _f32p), _kv_ptr(kc), _kv_ptr(vc), ksp, vsp, C.c_int(kind),
                           _p(out, _f64p), C.c_uint32(seqLen), C.c_uint32(nHeads), C.c_uint32(nKV),
                           C.c_uint32(cachePos), C.c_uint32(hd), C.c_double(scale))
    return out


def prefill_f16(q, k, v, S, nHeads, nKV, hd, scale):
    """Materialised fp16 prefill (cuBLAS detour semantics)."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    out = np.zeros((S, nHeads, hd), np.float32)
    _lib.orc_prefill_f16(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(out, _f32p), C.c_uint32(S),
                         C.c_uint32(nHeads), C.c_uint32(nKV), C.c_uint32(hd), C.c_float(scale))
    return out


def prefill_f16_rows(q, k, v, rows, S, nHeads, nKV, hd, scale, cachePos=0):
    """The same contract for a sample of query rows (indices into q's S rows) over a cache that
    already holds cachePos rows: k, v are [cachePos + S][nKV][hd]; returns [len(rows)][nHeads][hd]."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    rows = _c(rows, np.uint32)
    out = np.zeros((rows.size, nHeads, hd), np.float32)
    _lib.orc_prefill_f16_rows(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(out, _f32p), _p(rows, _u32p),
                              C.c_uint32(rows.size), C.c_uint32(S), C.c_uint32(cachePos), C.c_uint32(nHeads),
                              C.c_uint32(nKV), C.c_uint32(hd), C.c_float(scale))
    return out


# ---- RoPE / append -----------------------------------------------------------

def rope_tables(rows, headDim, theta):
    cosT = np.zeros((rows, headDim // 2), np.float32)
    sinT = np.zeros((rows, headDim // 2), np.float32)
    _lib.orc_rope_tables(_p(cosT, _f32p), _p(sinT, _f32p), C.c_uint32(rows), C.c_uint32(headDim),
                         C.c_float(theta))
    return cosT, sinT


def rope_q(q, cosT, sinT, seqLen, qHeads, headDim, pos):
    q = np.array(q, dtype=np.float32, copy=True, order="C")
    _lib.orc_rope_q(_p(q, _f32p), _p(cosT, _f32p), _p(sinT, _f32p), C.c_uint32(seqLen),
                    C.c_uint32(qHeads), C.c_uint32(headDim), C.c_uint32(pos))
    return q


def kv_append(kSrc, vSrc, kDst, vDst, seqLen, nKV, headDim, cachePos, ropePos=0, cosT=None, sinT=None):
    """kStoreKVRope / kQ35StoreKV into kDst/vDst (float32 or float16 arrays, in place)."""
    kSrc = _c(kSrc, np.float32)
    vSrc = _c(vSrc, np.float32)
    half = kDst.dtype == np.float16
    _lib.orc_kv_append(_p(kSrc, _f32p), _p(vSrc, _f32p), _kv_ptr(kDst), _kv_ptr(vDst), C.c_int(int(half)),
                       C.c_uint32(seqLen), C.c_uint32(nKV), C.c_uint32(headDim), C.c_uint32(cachePos),
                       C.c_uint32(ropePos), _p(cosT, _f32p) if cosT is not None else None,
                       _p(sinT, _f32p) if sinT is not None else None)


def kv_append_cpu(kSrc, vSrc, kDst, vDst, seqLen, cachePos, kHeads, headDim, cosT, sinT):
    kSrc = _c(kSrc, np.float32)
    vSrc = _c(vSrc, np.float32)
    _lib.orc_kv_append_cpu(_p(kSrc, _f32p), _p(vSrc, _f32p), _p(kDst, _f32p), _p(vDst, _f32p),
                           C.c_uint32(seqLen), C.c_uint32(cachePos), C.c_uint32(kHeads),
                           C.c_uint32(headDim), _p(cosT, _f32p), _p(sinT, _f32p))


def q8_1_blocks(x):
    x = _c(x, np.float32).reshape(-1)
    n = x.size // 32
    out = np.zeros(n * 40, np.uint8)
    _lib.orc_q8_1_blocks(_p(x, _f32p), _p(out, _u8p), C.c_uint64(n))
    return out


def sigmoid_gate(attnOut, qGate, seqLen, nHeads, hd):
    o = np.array(attnOut, dtype=np.float32, copy=True, order="C")
    g = _c(qGate, np.float32)
    _lib.orc_sigmoid_gate(_p(o, _f32p), _p(g, _f32p), C.c_uint32(seqLen), C.c_uint32(nHeads),
                          C.c_uint32(hd))
    return o


def norm_rope(x, w, hd, nDims, heads, seqLen, pos, cosT, sinT, in_stride=None):
    """kQ35QNormRoPE (in_stride = 2*hd, q then gate per head) / kQ35KNormRoPE (in_stride = hd)."""
    in_stride = hd if in_stride is None else in_stride
    xin = _c(x, np.float32)
    out = np.zeros((seqLen, heads, hd), np.float32)
    _lib.orc_norm_rope(_p(xin, _f32p), C.c_uint32(in_stride), _p(out, _f32p), _p(_c(w, np.float32), _f32p),
                       C.c_uint32(hd), C.c_uint32(nDims), C.c_uint32(heads), C.c_uint32(seqLen), C.c_uint32(pos),
                       _p(_c(cosT, np.float32), _f32p), _p(_c(sinT, np.float32), _f32p))
    return out


def mrope_tables(rows, nDims, thetaBase):
    cosT = np.zeros((rows, nDims // 2), np.float32)
    sinT = np.zeros((rows, nDims // 2), np.float32)
    _lib.orc_mrope_tables(_p(cosT, _f32p), _p(sinT, _f32p), C.c_uint32(rows), C.c_uint32(nDims),
                          C.c_float(thetaBase))
    return cosT, sinT


# ---- planner -----------------------------------------------------------------

_lib.orc_kv_bytes_per_token.restype = C.c_uint64
_lib.orc_kv_store_bytes_per_token.restype = C.c_uint64


def kv_bytes_per_token(req: ContextRequest, i8: bool, mirror: bool) -> int:
    return int(_lib.orc_kv_bytes_per_token(C.byref(req), C.c_int(int(i8)), C.c_int(int(mirror))))


def kv_store_bytes_per_token(req: ContextRequest, i8: bool, mirror: bool) -> int:
    return int(_lib.orc_kv_store_bytes_per_token(C.byref(req), C.c_int(int(i8)), C.c_int(int(mirror))))


def plan_context(req: ContextRequest) -> dict:
    p = ContextPlan()
    _lib.orc_plan_context(C.byref(req), C.byref(p))
    return p.as_dict()


def split_geometry(maxSeqLen, nHeads, headDim):
    a = C.c_uint32()
    b = C.c_uint32()
    _lib.orc_split_geometry(C.c_uint32(maxSeqLen), C.c_uint32(nHeads), C.c_uint32(headDim), C.byref(a),
                            C.byref(b))
    return a.value, b.value


# ---- reference-built library (oracle/_ref) -----------------------------------

class _Ref:
    """The reference project's own compiled planner, thread pool and AVX-512
    leaves behind ref_shim.cpp.  Present only where `make -C oracle ref` ran
    (or its output travelled with the tree)."""

    def __init__(self):
        self.lib = C.CDLL(_REF_PATH)
        self.lib.ref_kv_bytes_per_token.restype = C.c_uint64
        self.lib.ref_kv_store_bytes_per_token.restype = C.c_uint64
        self.lib.ref_default_gpu_fixed_overhead.restype = C.c_uint64
        self.lib.ref_pool_init.restype = C.c_uint32

    def default_overhead(self) -> int:
        return int(self.lib.ref_default_gpu_fixed_overhead())

    def kv_bytes_per_token(self, req, i8, mirror) -> int:
        return int(self.lib.ref_kv_bytes_per_token(C.byref(req), C.c_int(int(i8)), C.c_int(int(mirror))))

    def kv_store_bytes_per_token(self, req, i8, mirror) -> int:
        return int(self.lib.ref_kv_store_bytes_per_token(C.byref(req), C.c_int(int(i8)), C.c_int(int(mirror))))

    def plan_context(self, req) -> dict:
        p = ContextPlan()
        self.lib.ref_plan_context(C.byref(req), C.byref(p))
        return p.as_dict()

    def has_avx512(self) -> bool:
        return bool(self.lib.ref_cpu_has_avx512())

    def pool_init(self, threads=0) -> int:
        return int(self.lib.ref_pool_init(C.c_uint32(threads)))

    def attention_fused(self, q, kc, vc, cachePos, seqLen, nHeads, nKV, hd, batch=1, flatten=False):
        """q [batch][seqLen][nHeads][hd]; kc, vc [batch][rows][nKV][hd] f32;
        cachePos: int or per-sequence array."""
        q = _c(q, np.float32)
        kc = _c(kc, np.float32)
        vc = _c(vc, np.float32)
        pos = np.ascontiguousarray(np.broadcast_to(np.asarray(cachePos, np.uint32), (batch,)))
        out = np.zeros((batch, seqLen, nHeads, hd), np.float32)
        self.lib.ref_attention_fused(_p(q, _f32p), _p(kc, _f32p), _p(vc, _f32p), _p(out, _f32p),
                                     C.c_uint32(batch), C.c_uint64(q.size // batch),
                                     C.c_uint64(kc.size // batch), _p(pos, _u32p), C.c_uint32(seqLen),
                                     C.c_uint32(nHeads), C.c_uint32(nKV), C.c_uint32(hd),
                                     C.c_int(int(flatten)))
        return out


def ref_available() -> bool:
    return os.path.exists(_REF_PATH)


_ref_singleton = None


def ref() -> _Ref:
    global _ref_singleton
    if _ref_singleton is None:
        _ref_singleton = _Ref()
    return _ref_singleton
