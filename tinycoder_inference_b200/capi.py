"""ctypes view of libtc_attn.so (the C ABI declared in include/tc_attn.h).

Loading is strict: when the shared library is missing the import raises.  There
is no CPU path behind these calls -- a machine without the built CUDA library
cannot run the product.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtc_attn.so")

TC_OK = 0
TC_EINVAL = 1
TC_ECONTEXT_FULL = 2
TC_ECUDA = 3
TC_EUNSUPPORTED = 4
TC_EWORKSPACE = 5
TC_EDEVICE = 6
TC_KV_F32 = 0
TC_KV_I8 = 1
TC_DECODE_PDL = 1


class TcError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"tc_attn error {code}: {msg}")
        self.code = code


class ContextFull(TcError):
    """The write or read would pass the window; nothing was launched."""


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


class ContextShardPlan(C.Structure):
    _fields_ = [("plan", ContextPlan), ("headParts", C.c_uint32), ("ctxParts", C.c_uint32),
                ("kvHeadsPerGpu", C.c_uint32), ("rowsPerGpu", C.c_uint32)]


class KvPoolGeometry(C.Structure):
    _fields_ = [
        ("kvLayerStride", C.c_uint64),
        ("kvSlots", C.c_uint32),
        ("kvAllocBytes", C.c_uint64),
        ("kv8LayerStride", C.c_uint64),
        ("kv8ScaleStride", C.c_uint64),
        ("kv8AllocBytes", C.c_uint64),
        ("kv8ScaleAllocBytes", C.c_uint64),
        ("attnChunk", C.c_uint32),
        ("attnChunks", C.c_uint32),
        ("partialAccBytes", C.c_uint64),
        ("partialMLBytes", C.c_uint64),
    ]


class KvSessionConfig(C.Structure):
    _fields_ = [
        ("nHeads", C.c_uint32), ("nKV", C.c_uint32), ("hd", C.c_uint32),
        ("maxSeqLen", C.c_uint32), ("slots", C.c_uint32),
        ("kvStoreI8", C.c_int), ("kvMirror", C.c_int), ("kvHalf", C.c_int),
        ("kvK", C.c_void_p), ("kvV", C.c_void_p),
        ("kvK8", C.c_void_p), ("kvV8", C.c_void_p),
        ("kvK8Scale", C.c_void_p), ("kvV8Scale", C.c_void_p),
        ("pAcc", C.c_void_p), ("pM", C.c_void_p), ("pL", C.c_void_p),
        ("numChunks", C.c_uint32),
        ("ropeCos", C.c_void_p), ("ropeSin", C.c_void_p),
        ("prefillScratch", C.c_void_p), ("prefillScratchBytes", C.c_size_t),
    ]


class PeerGroup(C.Structure):
    _fields_ = [("buffers", C.c_void_p * 16), ("world", C.c_uint32), ("rank", C.c_uint32)]


class DecodeI8Batch(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("out", C.c_void_p),
        ("k8", C.c_void_p),
        ("v8", C.c_void_p),
        ("ks", C.c_void_p),
        ("vs", C.c_void_p),
        ("pAcc", C.c_void_p),
        ("pM", C.c_void_p),
        ("pL", C.c_void_p),
        ("lens", C.c_void_p),
        ("rowBase", C.c_void_p),
        ("rowsPerSeq", C.c_uint64),
        ("totalRows", C.c_uint64),
        ("batch", C.c_uint32),
        ("nHeads", C.c_uint32),
        ("nKV", C.c_uint32),
        ("hd", C.c_uint32),
        ("maxLen", C.c_uint32),
        ("numChunks", C.c_uint32),
        ("invSqrt", C.c_float),
        ("partialsOnly", C.c_int),
        ("chunksUsed", C.POINTER(C.c_uint32)),
        ("flags", C.c_uint32),
        ("prefetchRows", C.c_uint32),
        ("nextK8", C.c_void_p),
        ("nextV8", C.c_void_p),
        ("mergeTickets", C.c_void_p),
        ("appendK", C.c_void_p),
        ("appendV", C.c_void_p),
    ]


# every symbol include/tc_attn.h declares, with its argument types
_vp, _u32, _u64, _f, _i = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int
_sz_p = C.POINTER(C.c_size_t)
SIGNATURES = {
    "tc_strerror": (C.c_char_p, [_i]),
    "tc_last_error": (C.c_char_p, []),
    "tc_device_status": (_i, [_vp, C.POINTER(_u32)]),
    "tc_kv_append": (_i, [_vp, _vp, _vp, _vp, _i, _u32, _u32, _u32, _u32, _vp, _u32, _vp]),
    "tc_kv_append_rope": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _u32, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp,
                               _u32, _vp]),
    "tc_rope_q": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp]),
    "tc_kv_quantize_i8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u64, _u64, _vp, _u64, _vp]),
    "tc_attn_workspace_bytes": (_i, [_u32, _u32, _u32, _u32, _sz_p, _sz_p, _sz_p]),
    "tc_split_geometry": (_i, [_u32, _u32, _u32, C.POINTER(_u32), C.POINTER(_u32)]),
    "tc_attn_decode_i8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _u64,
                               _u32, _u32, _f, _vp]),
    "tc_attn_decode_i8_batch": (_i, [C.POINTER(DecodeI8Batch), _vp]),
    "tc_attn_decode_i8_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u64, _f, _vp]),
    "tc_attn_decode_kv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _u64, _u32,
                               _u32, _f, _i, _vp, _vp]),
    "tc_attn_merge_partials": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp]),
    "tc_attn_merge_gathered": (_i, [_vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "tc_kv_quantize_i8_batch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u64, _vp, _u32, _vp, C.c_int32,
                                    _u64, _vp]),
    "tc_kv_session_create": (_i, [C.POINTER(KvSessionConfig), C.POINTER(_vp)]),
    "tc_kv_session_destroy": (None, [_vp]),
    "tc_kv_session_clear": (_i, [_vp, _vp]),
    "tc_kv_session_begin": (_i, [_vp, _u32, C.POINTER(_u32)]),
    "tc_kv_session_commit": (_i, [_vp, _u32]),
    "tc_kv_session_pos": (_u32, [_vp]),
    "tc_kv_session_context_full": (_i, [_vp]),
    "tc_kv_session_rows8": (_u32, [_vp, _u32]),
    "tc_kv_session_attend": (_i, [_vp, _u32, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _i, _vp]),
    "tc_qk_norm_rope": (_i, [_vp, _u32, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _u32,
                            _vp]),
    "tc_rope_tables": (_i, [_vp, _vp, _u32, _u32, _f]),
    "tc_mrope_tables": (_i, [_vp, _vp, _u32, _u32, _f]),
    "tc_attn_exchange_bytes": (_i, [_u32, _u32, _u32, _sz_p]),
    "tc_attn_merge_exchange": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, C.POINTER(PeerGroup), _u32, _vp]),
    "tc_attn_merge_exchange_local": (_i, [C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                          C.POINTER(_vp), _u32, _u32, _u32, _u32, _u32, _vp]),
    "tc_attn_prefill_f16_scratch_bytes": (_i, [_u32, _u32, _u32, _u32, _u32, _sz_p]),
    "tc_attn_prefill_f16": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_size_t, _u32, _u32, _u32, _u32, _u32, _f, _vp]),
    "tc_attn_prefill_f16_kvhalf": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_size_t, _u32, _u32, _u32, _u32, _u32, _f, _vp]),
    "tc_attn_prefill_f16_i8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _u32, _u32, _u32, _u32, _u32, _f, _vp]),
    "tc_attn_prefill_f16_kv8": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_size_t, _u32, _u32, _u32, _u32, _u32, _f, _vp, _vp, _vp,
                                     _vp, _u64, _u64, _vp]),
    "tc_attn_prefill_kv": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _u64, _f, _i, _vp]),
    "tc_attn_prefill_i8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _u64, _f, _vp]),
    "tc_attn_sigmoid_gate": (_i, [_vp, _vp, _u32, _u32, _u32, _vp]),
    "tc_context_request_init": (None, [C.POINTER(ContextRequest)]),
    "tc_kv_bytes_per_token": (_u64, [C.POINTER(ContextRequest), _u32, _u32]),
    "tc_kv_store_bytes_per_token": (_u64, [C.POINTER(ContextRequest), _u32, _u32]),
    "tc_context_plan_compute": (_i, [C.POINTER(ContextRequest), C.POINTER(ContextPlan)]),
    "tc_context_plan_compute_sharded": (_i, [C.POINTER(ContextRequest), _u32, _u32, C.POINTER(ContextShardPlan)]),
    "tc_context_overhead_bytes": (_u64, [_u32, _u32, _u32, _u32, _u32, _u32, _i, _u32, _u64]),
    "tc_probe_free_vram_bytes": (_u64, []),
    "tc_probe_total_vram_bytes": (_u64, []),
    "tc_kv_pool_geometry_compute": (_i, [_u32, _u32, _u32, _u32, _u32, _u32, _i, _i, _i,
                                         C.POINTER(KvPoolGeometry)]),
}


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a).  There is no fallback path."
        )
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError names the missing symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


def check(code: int) -> None:
    if code == TC_OK:
        return
    msg = lib.tc_last_error().decode(errors="replace")
    if code == TC_ECONTEXT_FULL:
        raise ContextFull(code, msg)
    raise TcError(code, msg)
