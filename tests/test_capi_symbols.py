"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

from tinycoder_inference_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "tc_attn.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tc_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 20
    lib = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/tc_attn.h but not exported"
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert set(capi.SIGNATURES) == set(names)


def test_status_strings():
    assert capi.lib.tc_strerror(0) == b"ok"
    assert capi.lib.tc_strerror(capi.TC_ECONTEXT_FULL) == b"context window full"


def test_invalid_arguments_are_rejected_on_the_host():
    # shape checks run before any CUDA call, so they can be exercised without a device
    rc = capi.lib.tc_kv_quantize_i8(None, None, None, None, None, None, 1, 4, 128, 0, 0, None, 0, None)
    assert rc == capi.TC_EINVAL and b"null" in capi.lib.tc_last_error()
    rc = capi.lib.tc_attn_merge_partials(None, None, None, None, 1, 1, 1, 128, None, None)
    assert rc == capi.TC_EINVAL
    a = C.c_size_t()
    assert capi.lib.tc_attn_workspace_bytes(2, 28, 128, 64, C.byref(a), C.byref(C.c_size_t()),
                                            C.byref(C.c_size_t())) == 0
    assert a.value == 2 * 28 * 64 * 128 * 4


def test_prefill_entry_points_check_their_arguments_on_the_host():
    lib = capi.lib
    n = C.c_size_t()
    al = lambda x: (x + 1023) & ~1023
    # q twin + K and V twins of every cached row (1 KB aligned each) + 1 KB for the work counter
    for hd in (64, 128, 256):
        assert lib.tc_attn_prefill_f16_scratch_bytes(512, 1024, 28, 4, hd, C.byref(n)) == 0
        assert n.value == al(512 * 28 * hd * 2) + 2 * al(1536 * 4 * hd * 2) + 1024
    assert lib.tc_attn_prefill_f16_scratch_bytes(512, 0, 28, 4, 96, C.byref(n)) == capi.TC_EUNSUPPORTED
    assert lib.tc_attn_prefill_f16_scratch_bytes(512, 0, 28, 4, 128, None) == capi.TC_EINVAL
    # fake, suitably aligned addresses: every check below fails before anything is dereferenced or launched
    p = C.c_void_p(1 << 20)
    args = (p, p, p, p, p, 1 << 30, 512, 0, 28, 4, 128, 0.088, None)
    assert lib.tc_attn_prefill_f16(None, p, p, p, p, 1 << 30, 512, 0, 28, 4, 128, 0.088, None) == capi.TC_EINVAL
    assert lib.tc_attn_prefill_f16(p, p, p, p, p, 1 << 30, 512, 0, 28, 4, 96, 0.088, None) == capi.TC_EUNSUPPORTED
    assert lib.tc_attn_prefill_f16(p, p, p, p, p, 1 << 30, 512, 0, 28, 5, 128, 0.088, None) == capi.TC_EINVAL
    assert lib.tc_attn_prefill_f16(p, p, p, p, C.c_void_p((1 << 20) + 8), 1 << 30, 512, 0, 28, 4, 128, 0.088,
                                   None) == capi.TC_EINVAL                       # misaligned scratch
    assert lib.tc_attn_prefill_f16(p, p, p, p, p, 4096, 512, 0, 28, 4, 128, 0.088, None) == capi.TC_EWORKSPACE
    assert lib.tc_attn_prefill_f16(p, p, p, p, p, 1 << 30, 0, 0, 28, 4, 128, 0.088, None) == 0   # no rows: nothing to do
    # the int8 store needs its scales, the mirror its pool, and the mirror's rows have to fit the pool
    assert lib.tc_attn_prefill_f16_i8(p, p, p, None, None, p, p, 1 << 30, 512, 0, 28, 4, 128, 0.088,
                                      None) == capi.TC_EINVAL
    assert lib.tc_attn_prefill_f16_kv8(*args[:12], None, p, p, p, 0, 4096, None) == capi.TC_EINVAL
    assert lib.tc_attn_prefill_f16_kv8(*args[:12], p, p, p, p, 4000, 4096 + 16, None) == capi.TC_ECONTEXT_FULL
    assert b"pass the pool" in lib.tc_last_error()


def test_decode_batch_descriptor_is_checked_on_the_host():
    lib = capi.lib
    p = 1 << 20   # a fake, aligned address: every check below fails before anything is dereferenced or launched

    def desc(**kw):
        d = capi.DecodeI8Batch()
        for f in ("q", "out", "k8", "v8", "ks", "vs", "pAcc", "pM", "pL"):
            setattr(d, f, p)
        d.rowsPerSeq, d.totalRows, d.batch, d.nHeads, d.nKV, d.hd = 4096, 4096, 1, 28, 4, 128
        d.maxLen, d.numChunks, d.invSqrt = 4096, 64, 0.088
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    call = lambda d: lib.tc_attn_decode_i8_batch(C.byref(d), None)
    assert call(desc(q=None)) == capi.TC_EINVAL
    assert call(desc(hd=96)) == capi.TC_EUNSUPPORTED
    assert call(desc(nKV=5)) == capi.TC_EINVAL
    assert call(desc(batch=0)) == capi.TC_EINVAL
    assert call(desc(maxLen=0)) == capi.TC_EINVAL
    assert call(desc(totalRows=1 << 31)) == capi.TC_EUNSUPPORTED
    assert call(desc(k8=p + 4)) == capi.TC_EINVAL                 # misaligned pool
    assert call(desc(numChunks=0)) == capi.TC_EWORKSPACE
    # the rows of a new token come as a pair
    assert call(desc(appendK=p)) == capi.TC_EINVAL and b"come together" in lib.tc_last_error()
    assert call(desc(appendV=p)) == capi.TC_EINVAL
