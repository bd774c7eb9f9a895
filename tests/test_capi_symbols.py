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
