"""Host-side bookkeeping of tc_kv_session without a GPU: configuration checks, the window guard
(GPUModel::forward's refusal before any kernel writes) and the position counter.  The buffers
are never touched by these calls, so placeholder addresses stand in for device memory."""
import ctypes as C

import pytest

from tinycoder_inference_b200 import capi

lib = capi.lib
FAKE = 0x10000   # never dereferenced by create / begin / commit


def _cfg(**kw):
    c = capi.KvSessionConfig()
    c.nHeads, c.nKV, c.hd, c.maxSeqLen, c.slots = 28, 4, 128, 64, 3
    c.kvK = c.kvV = FAKE
    c.pAcc = c.pM = c.pL = FAKE
    c.numChunks = 16
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _create(cfg):
    h = C.c_void_p()
    rc = lib.tc_kv_session_create(C.byref(cfg), C.byref(h))
    return rc, h


def test_window_guard_and_position():
    rc, h = _create(_cfg())
    assert rc == capi.TC_OK and h.value
    pos = C.c_uint32(99)
    assert lib.tc_kv_session_begin(h, 40, C.byref(pos)) == capi.TC_OK and pos.value == 0
    assert lib.tc_kv_session_commit(h, 40) == capi.TC_OK and lib.tc_kv_session_pos(h) == 40
    assert lib.tc_kv_session_begin(h, 24, C.byref(pos)) == capi.TC_OK and pos.value == 40
    # 40 cached + 25 new > 64-token window: refused before anything is written, and it sticks
    assert lib.tc_kv_session_begin(h, 25, C.byref(pos)) == capi.TC_ECONTEXT_FULL
    assert lib.tc_kv_session_context_full(h) == 1 and lib.tc_kv_session_pos(h) == 40
    assert lib.tc_kv_session_commit(h, 25) == capi.TC_ECONTEXT_FULL and lib.tc_kv_session_pos(h) == 40
    assert lib.tc_kv_session_commit(h, 24) == capi.TC_OK and lib.tc_kv_session_pos(h) == 64
    assert lib.tc_kv_session_begin(h, 1, C.byref(pos)) == capi.TC_ECONTEXT_FULL
    for slot in range(3):
        assert lib.tc_kv_session_rows8(h, slot) == 0
    assert lib.tc_kv_session_rows8(h, 7) == 0          # out of range: 0, not a fault
    lib.tc_kv_session_destroy(h)


@pytest.mark.parametrize("bad", [
    dict(nHeads=30),                                    # not a multiple of nKV
    dict(slots=0), dict(maxSeqLen=0), dict(hd=0),
    dict(kvK=None),                                     # an f32 store needs its cache
    dict(kvMirror=1),                                   # a mirror needs the int8 pool
    dict(kvStoreI8=1, kvK=None, kvV=None),              # an int8 store needs the pool too
    dict(kvStoreI8=1, kvMirror=1, kvK8=FAKE, kvV8=FAKE, kvK8Scale=FAKE, kvV8Scale=FAKE),   # either, not both
    dict(ropeCos=FAKE),                                 # cos without sin
])
def test_rejected_configurations(bad):
    rc, h = _create(_cfg(**bad))
    assert rc == capi.TC_EINVAL and not h.value


I8 = dict(kvK8=FAKE, kvV8=FAKE, kvK8Scale=FAKE, kvV8Scale=FAKE)


@pytest.mark.parametrize("bad", [
    # rotation tables with an int8 pool: the int8 paths never rotate, the f32 prefill would
    dict(kvMirror=1, ropeCos=FAKE, ropeSin=FAKE, **I8),
    dict(kvStoreI8=1, kvK=None, kvV=None, ropeCos=FAKE, ropeSin=FAKE, **I8),
    # an fp16 store has no f32 rows to rebuild the decode pool from
    dict(kvHalf=1, kvMirror=1, **I8),
])
def test_unsupported_configurations(bad):
    rc, h = _create(_cfg(**bad))
    assert rc == capi.TC_EUNSUPPORTED and not h.value


def test_int8_store_needs_no_f32_cache():
    rc, h = _create(_cfg(kvStoreI8=1, kvK=None, kvV=None, kvK8=FAKE, kvV8=FAKE, kvK8Scale=FAKE, kvV8Scale=FAKE))
    assert rc == capi.TC_OK
    lib.tc_kv_session_destroy(h)
    assert lib.tc_kv_session_create(None, None) == capi.TC_EINVAL
    assert lib.tc_kv_session_pos(None) == 0 and lib.tc_kv_session_context_full(None) == 0
