"""The decode entry point that allocates nothing (its split-KV partials live in an
array inside the library, for callers that cannot allocate device memory) gives the
same output as the regular entry point, on two calls in a row that share the array.

Collected last on purpose: a run that stops at the first failure has then already
run every other test."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import ATOL, RTOL, assert_close, dev, host, make_i8_store

pytestmark = pytest.mark.gpu


def _store(nKV, hd, ctx, seed):
    rng = np.random.default_rng(seed)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd, extra_rows=16)
    return tuple(dev(x) for x in (k8, v8, ks, vs)), (k8[:ctx], v8[:ctx], ks[:ctx], vs[:ctx])


def test_no_alloc_entry_matches_regular_entry_twice_in_a_row():
    hd = 128
    inv = 1.0 / math.sqrt(hd)
    # two different shapes back to back: the second call finds the first call's partials in the array
    for nH, nKV, ctx, seed in [(28, 4, 20000, 1), (40, 8, 3000, 2)]:
        (k8, v8, ks, vs), host_store = _store(nKV, hd, ctx, seed)
        q = np.random.default_rng(seed + 10).standard_normal((1, nH, hd), dtype=np.float32)
        qd = dev(q)
        chunk, chunks = ops.split_geometry(ctx, nH, hd)
        ref_out = torch.empty((1, nH, hd), device="cuda")
        ops.decode_i8(qd, k8, v8, ks, vs, ref_out, ops.workspace(1, nH, hd, chunks), nH, nKV, hd, ctx - 1, chunks,
                      chunk, inv)
        out = torch.full((1, nH, hd), float("nan"), device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        # straight through the C ABI: inputs, output, nothing else
        rc = capi.lib.tc_attn_decode_i8_noalloc(C.c_void_p(qd.data_ptr()), C.c_void_p(k8.data_ptr()),
                                                C.c_void_p(v8.data_ptr()), C.c_void_p(ks.data_ptr()),
                                                C.c_void_p(vs.data_ptr()), C.c_void_p(out.data_ptr()), nH, nKV, hd,
                                                ctx - 1, k8.numel() // (nKV * hd), inv,
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == capi.TC_OK, capi.lib.tc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before   # no device memory was taken
        assert ops.device_status() == 0
        assert_close(host(out), host(ref_out), rtol=RTOL, atol=ATOL, what="no-alloc vs regular entry")
        want = oracle.attention_i8(q, *host_store, 1, nH, nKV, hd, ctx - 1, inv)
        assert_close(host(out), want, rtol=RTOL, atol=ATOL, what="no-alloc vs oracle")


def test_sizes_beyond_the_built_in_scratch_are_refused():
    (k8, v8, ks, vs), _ = _store(1, 128, 64, 3)
    q = torch.zeros((1, 65, 128), device="cuda")
    with pytest.raises(capi.TcError) as e:
        ops.decode_i8_noalloc(q, k8, v8, ks, vs, q.clone(), 65, 1, 128, 63)
    assert e.value.code == capi.TC_EWORKSPACE and "at most 64" in str(e.value)
    with pytest.raises(capi.TcError) as e:
        ops.decode_i8_noalloc(q, k8, v8, ks, vs, q.clone(), 8, 1, 64, 63)
    assert e.value.code == capi.TC_EWORKSPACE
