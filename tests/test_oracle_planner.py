"""The context planner: the oracle restatement, the library's C++ planner and
(where it was built) the reference's own compiled planner all reproduce the
known answers of the reference's unit tests (unit_tests/ContextPlanTest.cpp)."""
import json
import os

import pytest

import oracle
from tinycoder_inference_b200 import capi, ops

MiB = 1 << 20
GiB = 1 << 30
HERE = os.path.dirname(os.path.abspath(__file__))

G27 = dict(modelMax=262144, numLayers=64, numAttentionLayers=16, numKVHeads=4, headDim=256, ropeDims=320,
           int8KvSupported=1)
G9 = dict(modelMax=262144, numLayers=32, numAttentionLayers=8, numKVHeads=4, headDim=256, ropeDims=320,
          int8KvSupported=1)


def _impls():
    out = [("oracle", oracle.make_request, oracle.plan_context,
            lambda r, kv, m: oracle.kv_bytes_per_token(r, kv, m)),
           ("library", ops.context_request, ops.plan_context, ops.kv_bytes_per_token)]
    if oracle.ref_available():
        ref = oracle.ref()
        out.append(("reference", oracle.make_request, ref.plan_context, ref.kv_bytes_per_token))
    return out


IMPLS = _impls()
IDS = [i[0] for i in IMPLS]


@pytest.mark.parametrize("impl", IMPLS, ids=IDS)
def test_kv_bytes_known_answers(impl):
    _, mk, _, bpt = impl
    # unit_tests/ContextPlanTest.cpp:63-75
    r = mk(**G27)
    assert [bpt(r, 0, 1), bpt(r, 0, 0), bpt(r, 1, 0)] == [165632, 132352, 34560]
    r = mk(**G9)
    assert [bpt(r, 0, 1), bpt(r, 0, 0), bpt(r, 1, 0)] == [83456, 66816, 17920]


@pytest.mark.parametrize("impl", IMPLS, ids=IDS)
def test_plan_known_answers(impl):
    _, mk, plan, _ = impl
    pin = dict(gpuFixedOverhead=900 * MiB)
    # :81-98 auto -> 2048 f32+mirror, ceiling 213248 named with int8
    p = plan(mk(**G27, **pin, weightBytes=4 * GiB, freeVram=12 * GiB))
    assert (p["seqLen"], p["kv"], p["kvMirror"], p["kvOnGpu"], p["maxAllowed"]) == (2048, 0, 1, 1, 213248)
    assert "auto" in p["reason"] and "int8" in p["reason"]
    # :102-113
    p = plan(mk(**G27, **pin, weightBytes=4 * GiB, freeVram=12 * GiB, requested=40960))
    assert (p["seqLen"], p["kv"], p["kvMirror"], p["kvBytes"]) == (40960, 0, 1, 40960 * 165632)
    # :117-128 escalate to int8
    p = plan(mk(**G27, **pin, weightBytes=4 * GiB, freeVram=8 * GiB, requested=65536))
    assert (p["seqLen"], p["kv"], p["kvMirror"], p["maxAllowed"]) == (65536, 1, 0, 89088)
    # :130-145 reduced by memory
    p = plan(mk(**G27, **pin, weightBytes=4 * GiB, freeVram=8 * GiB, requested=524288))
    assert p["seqLen"] == p["maxAllowed"] == 89088 and p["kv"] == 1 and "VRAM" in p["reason"]
    # :151-171 model max
    p = plan(mk(**G27, weightBytes=1 * GiB, freeVram=40 * GiB, requested=262144))
    assert p["seqLen"] == 262144 and "model max" not in p["reason"]
    p = plan(mk(**G27, **pin, weightBytes=1 * GiB, freeVram=40 * GiB, requested=300000))
    assert p["seqLen"] == 262144 and "model max" in p["reason"]
    # :173-184 no int8 support
    r = dict(G27)
    r["int8KvSupported"] = 0
    p = plan(mk(**r, **pin, weightBytes=4 * GiB, freeVram=8 * GiB, requested=65536))
    assert (p["kv"], p["kvMirror"], p["seqLen"]) == (0, 0, 23040)
    # :192-203 long request reduced to the full-residency fit
    p = plan(mk(**G27, **pin, freeVram=11 << 30, weightBytes=7 << 30, requested=262144))
    assert 0 < p["seqLen"] < 262144 and p["seqLen"] == p["maxAllowed"] and p["kv"] == 1
    # :205-216 RAM path
    p = plan(mk(**G27, weightBytes=5 * GiB, availableRam=40 * GiB, requested=65536))
    assert (p["kvOnGpu"], p["kv"], p["kvMirror"], p["seqLen"]) == (0, 0, 0, 65536) and "RAM" in p["reason"]
    # :218-235 floor
    p = plan(mk(**G9, weightBytes=5 * GiB, freeVram=12 * GiB, requested=512))
    assert p["seqLen"] == 0 and p["reason"]
    p = plan(mk(**G9, weightBytes=5 * GiB, freeVram=12 * GiB, requested=1024))
    assert p["seqLen"] == 1024
    # :237-245 nothing fits
    p = plan(mk(**G27, weightBytes=1 * GiB, freeVram=700 * MiB))
    assert p["seqLen"] == 0 and p["maxAllowed"] == 0 and p["reason"]
    # :264-280 forced precision
    base = dict(G27, requested=4096, freeVram=12 << 30, weightBytes=4 << 30)
    assert plan(mk(**base))["kv"] == 0
    q = plan(mk(**base, forceKv=1, forceKvSet=1))
    assert (q["kv"], q["seqLen"], q["kvMirror"]) == (1, 4096, 0)
    assert plan(mk(**base, forceKv=0, forceKvSet=1))["kv"] == 0
    # :282-291 missing model max
    r = dict(G9)
    r["modelMax"] = 0
    p = plan(mk(**r, weightBytes=1 * GiB, freeVram=40 * GiB, requested=65536))
    assert p["seqLen"] == 4096 and "4096" in p["reason"]


def test_default_overhead_window():
    # :252-260
    r = ops.context_request()
    assert 1280 * MiB <= r.gpuFixedOverhead <= 1536 * MiB
    assert oracle.DEFAULT_GPU_FIXED_OVERHEAD == r.gpuFixedOverhead
    if oracle.ref_available():
        assert oracle.ref().default_overhead() == r.gpuFixedOverhead


def _random_requests(n, seed=7):
    import numpy as np

    rng = np.random.default_rng(seed)
    for _ in range(n):
        yield dict(
            requested=int(rng.choice([0, 512, 1024, 2048, 3000, 40960, 65536, 262144, 524288])),
            modelMax=int(rng.choice([0, 4096, 32768, 131072, 262144])),
            numLayers=int(rng.choice([24, 28, 32, 64])),
            numAttentionLayers=int(rng.choice([8, 16, 28, 64])),
            numKVHeads=int(rng.choice([2, 4, 8])),
            headDim=int(rng.choice([64, 128, 256])),
            ropeDims=int(rng.choice([64, 128, 320])),
            int8KvSupported=int(rng.integers(0, 2)),
            forceKv=int(rng.integers(0, 2)),
            forceKvSet=int(rng.integers(0, 4) == 0),
            weightBytes=int(rng.integers(0, 60)) * GiB // 4,
            freeVram=int(rng.choice([0, 1, 8, 11, 24, 80, 178])) * GiB,
            availableRam=int(rng.choice([0, 4, 40, 400])) * GiB,
            gpuFixedOverhead=int(rng.choice([900, 1408, 2560])) * MiB,
        )


def test_library_planner_matches_oracle_and_reference_on_random_requests():
    ref = oracle.ref() if oracle.ref_available() else None
    for kw in _random_requests(400):
        a = oracle.plan_context(oracle.make_request(**kw))
        b = ops.plan_context(ops.context_request(**kw))
        assert a == b, kw
        if ref is not None:
            assert ref.plan_context(oracle.make_request(**kw)) == a, kw


def test_invariants_hold_on_random_requests():
    # unit_tests/ContextPlanTest.cpp:294-335
    for kw in _random_requests(200, seed=11):
        p = ops.plan_context(ops.context_request(**kw))
        ceiling = kw["modelMax"] or 4096
        if kw["requested"] == 0:
            assert p["seqLen"] % 256 == 0
        else:
            assert p["seqLen"] <= min(kw["requested"], ceiling)
        assert p["seqLen"] <= ceiling and p["maxAllowed"] >= p["seqLen"]


def test_golden_fixture():
    """Plans recorded from the reference's compiled planner (tests/golden/make_planner_golden.py)."""
    with open(os.path.join(HERE, "golden", "planner_golden.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 100
    for c in cases:
        assert oracle.plan_context(oracle.make_request(**c["request"])) == c["plan"]
        assert ops.plan_context(ops.context_request(**c["request"])) == c["plan"]


def test_split_geometry_rule():
    # window -> (chunk, chunks): GPUComputeUpload.cu:318-334
    for window, nH, hd, want in [(2048, 14, 64, (32, 64)), (8192, 28, 128, (32, 256)), (32768, 28, 128, (64, 512)),
                                 (131072, 40, 128, (256, 512)), (2048, 12, 128, (32, 64)),
                                 (262144, 24, 256, (512, 512))]:
        assert oracle.split_geometry(window, nH, hd) == want
        assert ops.split_geometry(window, nH, hd) == want


def test_pool_geometry():
    g = ops.kv_pool_geometry(65536, 64, 4, 24, 4, 256, kvStoreI8=True)
    assert g.kvSlots == 16 and g.kvAllocBytes == 0
    assert g.kv8LayerStride == (65536 + 16) * 4 * 256 and g.kv8ScaleStride == (65536 + 16) * 4 * 4
    assert (g.attnChunk, g.attnChunks) == (128, 512)
    assert g.partialAccBytes == 24 * 512 * 256 * 4
    g = ops.kv_pool_geometry(2048, 28, 0, 28, 4, 128)
    assert g.kvSlots == 28 and g.kvLayerStride == 2048 * 4 * 128 * 4 and g.kv8AllocBytes == 0


# ---- the partitioned planner (no counterpart in the reference) --------------------------------

def _req32b(**kw):
    """The 32B-shaped request of the long-context configuration: 64 attention layers, 8 kv heads, head_dim 128."""
    base = dict(requested=131072, modelMax=131072, numLayers=64, numAttentionLayers=64, numKVHeads=8, headDim=128,
                ropeDims=128, int8KvSupported=1, weightBytes=0, freeVram=24 << 30, gpuFixedOverhead=900 << 20)
    base.update(kw)
    return ops.context_request(**base)


def test_sharded_plan_of_one_gpu_is_the_reference_plan():
    with open(os.path.join(os.path.dirname(__file__), "golden", "planner_golden.json")) as f:
        cases = json.load(f)
    for c in cases[:160]:
        req = ops.context_request(**c["request"])
        assert {k: v for k, v in ops.plan_context_sharded(req, 1, 1).items()
                if k in c["plan"]} == ops.plan_context(req)


def test_long_context_fits_a_partition_where_one_gpu_cannot():
    one = ops.plan_context(_req32b())
    per_token_i8 = 64 * (2 * 8 * 128 + 2 * 8 * 4) + 4 * 128          # 135,680 bytes: 131072 rows = 17.8 GB
    assert ops.kv_bytes_per_token(_req32b(), capi.TC_KV_I8, 0) == per_token_i8
    assert one["seqLen"] == 131072 and one["kv"] == capi.TC_KV_I8    # 24 GB: only the int8 store holds the window
    tight = ops.plan_context(_req32b(freeVram=12 << 30))
    assert tight["reduced"] == 1 and tight["seqLen"] < 131072        # 12 GB: not even int8
    for hp, cp in ((8, 1), (4, 2), (2, 4), (1, 8)):
        p = ops.plan_context_sharded(_req32b(freeVram=12 << 30), hp, cp)
        assert p["seqLen"] == 131072 and p["reduced"] == 0, (hp, cp, p)
        assert p["kvHeadsPerGpu"] == 8 // hp and p["rowsPerGpu"] == 131072 // cp
        # what one GPU stores: its heads of its rows
        req_g = _req32b(numKVHeads=8 // hp)
        assert p["kvBytes"] == p["rowsPerGpu"] * ops.kv_bytes_per_token(req_g, p["kv"], p["kvMirror"])
    # with 8 GPUs by heads even the f32 store with its int8 decode pool fits in 24 GB per GPU
    best = ops.plan_context_sharded(_req32b(), 8, 1)
    assert best["kv"] == capi.TC_KV_F32 and best["kvMirror"] == 1 and best["seqLen"] == 131072


def test_sharded_plan_edges():
    # an auto request keeps the single-device window, the ceiling grows with the context ranges
    auto = ops.plan_context_sharded(_req32b(requested=0, freeVram=12 << 30), 1, 4)
    assert auto["seqLen"] == 2048 and auto["maxAllowed"] >= ops.plan_context(_req32b(requested=0, freeVram=12 << 30))["maxAllowed"]
    # a context range below the 1024-row floor is refused like a window below it
    tiny = ops.plan_context_sharded(_req32b(requested=4096), 1, 8)
    assert tiny["seqLen"] == 0 and "floor" in tiny["reason"]
    # ragged division: 7 ranges of a 100000-row window, 256-row units
    rag = ops.plan_context_sharded(_req32b(requested=100000), 2, 7)
    assert rag["seqLen"] == 100000 and rag["rowsPerGpu"] == 14336 and rag["rowsPerGpu"] * 7 >= 100000
    with pytest.raises(capi.TcError):
        ops.plan_context_sharded(_req32b(), 0, 1)


def test_overhead_follows_the_library_scratch():
    base = ops.context_overhead_bytes(40, 8, 128, 131072, runtime_reserve=0)
    assert base == 40 * 512 * 130 * 4                                # partial buffers only (int8 store, one GPU)
    split = ops.context_overhead_bytes(40, 8, 128, 131072, head_parts=2, ctx_parts=4, runtime_reserve=0)
    assert split > 20 * 512 * 130 * 4 and split < base                # half the heads, plus exchange buffers
    f32 = ops.context_overhead_bytes(28, 4, 128, 32768, kv_store_i8=False, runtime_reserve=0)
    twins = 512 * 28 * 128 * 2 + 2 * 32768 * 4 * 128 * 2 + 1024        # q of a 512-row chunk, K/V of the window, fp16; work counter
    assert f32 == 28 * 512 * 130 * 4 + twins
    assert ops.context_overhead_bytes(28, 4, 128, 32768, runtime_reserve=1 << 20) - ops.context_overhead_bytes(
        28, 4, 128, 32768, runtime_reserve=0) == 1 << 20
