"""The context planner: the oracle restatement, the library's C++ planner and
(where it was built) the reference's own compiled planner all reproduce the
known answers of the reference's unit tests (unit_tests/ContextPlanTest.cpp)."""
import json
import os

import pytest

import oracle
from tinycoder_inference_b200 import ops

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
