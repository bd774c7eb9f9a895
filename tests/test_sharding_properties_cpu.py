"""Properties of the multi-GPU planning functions over random inputs (hypothesis)."""
from hypothesis import given, settings, strategies as st

from tinycoder_inference_b200 import sharding


@settings(max_examples=200, deadline=None)
@given(st.lists(st.integers(1, 40000), min_size=1, max_size=80), st.integers(1, 8))
def test_sequence_shards_partition_and_balance(lens, parts):
    shards = sharding.plan_sequence_shards(lens, parts)
    flat = sorted(i for s in shards for i in s)
    assert flat == list(range(len(lens))), "every sequence on exactly one rank"
    loads = [sum(lens[i] for i in s) for s in shards]
    # longest-first greedy: no rank exceeds the lightest one by more than the longest sequence
    assert max(loads) - min(loads) <= max(lens)


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 300000), st.integers(1, 16), st.sampled_from([64, 128, 256]))
def test_context_ranges_partition_in_order(length, parts, quantum):
    r = sharding.plan_context_ranges(length, parts, quantum)
    assert len(r) == parts and r[0][0] == 0 and r[-1][1] == length
    for (lo, hi), (lo2, _) in zip(r, r[1:]):
        assert lo <= hi == lo2
    # every cut point is a multiple of the quantum, or the end of the sequence (empty tail ranges)
    for lo, hi in r:
        assert lo % quantum == 0 or lo == length
        assert hi % quantum == 0 or hi == length
    blocks = [(hi - lo + quantum - 1) // quantum for lo, hi in r]
    assert max(blocks) - min(blocks) <= 1, "ranks differ by at most one block of rows"


@settings(max_examples=100, deadline=None)
@given(st.sampled_from([1, 2, 4, 8]), st.sampled_from([1, 2, 4, 8]), st.integers(1, 64))
def test_grid_plan_uses_every_rank_once(world, nKV, nseq):
    g = sharding.plan_grid(world, nKV, nseq)
    assert g.head_parts * g.seq_parts * g.ctx_parts == world
    assert nKV % g.head_parts == 0
    coords = {g.coords(r) for r in range(world)}
    assert len(coords) == world
