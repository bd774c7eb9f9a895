"""Host logic of the multi-GPU partitioning, on CPU: the planners, and the
context-axis split with its partial exchange run as two gloo ranks (the partials of
each rank come from the oracle; the exchange and the merge rule are what is tested)."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tinycoder_inference_b200 import sharding, synth


def test_kv_head_shards():
    s = sharding.plan_kv_head_shards(40, 8, 4)
    assert [(x.kv_lo, x.kv_hi, x.q_lo, x.q_hi) for x in s] == [(0, 2, 0, 10), (2, 4, 10, 20), (4, 6, 20, 30),
                                                               (6, 8, 30, 40)]
    with pytest.raises(ValueError):
        sharding.plan_kv_head_shards(28, 4, 8)


def test_sequence_shards_balance_tokens_not_sequences():
    lens = synth.ragged_lengths(5, 64)
    assert lens.min() >= 512 and lens.max() <= 32768
    for parts in (2, 4, 8):
        shards = sharding.plan_sequence_shards(lens, parts)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [int(sum(lens[i] for i in s)) for s in shards]
        assert max(loads) - min(loads) <= int(lens.max())          # LPT bound
        assert max(loads) <= 1.05 * (sum(loads) / parts)            # within 5 % of perfect at these sizes
    # deterministic, ties to the lower rank
    assert sharding.plan_sequence_shards([5, 5, 5, 5], 2) == [[0, 2], [1, 3]]
    assert sharding.plan_sequence_shards([], 3) == [[], [], []]


def test_context_ranges_cover_and_align():
    for length, parts in [(131072, 8), (131073, 8), (1000, 4), (100, 8), (1, 2), (32768, 3)]:
        r = sharding.plan_context_ranges(length, parts)
        assert r[0][0] == 0 and r[-1][1] == length
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(lo % 256 == 0 or lo == length for lo, _ in r)
        sizes = [hi - lo for lo, hi in r]
        assert max(sizes) - min(s for s in sizes) <= 256 + 255


def test_grid_plan_fills_the_box():
    g = sharding.plan_grid(8, 8, 1)          # 32B shape, one sequence: 8 head groups
    assert (g.head_parts, g.seq_parts, g.ctx_parts) == (8, 1, 1)
    g = sharding.plan_grid(8, 4, 64)         # 7B shape, 64 sequences: 4 head groups x 2 sequence groups
    assert (g.head_parts, g.seq_parts, g.ctx_parts) == (4, 2, 1)
    g = sharding.plan_grid(8, 4, 1)          # one sequence, 4 kv heads: the context axis takes the rest
    assert (g.head_parts, g.seq_parts, g.ctx_parts) == (4, 1, 2)
    g = sharding.plan_grid(8, 8, 1, prefer_context=True)
    assert (g.head_parts, g.seq_parts, g.ctx_parts) == (1, 1, 8)
    assert sorted(g.coords(r) for r in range(8)) == [(0, 0, c) for c in range(8)]
    g = sharding.plan_grid(4, 4, 64)
    assert {g.coords(r) for r in range(4)} == {(h, 0, 0) for h in range(4)}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ctx_split_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        nH, nKV, hd, ctx, C = 10, 2, 128, 1500, 4
        rng = np.random.default_rng(3)                      # same data on every rank
        q = rng.standard_normal((1, nH, hd), dtype=np.float32)
        k = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
        v = rng.standard_normal((ctx, nKV, hd), dtype=np.float32)
        k8, v8, ks, vs = oracle.quant_kv8(k, v, nKV, hd)
        inv = 1.0 / math.sqrt(hd)
        lo, hi = sharding.plan_context_ranges(ctx, world)[rank]
        n = hi - lo
        acc = np.zeros((nH, C, hd), np.float32)
        m = np.full((nH, C), -1e30, np.float32)
        l = np.zeros((nH, C), np.float32)
        if n > 0:
            chunk = (n + C - 2) // (C - 1)                  # leaves the last slot unused: it must read as empty
            a, b, c = oracle.decode_i8_split(q, k8[lo:hi], v8[lo:hi], ks[lo:hi], vs[lo:hi], nH, nKV, hd, n - 1, C - 1,
                                             chunk, inv)
            acc[:, :C - 1], m[:, :C - 1], l[:, :C - 1] = a, b, c
        gacc, gm, gl = sharding.gather_partials(torch.from_numpy(acc), torch.from_numpy(m), torch.from_numpy(l))
        assert gacc.shape == (nH, world * C, hd)
        got = oracle.combine_partials(gacc.numpy(), gm.numpy(), gl.numpy(), 1, nH, world * C, hd)
        want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, inv)
        err = np.abs(got - want)
        ok = bool((err <= 1e-4 + 1e-3 * np.abs(want)).all())
        # the failure rule: a rank whose partial never arrives is noticed on the host, not waited for on a device
        ret[rank] = (ok, float(err.max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_split_merge_over_gloo(world):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_ctx_split_worker, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world and all(v[0] for v in ret.values()), dict(ret)


def _timeout_worker(rank, world, port, ret):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            ret[rank] = "left"          # leaves between steps without joining the exchange
            return
        t = torch.zeros(4)
        try:
            sharding.gather_partials(t.view(1, 1, 4), t[:1].view(1, 1), t[:1].view(1, 1))
            ret[rank] = "no error"
        except Exception as e:          # the short process-group timeout ends the collective with an error
            ret[rank] = "error: " + type(e).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_ends_the_exchange_with_an_error():
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_timeout_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret[1] == "left" and str(ret[0]).startswith("error"), dict(ret)
