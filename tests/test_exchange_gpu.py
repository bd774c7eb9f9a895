"""The context-axis exchange-merge kernel on one GPU: all ranks of the protocol in one
cooperative launch, against the oracle's attention over the whole context."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import ops, sharding
from tests.util import assert_close, dev, host, make_i8_store

pytestmark = pytest.mark.gpu


def _shards(nH, nKV, hd, ctx, ranks, C, seed):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((1, nH, hd), dtype=np.float32)
    k8, v8, ks, vs = make_i8_store(rng.standard_normal((ctx, nKV, hd), dtype=np.float32),
                                   rng.standard_normal((ctx, nKV, hd), dtype=np.float32), nKV, hd)
    inv = 1.0 / math.sqrt(hd)
    want = oracle.attention_i8(q, k8, v8, ks, vs, 1, nH, nKV, hd, ctx - 1, inv)
    wss, used_all = [], []
    for lo, hi in sharding.plan_context_ranges(ctx, ranks):
        ws = ops.workspace(1, nH, hd, C)
        for w in ws:
            w.fill_(float("nan"))       # unwritten slots must not matter
        used = 0
        if hi > lo:
            scratch = torch.empty((1, nH, hd), device="cuda")
            used = ops.decode_i8_batch(dev(q), dev(k8[lo:hi]), dev(v8[lo:hi]), dev(ks[lo:hi]), dev(vs[lo:hi]), scratch,
                                       ws, None, 1, nH, nKV, hd, hi - lo, C, invSqrt=inv, partials_only=True)
        wss.append(ws)
        used_all.append(used)
    return want, wss, used_all


@pytest.mark.parametrize("nH,nKV,hd,ctx,ranks", [(28, 4, 128, 5000, 3), (40, 8, 128, 9000, 4), (8, 8, 128, 4000, 8), (8, 2, 256, 1300, 2),
                                                 (16, 4, 128, 300, 4)])
def test_all_ranks_in_one_launch_match_the_oracle(nH, nKV, hd, ctx, ranks):
    C = 32
    want, wss, used = _shards(nH, nKV, hd, ctx, ranks, C, seed=ctx + ranks)
    words = ops.exchange_bytes(nH, hd, ranks) // 4
    bufs = [torch.zeros(words, device="cuda") for _ in range(ranks)]
    # ranks whose range is empty (short context) hold no partials: give them zero active chunks by
    # zeroing l -- the launch takes one active count, the largest
    active = max(used)
    for ws, u in zip(wss, used):
        ws[2].view(nH, C)[:, u:] = 0.0
    for step in range(3):                 # epochs advance, both parities are used
        outs = [torch.full((1, nH, hd), float("nan"), device="cuda") for _ in range(ranks)]
        ops.merge_exchange_local(wss, outs, bufs, nH, C, active, hd)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        for r in range(ranks):
            assert_close(host(outs[r]), want, what=f"rank {r}, step {step}")
        for r in range(1, ranks):
            assert torch.equal(outs[r], outs[0]), "every rank merges the same partials in the same order"


def test_single_rank_is_the_plain_merge():
    nH, nKV, hd, ctx, C = 28, 4, 128, 4000, 64
    want, wss, used = _shards(nH, nKV, hd, ctx, 1, C, seed=5)
    buf = torch.zeros(ops.exchange_bytes(nH, hd, 1) // 4, device="cuda")
    out = torch.empty((1, nH, hd), device="cuda")
    for _ in range(2):
        ops.merge_exchange(wss[0], out, nH, C, used[0], hd, [buf.data_ptr()], 0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), want, what="world 1")


def test_a_missing_rank_ends_the_wait_with_a_status_not_a_hang():
    """Rank 1 never publishes (its buffer pointer is given, nobody launches for it): rank 0's
    blocks give up after the bounded wait, report it through tc_device_status and return."""
    nH, nKV, hd, ctx, C = 4, 2, 128, 600, 8
    _, wss, used = _shards(nH, nKV, hd, ctx, 1, C, seed=9)
    words = ops.exchange_bytes(nH, hd, 2) // 4
    b0, b1 = torch.zeros(words, device="cuda"), torch.zeros(words, device="cuda")
    out = torch.zeros((1, nH, hd), device="cuda")
    ops.merge_exchange(wss[0], out, nH, C, used[0], hd, [b0.data_ptr(), b1.data_ptr()], 0)
    torch.cuda.synchronize()
    from tinycoder_inference_b200 import capi
    with pytest.raises(capi.TcError, match="0x10"):     # TC_EDEVICE, flag "merge wait"
        ops.device_status()
    assert ops.device_status() == 0, "reading the status clears it"
    # the context is intact: a complete exchange on fresh buffers works afterwards
    buf = torch.zeros(ops.exchange_bytes(nH, hd, 1) // 4, device="cuda")
    ops.merge_exchange(wss[0], out, nH, C, used[0], hd, [buf.data_ptr()], 0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0


def test_guards():
    from tinycoder_inference_b200 import capi
    with pytest.raises(capi.TcError):
        ops.exchange_bytes(28, 128, 17)
    with pytest.raises(capi.TcError):
        ops.exchange_bytes(28, 100, 2)
