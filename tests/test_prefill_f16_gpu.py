"""Causal fp16 prefill on tcgen05 against the oracle's restatement of the
reference's materialised path (fp16 operands, f32 accumulation, fp16
probabilities).  Tolerance for this path: 2e-2 (relative), as the reference's own
fp16-vs-f32 comparison allows (max abs diff 0.0146 on its outputs)."""
import math

import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import capi, ops
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu

RTOL16, ATOL16 = 2e-2, 2e-3


def _run(S, nH, nKV, seed, scale=1.0, hd=128):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((S, nH, hd), dtype=np.float32) * scale
    k = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((S, nKV, hd), dtype=np.float32)
    inv = 1.0 / math.sqrt(hd)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    nbytes = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd)
    scratch = torch.empty(nbytes + 1024, dtype=torch.uint8, device="cuda")
    off = (-scratch.data_ptr()) % 1024
    ops.prefill_f16(dev(q), dev(k), dev(v), out, scratch[off:off + nbytes], S, nH, nKV, hd, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    return q, k, v, got, inv


@pytest.mark.parametrize("S,nH,nKV", [(128, 1, 1), (256, 4, 2), (300, 8, 2), (1, 4, 4), (129, 7, 1), (512, 28, 4)])
def test_against_materialised_reference_path(S, nH, nKV):
    q, k, v, got, inv = _run(S, nH, nKV, seed=S + nH)
    want = oracle.prefill_f16(q, k, v, S, nH, nKV, 128, inv)
    assert_close(got, want, rtol=RTOL16, atol=ATOL16, what=f"prefill_f16 S={S} nH={nH}")
    # and close to exact attention on the fp16-rounded operands (shows where both sit)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, S, nH, nKV, 128, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="vs f64 on fp16 operands")


@pytest.mark.parametrize("S,nH,nKV", [(128, 1, 1), (300, 14, 2), (1, 4, 4), (129, 7, 1), (1100, 4, 2)])
def test_head_dim_64(S, nH, nKV):
    # the 14 / 2 / 64 shape of the smallest model, ragged ends, more than one item per block
    q, k, v, got, inv = _run(S, nH, nKV, seed=64 + S + nH, hd=64)
    want = oracle.prefill_f16(q, k, v, S, nH, nKV, 64, inv)
    assert_close(got, want, rtol=RTOL16, atol=ATOL16, what=f"prefill_f16 hd 64 S={S} nH={nH}")


@pytest.mark.parametrize("S,nH,nKV", [(128, 1, 1), (300, 8, 2), (1, 4, 4), (129, 6, 1), (1100, 4, 2)])
def test_head_dim_256(S, nH, nKV):
    # the gated models' shape: one query tile per block, 32-token KV tiles, a 256-column accumulator
    q, k, v, got, inv = _run(S, nH, nKV, seed=256 + S + nH, hd=256)
    want = oracle.prefill_f16(q, k, v, S, nH, nKV, 256, inv)
    assert_close(got, want, rtol=RTOL16, atol=ATOL16, what=f"prefill_f16 hd 256 S={S} nH={nH}")


def test_head_dim_256_peaked_scores_continued_rows_and_mirror():
    hd, nH, nKV = 256, 4, 2
    q, k, v, got, inv = _run(700, nH, nKV, seed=12, scale=6.0, hd=hd)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, 700, nH, nKV, hd, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="hd 256, peaked scores")
    out = torch.full((250, nH, hd), float("nan"), device="cuda")
    sc = _scratch(250, nH, nKV, 450, hd=hd)
    k8 = torch.zeros((716, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.zeros_like(k8)
    ks = torch.zeros((716, nKV), device="cuda")
    vs = torch.zeros_like(ks)
    ops.prefill_f16(dev(q[450:]), dev(k), dev(v), out, sc, 250, nH, nKV, hd, invSqrt=inv, cachePos=450, kv8=(k8, v8, ks, vs))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), got[450:], rtol=RTOL16, atol=ATOL16, what="hd 256: continued rows against the single call")
    w8 = oracle.quant_kv8(k[450:], v[450:], nKV, hd)
    for got8, want8, name in zip((k8, v8, ks, vs), w8, ("k8", "v8", "ks", "vs")):
        assert np.array_equal(host(got8[450:700]), want8), f"hd 256 mirror {name}"


def test_head_dim_64_peaked_scores_and_continued_rows():
    q, k, v, got, inv = _run(900, 4, 2, seed=11, scale=6.0, hd=64)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, 900, 4, 2, 64, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="hd 64, peaked scores")
    # query rows 600 .. 899 over the same cache in a call of their own
    out = torch.full((300, 4, 64), float("nan"), device="cuda")
    sc = _scratch(300, 4, 2, 600, hd=64)
    ops.prefill_f16(dev(q[600:]), dev(k), dev(v), out, sc, 300, 4, 2, 64, invSqrt=inv, cachePos=600)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(out), got[600:], rtol=RTOL16, atol=ATOL16, what="hd 64: continued rows against the single call")


@pytest.mark.parametrize("hd,nH,nKV", [(128, 8, 2), (64, 14, 2)])
def test_int8_mirror_from_the_twins_launch_equals_the_quantise_kernel(hd, nH, nKV):
    """tc_attn_prefill_f16_kv8: the pool rows of the call's new positions, bit-identical to
    tc_kv_quantize_i8 and to the oracle; rows before cachePos and after the call stay untouched;
    the attention output is the one of the plain call."""
    total, c0, S = 700, 300, 400
    rng = np.random.default_rng(hd)
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    k[c0 + 5, 1] = 0.0                                   # an all-zero row: scale 1, bytes 0
    dq, dk, dv = dev(q), dev(k), dev(v)
    sc = _scratch(S, nH, nKV, c0, hd=hd)
    plain = torch.empty((S, nH, hd), device="cuda")
    ops.prefill_f16(dq, dk, dv, plain, sc, S, nH, nKV, hd, cachePos=c0)
    pool_rows = total + 16
    k8 = torch.full((pool_rows, nKV, hd), 77, dtype=torch.int8, device="cuda")
    v8 = torch.full_like(k8, 77)
    ks = torch.full((pool_rows, nKV), -3.0, device="cuda")
    vs = torch.full_like(ks, -3.0)
    out = torch.empty_like(plain)
    ops.prefill_f16(dq, dk, dv, out, sc, S, nH, nKV, hd, cachePos=c0, kv8=(k8, v8, ks, vs))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(out, plain)
    r8 = [torch.empty_like(k8), torch.empty_like(v8), torch.empty_like(ks), torch.empty_like(vs)]
    ops.kv_quantize_i8(dk, dv, *r8, S, nKV, hd, dst_base=c0, src_base=c0)
    w8 = oracle.quant_kv8(k[c0:], v[c0:], nKV, hd)
    for got, ref, want, name in zip((k8, v8, ks, vs), r8, w8, ("k8", "v8", "ks", "vs")):
        assert torch.equal(got[c0:c0 + S], ref[c0:c0 + S]), f"{name}: fused against the quantise kernel"
        assert np.array_equal(host(got[c0:c0 + S]), want), f"{name}: fused against the oracle"
    assert bool((k8[:c0] == 77).all()) and bool((k8[c0 + S:] == 77).all()) and bool((ks[:c0] == -3.0).all())
    # a pool too small for the rows is refused on the host
    with pytest.raises(capi.TcError) as e:
        ops.prefill_f16(dq, dk, dv, out, sc, S, nH, nKV, hd, cachePos=c0, kv8=(k8[:c0 + 10], v8[:c0 + 10], ks[:c0 + 10], vs[:c0 + 10]))
    assert e.value.code == capi.TC_ECONTEXT_FULL


@pytest.mark.parametrize("hd,nH,nKV,total,c0", [(128, 8, 2, 700, 300), (64, 14, 2, 520, 0), (128, 4, 4, 130, 129)])
def test_fp16_store_and_int8_store_as_the_kv_source(hd, nH, nKV, total, c0):
    """tc_attn_prefill_f16_kvhalf reads the fp16 store in place, tc_attn_prefill_f16_i8 makes its twins
    from bytes x row scale; both against the oracle's kernels for those stores."""
    S = total - c0
    inv = 1.0 / math.sqrt(hd)
    rng = np.random.default_rng(7 * hd + total)
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    dq = dev(q)
    sc = _scratch(S, nH, nKV, c0, hd=hd)
    # fp16 store
    k16, v16 = k.astype(np.float16), v.astype(np.float16)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    n_q = ops.prefill_f16_scratch_bytes(S, nH, 0, hd)             # q's twin and the counter are all it needs
    ops.prefill_f16_kvhalf(dq, dev(k16), dev(v16), out, sc[:n_q], S, nH, nKV, hd, invSqrt=inv, cachePos=c0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = oracle.attention_kv(q, k16, v16, S, nH, nKV, hd, c0, inv)
    assert_close(host(out), want, rtol=RTOL16, atol=ATOL16, what=f"fp16 store, hd {hd}, rows {c0}..{total}")
    # int8 store
    k8, v8, ks, vs = oracle.quant_kv8(k, v, nKV, hd)
    out.fill_(float("nan"))
    ops.prefill_f16_i8(dq, dev(k8), dev(v8), dev(ks), dev(vs), out, sc, S, nH, nKV, hd, invSqrt=inv, cachePos=c0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = oracle.attention_i8(q, k8, v8, ks, vs, S, nH, nKV, hd, c0, inv)
    assert_close(host(out), want, rtol=RTOL16, atol=ATOL16, what=f"int8 store, hd {hd}, rows {c0}..{total}")


@pytest.mark.parametrize("S,nH,nKV,hd", [(1024, 28, 4, 128), (2048, 16, 2, 256), (900, 40, 8, 64)])
def test_one_tile_items_with_several_items_per_block(S, nH, nKV, hd):
    """Calls cut into one-tile work items (too few two-tile items for every SM; always at head_dim
    256) with more items than blocks: tile B is absent in consecutive items of a block, and its warps
    must not run a phase ahead of the producer.  A row sample against the oracle."""
    inv = 1.0 / math.sqrt(hd)
    g = torch.Generator(device="cuda")
    g.manual_seed(S + hd)
    q = torch.randn((S, nH, hd), device="cuda", generator=g)
    k = torch.randn((S, nKV, hd), device="cuda", generator=g)
    v = torch.randn((S, nKV, hd), device="cuda", generator=g)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_f16(q, k, v, out, _scratch(S, nH, nKV, 0, hd=hd), S, nH, nKV, hd, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    rows = np.array(sorted(set(range(0, S, 61)) | {127, 128, S - 129, S - 128, S - 1}), np.uint32)
    want = oracle.prefill_f16_rows(host(q), host(k), host(v), rows, S, nH, nKV, hd, inv)
    assert_close(got[rows], want, rtol=RTOL16, atol=ATOL16, what=f"one-tile items, S={S} hd={hd}")


def test_seeded_random_shapes():
    """Forty seeded shapes -- head_dim 64 / 128 / 256, 1 to 40 q heads in groups of 1 to 8, 1 to 2600 query
    rows behind 0 to 1500 cached rows, so one-tile and two-tile items, one to a dozen items per block,
    tile B present, absent and ragged -- each against the oracle on a row sample."""
    rng = np.random.default_rng(20261125)
    for case in range(40):
        hd = int(rng.choice([64, 128, 256]))
        nKV = int(rng.choice([1, 2, 4, 8]))
        group = int(rng.choice([1, 2, 3, 5, 7, 8]))
        nH = nKV * group
        if nH > 40:
            nKV, nH = 4, 4 * group
        S = int(rng.choice([1, 2, 127, 128, 129, 255, 256, 257, 300, 511, 640, 900, 1024, 1500, 2600]))
        c0 = int(rng.choice([0, 0, 1, 63, 64, 200, 513, 1500]))
        if (c0 + S) * nH > 60000:           # keep the oracle quick
            c0 = 0
            S = min(S, 60000 // nH)
        inv = 1.0 / math.sqrt(hd)
        g = torch.Generator(device="cuda")
        g.manual_seed(1000 + case)
        q = torch.randn((S, nH, hd), device="cuda", generator=g)
        k = torch.randn((c0 + S, nKV, hd), device="cuda", generator=g)
        v = torch.randn((c0 + S, nKV, hd), device="cuda", generator=g)
        out = torch.full((S, nH, hd), float("nan"), device="cuda")
        ops.prefill_f16(q, k, v, out, _scratch(S, nH, nKV, c0, hd=hd), S, nH, nKV, hd, invSqrt=inv, cachePos=c0)
        torch.cuda.synchronize()
        what = f"case {case}: S={S} cachePos={c0} nH={nH} nKV={nKV} hd={hd}"
        assert ops.device_status(raise_on_flags=False) == 0, what
        got = host(out)
        assert np.isfinite(got).all(), what
        rows = np.array(sorted(set(range(0, S, max(1, S // 12))) | {S - 1, min(S - 1, 127), min(S - 1, 128)}), np.uint32)
        want = oracle.prefill_f16_rows(host(q), host(k), host(v), rows, S, nH, nKV, hd, inv, cachePos=c0)
        assert_close(got[rows], want, rtol=RTOL16, atol=ATOL16, what=what)


def test_many_work_items_per_block():
    """12288 rows x 28 heads = 1344 work items for the persistent blocks (nine and more per block: the
    item slots and every ring index wrap several times); a row sample against the oracle."""
    from concurrent.futures import ThreadPoolExecutor
    S, nH, nKV, hd = 12288, 28, 4, 128
    inv = 1.0 / math.sqrt(hd)
    g = torch.Generator(device="cuda")
    g.manual_seed(12288)
    q = torch.randn((S, nH, hd), device="cuda", generator=g)
    k = torch.randn((S, nKV, hd), device="cuda", generator=g)
    v = torch.randn((S, nKV, hd), device="cuda", generator=g)
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_f16(q, k, v, out, _scratch(S, nH, nKV, 0), S, nH, nKV, hd, invSqrt=inv)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = host(out)
    assert np.isfinite(got).all()
    rows = sorted(set(range(5, S, 1024)) | {0, 127, 128, 255, 256, 6143, 6144, S - 257, S - 129, S - 128, S - 1})
    hq, hk, hv = host(q), host(k), host(v)
    parts = np.array_split(np.array(rows, np.uint32), 8)
    with ThreadPoolExecutor(8) as ex:
        want = np.concatenate(list(ex.map(lambda r: oracle.prefill_f16_rows(hq, hk, hv, r, S, nH, nKV, hd, inv), parts)))
    assert_close(got[rows], want, rtol=RTOL16, atol=ATOL16, what="12288 rows, row sample")


def test_long_rows_and_peaked_scores():
    # 1536 rows: 12 query tiles, lazy rescale exercised by scores with a wide range
    q, k, v, got, inv = _run(1536, 4, 2, seed=5, scale=6.0)
    q16, k16, v16 = (x.astype(np.float16) for x in (q, k, v))
    exact = oracle.attention_f64(q16.astype(np.float32), k16, v16, None, None, 1536, 4, 2, 128, 0, inv)
    assert_close(got, exact, rtol=RTOL16, atol=ATOL16, what="peaked scores")


def test_matches_f32_causal_kernel_within_fp16_tolerance():
    q, k, v, got, inv = _run(384, 8, 4, seed=9)
    out = torch.empty((384, 8, 128), device="cuda")
    ops.prefill_kv(dev(q), dev(k), dev(v), out, 384, 8, 4, 128, 0, invSqrt=inv)
    assert_close(got, host(out), rtol=RTOL16, atol=2e-2, what="fp16 tcgen05 vs f32 kernel")


def test_scratch_too_small_is_refused():
    q = torch.zeros((128, 4, 128), device="cuda")
    k = torch.zeros((128, 2, 128), device="cuda")
    s = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.TcError) as e:
        ops.prefill_f16(q, k, k, q.clone(), s, 128, 4, 2, 128)
    assert e.value.code == capi.TC_EWORKSPACE


def _scratch(S, nH, nKV, cachePos, hd=128):
    n = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd, cachePos=cachePos)
    buf = torch.empty(n + 1024, dtype=torch.uint8, device="cuda")
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + n]


@pytest.mark.parametrize("cachePos,S,nH,nKV", [(100, 300, 4, 2), (64, 64, 2, 1), (1, 1, 4, 4), (513, 257, 7, 1), (1000, 40, 8, 2)])
def test_continued_prefill_over_an_existing_cache(cachePos, S, nH, nKV):
    """Query rows at positions cachePos.. over cache rows [0, cachePos + S): positions that are no
    multiple of the 64-token KV tile, a diagonal that crosses three tiles, a single row."""
    hd = 128
    rng = np.random.default_rng(cachePos + S)
    total = cachePos + S
    q = rng.standard_normal((S, nH, hd), dtype=np.float32)
    k = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    v = rng.standard_normal((total, nKV, hd), dtype=np.float32)
    inv = 1.0 / math.sqrt(hd)
    # rows behind the window of this call: must never be read as data
    kd = torch.cat([dev(k), torch.full((70, nKV, hd), float("nan"), device="cuda")])
    vd = torch.cat([dev(v), torch.full((70, nKV, hd), float("nan"), device="cuda")])
    out = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_f16(dev(q), kd, vd, out, _scratch(S, nH, nKV, cachePos), S, nH, nKV, hd, invSqrt=inv, cachePos=cachePos)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = oracle.prefill_f16_rows(q, k, v, np.arange(S), S, nH, nKV, hd, inv, cachePos=cachePos)
    assert_close(host(out), want, rtol=RTOL16, atol=ATOL16, what=f"continued prefill at {cachePos}+{S}")


def test_eight_chunks_of_512_equal_one_prefill_of_4096():
    """The engine feeds a long prompt in 512-token calls (ModelForward.cpp:115-127).  Every chunk runs on
    the tensor-core kernel; the chunks together equal the single call and both match the oracle."""
    nH, nKV, hd, S, C = 28, 4, 128, 4096, 512
    inv = 1.0 / math.sqrt(hd)
    g = torch.Generator(device="cuda")
    g.manual_seed(77)
    q = torch.randn((S, nH, hd), generator=g, device="cuda")
    k = torch.randn((S, nKV, hd), generator=g, device="cuda")
    v = torch.randn((S, nKV, hd), generator=g, device="cuda")
    whole = torch.full((S, nH, hd), float("nan"), device="cuda")
    ops.prefill_f16(q, k, v, whole, _scratch(S, nH, nKV, 0), S, nH, nKV, hd, invSqrt=inv)
    parts = torch.full((S, nH, hd), float("nan"), device="cuda")
    sc = _scratch(C, nH, nKV, S - C)
    for c0 in range(0, S, C):
        ops.prefill_f16(q[c0:c0 + C], k, v, parts[c0:c0 + C], sc, C, nH, nKV, hd, invSqrt=inv, cachePos=c0)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(host(parts), host(whole), rtol=RTOL16, atol=ATOL16, what="8 x 512 against 1 x 4096")
    rows = np.array(sorted(set(range(0, S, 128)) | {511, 512, 513, 1023, 1024, 2047, 2048, 3583, 3584} | set(range(S - 32, S))), np.uint32)
    want = oracle.prefill_f16_rows(host(q), host(k), host(v), rows, S, nH, nKV, hd, inv)
    assert_close(host(parts)[rows], want, rtol=RTOL16, atol=ATOL16, what="chunked prefill against the oracle")
    assert_close(host(whole)[rows], want, rtol=RTOL16, atol=ATOL16, what="single prefill against the oracle")
