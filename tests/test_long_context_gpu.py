"""Kernel-level twins of the reference's tool-level gates: the needle probe
(scripts/context_gate.sh: a fact near token 20, the question at the far end of an 8k / 32k / 64k
window) and the two-arm f32-vs-int8 check (BENCHMARKS.md: same top-1, small logit delta)."""
import math

import numpy as np
import pytest
import torch

from tinycoder_inference_b200 import ops

pytestmark = pytest.mark.gpu


def _needle_store(ctx, nKV, hd, needle_row, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    k = torch.randn((ctx, nKV, hd), generator=g, device="cuda") * 0.05
    v = torch.randn((ctx, nKV, hd), generator=g, device="cuda")
    q_dir = torch.randn((nKV, hd), generator=g, device="cuda")
    q_dir = q_dir / q_dir.norm(dim=-1, keepdim=True)
    k[needle_row] = q_dir * 6.0            # the one row every query points at
    return k, v, q_dir


@pytest.mark.parametrize("ctx", [8192, 32768, 65536, 131072])
def test_needle_near_the_start_of_a_long_window(ctx):
    nH, nKV, hd, needle = 8, 2, 128, 20
    k, v, q_dir = _needle_store(ctx, nKV, hd, needle, seed=ctx)
    group = nH // nKV
    q = (q_dir.repeat_interleave(group, dim=0) * 40.0).reshape(1, nH, hd).contiguous()   # score ~ 240 / sqrt(128) = 21
    want = v[needle].repeat_interleave(group, dim=0)                                    # softmax ~ one-hot
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(1, nH, hd, chunks)
    # f32 cache
    out = torch.empty((1, nH, hd), device="cuda")
    ops.decode_kv(q, k, v, out, ws, 1, nH, nKV, hd, ctx - 1, chunks)
    assert torch.allclose(out[0], want, rtol=1e-3, atol=2e-3), "f32 cache lost the needle"
    # int8 store built by the library's quantiser
    k8 = torch.empty((ctx + 16, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.empty_like(k8)
    ks = torch.empty((ctx + 16, nKV), device="cuda")
    vs = torch.empty_like(ks)
    ops.kv_quantize_i8(k, v, k8, v8, ks, vs, ctx, nKV, hd)
    out8 = torch.empty_like(out)
    ops.decode_i8(q, k8, v8, ks, vs, out8, ws, nH, nKV, hd, ctx - 1, chunks)
    v_deq = v8[needle].float() * vs[needle].unsqueeze(-1)
    want8 = v_deq.repeat_interleave(group, dim=0)
    assert torch.allclose(out8[0], want8, rtol=1e-3, atol=2e-3), "int8 store lost the needle"
    torch.cuda.synchronize()
    assert ops.device_status() == 0


def test_int8_and_f32_arms_agree_on_the_same_rows():
    """The reference's two-arm check at kernel level: attention over the int8 store stays within the
    quantisation noise of attention over the f32 cache."""
    nH, nKV, hd, ctx = 28, 4, 128, 6000
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    k = torch.randn((ctx, nKV, hd), generator=g, device="cuda")
    v = torch.randn((ctx, nKV, hd), generator=g, device="cuda")
    q = torch.randn((1, nH, hd), generator=g, device="cuda") * 3.0     # peaked enough for a stable arg-max
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(1, nH, hd, chunks)
    out32 = torch.empty((1, nH, hd), device="cuda")
    ops.decode_kv(q, k, v, out32, ws, 1, nH, nKV, hd, ctx - 1, chunks)
    k8 = torch.empty((ctx + 16, nKV, hd), dtype=torch.int8, device="cuda")
    v8 = torch.empty_like(k8)
    ks = torch.empty((ctx + 16, nKV), device="cuda")
    vs = torch.empty_like(ks)
    ops.kv_quantize_i8(k, v, k8, v8, ks, vs, ctx, nKV, hd)
    out8 = torch.empty_like(out32)
    ops.decode_i8(q, k8, v8, ks, vs, out8, ws, nH, nKV, hd, ctx - 1, chunks)
    delta = (out8 - out32).abs().max().item()
    assert delta < 0.05, f"int8 arm differs from the f32 arm by {delta}"
    cos = torch.nn.functional.cosine_similarity(out8[0], out32[0], dim=-1).min().item()
    assert cos > 0.995, f"int8 and f32 outputs point in different directions (cosine {cos})"
