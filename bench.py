#!/usr/bin/env python
"""Benchmark of the attention hot path.

Default workload (`--workload decode32k`): Qwen2.5-7B-shaped decode attention over
an int8 KV store at context 32768 -- 28 query heads, 4 KV heads, head_dim 128,
batch 1 per GPU, one decode step = the attention of all 28 layers (each layer has
its own KV pool, so a step streams 28 x 34.6 MB = 969 MB, far more than the 126 MB
L2: no layer's KV survives in cache until the next step).  Metric: algorithmic KV
bytes (int8 rows + f32 scales, read once) per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload decode32k|decode32k_b8|decode8k_b8|decode8k_b1|c4_32b_128k|c4_heads|
                                c4_ctxsplit|ragged64|prefill4k]

N > 1 (torchrun): every rank runs the same per-GPU workload on its own sequences
(sharding by sequence, no data-path collective) -- weak scaling; the time is the
max over ranks, the value the sum of bytes over ranks divided by it.

`--impl reference` times the reference engine's CPU attention path (its own
thread pool and AVX-512 leaf kernels behind the restated task loop, built from
the reference sources into oracle/_ref; the plain C restatement when that
library is absent) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (nHeads, nKV, hd, ctx, batch, layers)
    "decode32k": (28, 4, 128, 32768, 1, 28),
    "decode8k_b8": (28, 4, 128, 8192, 8, 28),
    "decode8k_b1": (28, 4, 128, 8192, 1, 28),
    "decode32k_b8": (28, 4, 128, 32768, 8, 8),   # 8 of the 28 layers resident (8 x 277 MB)
    "c4_32b_128k": (40, 8, 128, 131072, 1, 8),  # 8 of the 64 layers resident (64 x 277 MB pools are cycled per 8)
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid = uuid
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(nKV, hd, tokens):
    """int8 K and V rows plus one f32 scale each per (token, kv head), read once."""
    return tokens * nKV * 2 * (hd + 4)


# ---------------------------------------------------------------------------------
# CPU baseline / reference arm
# ---------------------------------------------------------------------------------

class CpuAttention:
    """The reference CPU attention path on ONE layer of a decode workload (the CPU
    engine keeps K/V in f32 only, so it attends over the dequantised f32 copy of the
    int8 store), or on a slice of query rows of the prefill workload."""

    def __init__(self, nH, nKV, hd, ctx, q_rows=1, threads=0):
        import numpy as np

        import oracle
        from tinycoder_inference_b200 import synth

        self.shape = (nH, nKV, hd, ctx, q_rows)
        self.q = synth.normal(2, 1, (q_rows, nH, hd))
        k = synth.normal(2, 2, (ctx, nKV, hd))
        v = synth.normal(2, 3, (ctx, nKV, hd))
        if q_rows == 1:
            k8, v8, ks, vs = oracle.quant_kv8(k, v, nKV, hd)
            k = (k8.astype(np.float32) * ks[:, :, None]).astype(np.float32)
            v = (v8.astype(np.float32) * vs[:, :, None]).astype(np.float32)
        self.k, self.v = k, v
        self.use_ref = oracle.ref_available() and oracle.ref().has_avx512()
        if self.use_ref:
            self.ref = oracle.ref()
            self.cores = self.ref.pool_init(threads)
            self.kind = "reference"
            self.how = (f"reference ThreadPool::parallelFor2D({q_rows} x {nKV} tasks) + AVX-512 dot/axpy leaves, "
                        "restated attentionFused task loop")
        else:
            self.oracle = oracle
            self.cores = 1
            self.kind = "port"
            self.how = "scalar C restatement of Model::attentionFused"

    def run(self):
        nH, nKV, hd, ctx, rows = self.shape
        if self.use_ref:
            return self.ref.attention_fused(self.q, self.k, self.v, ctx - rows, rows, nH, nKV, hd)
        return self.oracle.attention_fused_cpu(self.q, self.k, self.v, rows, ctx - rows, nH, nKV, hd)

    def time(self, reps):
        t0 = time.perf_counter()
        for _ in range(reps):
            self.run()
        return (time.perf_counter() - t0) / reps


def cpu_attention_sample(nH, nKV, hd, ctx, budget_s=12.0, threads=0):
    """(seconds per layer, cores, kind, sample text) on a bounded sample."""
    c = CpuAttention(nH, nKV, hd, ctx, 1, threads)
    one = c.time(1)
    reps = max(1, min(400, int(budget_s / max(one, 1e-6))))
    per_layer = c.time(reps)
    return per_layer, c.cores, c.kind, f"1 layer x {reps} repetitions, f32 copy of the int8 store, ctx {ctx}; {c.how}"


def run_reference(args):
    """The reference arm: the reference engine's CPU implementation of the path on the
    host cores.  A step is a bounded sample: one layer of the decode workload, or the
    last 32 query rows (full 4096-row causal prefix each) of the prefill workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "prefill4k":
        S, nH, nKV, hd, layers, rows = 4096, 28, 4, 128, 4, 32
        c = CpuAttention(nH, nKV, hd, S, rows)
        flops = sum(4.0 * hd * nH * (S - rows + r + 1) for r in range(rows))
        metric, unit = "prefill_attn_tflops_s4096", "TFLOP/s"
        per_unit = lambda t: flops / t / 1e12  # noqa: E731
        sample = f"last {rows} query rows of one layer at the full causal prefix, f32; {c.how}"
        cfg = {"workload": f"prefill4k: causal prefill, {S} rows, {nH} q heads / {nKV} kv heads / head_dim {hd} "
                           "(CPU arm: a 32-row slice, f32)"}
        ms_scale = (2.0 * hd * nH * S * (S + 1)) / flops * layers
    else:
        # sharded / ragged workloads: the CPU arm times one layer of their shape (the 131072-row
        # sequence for the 32B workloads; one 32768-row sequence for the ragged mix)
        wl = {"c4_heads": "c4_32b_128k", "c4_ctxsplit": "c4_32b_128k", "ragged64": "decode32k"}.get(args.workload,
                                                                                                   args.workload)
        nH, nKV, hd, ctx, batch, layers = WORKLOADS[wl]
        c = CpuAttention(nH, nKV, hd, ctx, 1)
        nbytes = algorithmic_bytes(nKV, hd, ctx)
        metric = ("decode_attn_kv_gbs_ctx32k" if args.workload == "decode32k"
                  else f"decode_attn_kv_gbs_{args.workload}")
        unit = "GB/s"
        per_unit = lambda t: nbytes / t / 1e9  # noqa: E731
        sample = f"one layer of one sequence per step, f32 copy of the int8 store, ctx {ctx}; {c.how}"
        cfg = workload_config(wl, args.gpus)
        ms_scale = layers * batch
    one = c.time(1)
    # keep the whole run within a few minutes whatever K and W are
    per_step_reps = 1
    total = (args.steps + args.warmup) * one
    steps, warmup = args.steps, args.warmup
    if total > 150.0:
        warmup = min(warmup, 3)
        steps = max(1, int(150.0 / one) - warmup)
    for _ in range(warmup):
        c.run()
    per = c.time(steps * per_step_reps)
    val = per_unit(per)
    line = {
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": per * ms_scale * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": val, "unit": unit, "cores": c.cores, "kind": c.kind, "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, gpus):
    nH, nKV, hd, ctx, batch, layers = WORKLOADS[name]
    return {"workload": f"{name}: {nH} q heads / {nKV} kv heads / head_dim {hd}, int8 KV, context {ctx}, "
                        f"batch {batch} per GPU, {layers} layers per step",
            "sharding": "by sequence, one replica of the workload per GPU, no collective" if gpus > 1 else "single GPU",
            "l2": f"inputs larger than L2: a step streams {layers} distinct KV pools "
                  f"({layers * batch * algorithmic_bytes(nKV, hd, ctx) / 1e6:.0f} MB)",
            "launch": "cuda_graph; kernels chained by programmatic dependent launch (old KV rows stream in "
                      "while the previous kernel drains; us_per_layer_plain_stream_order is the same step without it)"}


# ---------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------

def run_prefill(args):
    """Qwen2.5-7B-shaped causal prefill: 4096 rows, 28 q heads, 4 kv heads, head_dim 128.
    A step = the fp16 twins, the tcgen05 attention kernel and the int8 mirror of all
    4096 K/V rows, for `layers` layers with their own inputs (4 x 126 MB > L2)."""
    import torch
    import torch.distributed as dist

    from tinycoder_inference_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    S, nH, nKV, hd, layers = 4096, 28, 4, 128, 4
    inv = 1.0 / math.sqrt(hd)
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE003 + rank)
    q = torch.randn((layers, S, nH, hd), generator=g, device=dev)
    k = torch.randn((layers, S, nKV, hd), generator=g, device=dev)
    v = torch.randn((layers, S, nKV, hd), generator=g, device=dev)
    # the reference rounds the operands to fp16; do it to the inputs so both arms see the same values
    q, k, v = (x.half().float() for x in (q, k, v))
    out = torch.empty_like(q)
    k8 = torch.empty((layers, S + 16, nKV, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.empty((layers, S + 16, nKV), device=dev)
    vs = torch.empty_like(ks)
    nbytes = ops.prefill_f16_scratch_bytes(S, nH, nKV, hd)
    scratch = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
    off = (-scratch.data_ptr()) % 1024
    scratch = scratch[off:off + nbytes]

    def step():
        for l in range(layers):
            ops.prefill_f16(q[l], k[l], v[l], out[l], scratch, S, nH, nKV, hd, invSqrt=inv)
            ops.kv_quantize_i8(k[l], v[l], k8[l], v8[l], ks[l], vs[l], S, nKV, hd)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    props = torch.cuda.get_device_properties(local)
    gpu_id = str(getattr(props, "uuid", local))
    if "-" in gpu_id and not gpu_id.startswith("GPU-"):
        gpu_id = "GPU-" + gpu_id
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    # attention kernel alone (the dominant kernel), same inputs
    ek0, ek1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kern_ms = 0.0
    reps = max(3, min(args.steps, 20))
    for r in range(reps):
        l = r % layers
        ops.prefill_f16(q[l], k[l], v[l], out[l], scratch, S, nH, nKV, hd, invSqrt=inv)
    torch.cuda.synchronize()
    ek0.record()
    for r in range(reps):
        l = r % layers
        ops.prefill_f16(q[l], k[l], v[l], out[l], scratch, S, nH, nKV, hd, invSqrt=inv)
    ek1.record()
    torch.cuda.synchronize()
    kern_ms = ek0.elapsed_time(ek1) / reps
    # end to end with host buffers: q, k, v of a layer from pinned memory, the output back
    hq, hk, hv = q[0].cpu().pin_memory(), k[0].cpu().pin_memory(), v[0].cpu().pin_memory()
    hout = torch.empty_like(hq).pin_memory()
    dq, dk, dv, dout = torch.empty_like(q[0]), torch.empty_like(k[0]), torch.empty_like(v[0]), torch.empty_like(q[0])

    def e2e_step():
        for l in range(layers):
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            ops.prefill_f16(dq, dk, dv, dout, scratch, S, nH, nKV, hd, invSqrt=inv)
            ops.kv_quantize_i8(dk, dv, k8[l], v8[l], ks[l], vs[l], S, nKV, hd)
            hout.copy_(dout, non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    n_e2e = max(2, min(args.steps, 10))
    for _ in range(n_e2e):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    flags = ops.device_status()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    flops_layer = 2.0 * hd * nH * S * (S + 1)  # causal count: QK^T and PV over the lower triangle
    pk = peaks()
    tf = world * layers * flops_layer / (ms_per_step * 1e-3) / 1e12
    tf_kernel = flops_layer / (kern_ms * 1e-3) / 1e12
    line = {
        "metric": "prefill_attn_tflops_s4096", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3 / layers,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 operands, f32 accumulate (tcgen05), f32 softmax", "data": "synthetic",
        "config": {"workload": f"prefill4k: causal prefill, {S} rows, {nH} q heads / {nKV} kv heads / head_dim {hd}, "
                               f"{layers} layers per step, each with fp16 twins + attention + int8 mirror of all rows",
                   "l2": f"inputs larger than L2: {layers} layers x 126 MB of q/k/v/out"},
        "roofline": {"bound": "tensor", "achieved": tf_kernel, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tf_kernel / pk["bf16_tflops"], "peak_source": pk["source"] + " (burst)", "traffic": None,
                     "note": "attention launch alone (f32->fp16 twins + tcgen05 kernel), causal flop count"},
        "e2e": {"value": world * layers * flops_layer / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": layers * (S * nH * hd + 2 * S * nKV * hd) * 4,
                "d2h_bytes_per_step": layers * S * nH * hd * 4},
        "gpu_launches": args.steps * layers * 3, "clocks": clocks, "device_error_flags": flags,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def quick_decode(name, dev, steps=20, warmup=5):
    """Device-resident decode measurement of one workload (graph + dependent launch), for
    the secondary figures of the default line."""
    import torch

    from tinycoder_inference_b200 import ops

    nH, nKV, hd, ctx, batch, layers = WORKLOADS[name]
    inv = 1.0 / math.sqrt(hd)
    rows = ctx + 16
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE012)
    k8 = torch.empty((layers, batch, rows, nKV, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.zeros((layers, batch, rows, nKV), device=dev)
    vs = torch.zeros_like(ks)
    for l in range(layers):
        for b in range(batch):
            kf = torch.randn((ctx, nKV, hd), generator=g, device=dev)
            vf = torch.randn((ctx, nKV, hd), generator=g, device=dev)
            ops.kv_quantize_i8(kf, vf, k8[l, b], v8[l, b], ks[l, b], vs[l, b], ctx, nKV, hd)
    q = torch.randn((layers, batch, nH, hd), generator=g, device=dev)
    out = torch.empty_like(q)
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(batch, nH, hd, chunks)

    def step():
        for l in range(layers):
            ops.decode_i8_batch(q[l], k8[l], v8[l], ks[l], vs[l], out[l], ws, None, batch, nH, nKV, hd, ctx, chunks,
                                rows_per_seq=rows, invSqrt=inv, pdl=True, prefetch_rows=ctx - 1,
                                next_kv=(k8[(l + 1) % layers], v8[(l + 1) % layers]))

    step()
    torch.cuda.synchronize()
    s_ = torch.cuda.Stream()
    s_.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s_):
        step()
    torch.cuda.current_stream().wait_stream(s_)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        step()
    for _ in range(warmup):
        gr.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    gbs = layers * batch * algorithmic_bytes(nKV, hd, ctx) / (ms * 1e-3) / 1e9
    pk = peaks()
    return {"workload": workload_config(name, 1)["workload"], "us_per_layer": ms * 1e3 / layers, "value": gbs,
            "unit": "GB/s", "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "steps": steps, "warmup": warmup}


def run_ragged(args):
    """Batched decode serving mix: 64 sequences with context lengths drawn uniformly from
    [512, 32768] by seed (28 q heads, 4 kv heads, head_dim 128, int8 KV), one decode step =
    28 layers.  The 64 sequences are dealt to the ranks so that the TOKEN counts balance
    (longest first onto the lightest rank) -- strong scaling, no collective.  Every rank keeps
    4 layer pools of its sequences resident and cycles them 7 times per step."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from tinycoder_inference_b200 import ops, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    nH, nKV, hd, nseq, layers, resident = 28, 4, 128, 64, 28, 4
    inv = 1.0 / math.sqrt(hd)
    rng = np.random.Generator(np.random.Philox(key=[0x7C0DE005, 0]))
    lens_all = (512 + rng.integers(0, 32257, nseq, dtype=np.uint64)).astype(np.int64)   # 512 + (u64 mod 32257)
    mine = sharding.plan_sequence_shards(lens_all.tolist(), world)[rank]
    lens = lens_all[mine]
    B = len(mine)
    base = np.zeros(B, dtype=np.uint64)
    base[1:] = np.cumsum(lens[:-1] + 16)      # 16 rows of slack behind every sequence
    rows = int((lens + 16).sum())
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE005 + rank)
    k8 = torch.empty((resident, rows, nKV, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.zeros((resident, rows, nKV), device=dev)
    vs = torch.zeros_like(ks)
    blk = 32768
    for l in range(resident):
        for r0 in range(0, rows, blk):
            n = min(blk, rows - r0)
            kf = torch.randn((n, nKV, hd), generator=g, device=dev)
            vf = torch.randn((n, nKV, hd), generator=g, device=dev)
            ops.kv_quantize_i8(kf, vf, k8[l], v8[l], ks[l], vs[l], n, nKV, hd, dst_base=r0)
    q = torch.randn((resident, B, nH, hd), generator=g, device=dev)
    out = torch.empty_like(q)
    dlens = torch.tensor(lens, dtype=torch.int32, device=dev)
    dbase = torch.tensor(base.astype(np.int64), dtype=torch.int64, device=dev)
    maxlen = int(lens.max())
    _, chunks = ops.split_geometry(maxlen, nH, hd)
    chunks = min(chunks, 64)
    ws = ops.workspace(B, nH, hd, chunks)

    def step():
        for l in range(layers):
            r = l % resident
            ops.decode_i8_batch(q[r], k8[r], v8[r], ks[r], vs[r], out[r], ws, dlens, B, nH, nKV, hd, maxlen, chunks,
                                row_base=dbase, invSqrt=inv, pdl=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step()
    torch.cuda.synchronize()
    s_ = torch.cuda.Stream()
    s_.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s_):
        step()
    torch.cuda.current_stream().wait_stream(s_)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        step()
    for _ in range(args.warmup):
        gr.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gr.replay()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    flags = ops.device_status()
    if rank == 0:
        tokens = int(lens_all.sum())
        total_bytes = layers * algorithmic_bytes(nKV, hd, tokens)
        val = total_bytes / (ms_per_step * 1e-3) / 1e9
        pk = peaks()
        line = {
            "metric": "decode_attn_kv_gbs_ragged64", "value": val, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3 / layers, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 KV, f32 q/out", "data": "synthetic",
            "config": {"workload": f"ragged64: {nseq} sequences, context lengths uniform in [512, 32768] by seed "
                                   f"({tokens} tokens), {nH} q heads / {nKV} kv heads / head_dim {hd}, int8 KV, "
                                   f"{layers} layers per step ({resident} resident pools cycled)",
                       "sharding": "whole sequences dealt to ranks by token count (longest first), no collective",
                       "rank0_sequences": B, "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": val / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": val / world / pk["hbm_gbs"], "peak_source": pk["source"], "traffic": None,
                         "note": "per-GPU share of the algorithmic bytes over the step time"},
            "gpu_launches": args.steps * layers * 2, "device_error_flags": flags,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_sharded(args):
    """Qwen2.5-32B-shaped long-context decode (40 q heads, 8 kv heads, head_dim 128, ctx
    131072, int8 KV), ONE sequence split over the ranks -- strong scaling:
      c4_heads    : kv-head groups (each rank holds nKV/N heads of every row; disjoint output
                    slices, no collective on the data path);
      c4_ctxsplit : the context axis (each rank holds all heads of ctx/N rows; split-KV
                    partials are all-gathered over NCCL and merged on every rank).
    8 layers are resident per rank and cycled (a step = 8 layers)."""
    import torch
    import torch.distributed as dist

    from tinycoder_inference_b200 import ops, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    nH, nKV, hd, ctx, layers = 40, 8, 128, 131072, 8
    inv = 1.0 / math.sqrt(hd)
    by_ctx = args.workload == "c4_ctxsplit"
    if by_ctx:
        lo, hi = sharding.plan_context_ranges(ctx, world)[rank]
        my_rows, my_kv, my_q = hi - lo, nKV, nH
    else:
        if nKV % world != 0:
            raise SystemExit(f"c4_heads needs a rank count that divides {nKV} kv heads")
        sh = sharding.plan_kv_head_shards(nH, nKV, world)[rank]
        my_rows, my_kv, my_q = ctx, sh.kv_hi - sh.kv_lo, sh.q_hi - sh.q_lo
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE004 + rank)
    rows = my_rows + 16
    k8 = torch.empty((layers, rows, my_kv, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.zeros((layers, rows, my_kv), device=dev)
    vs = torch.zeros_like(ks)
    step_rows = 16384
    for l in range(layers):
        for r0 in range(0, my_rows, step_rows):
            n = min(step_rows, my_rows - r0)
            kf = torch.randn((n, my_kv, hd), generator=g, device=dev)
            vf = torch.randn((n, my_kv, hd), generator=g, device=dev)
            ops.kv_quantize_i8(kf, vf, k8[l], v8[l], ks[l], vs[l], n, my_kv, hd, dst_base=r0)
    g2 = torch.Generator(device=dev)
    g2.manual_seed(0x7C0DE005)                 # q is the same on every rank
    q_all = torch.randn((layers, 1, nH, hd), generator=g2, device=dev)
    q = q_all if by_ctx else q_all[:, :, sh.q_lo:sh.q_hi].contiguous()
    out = torch.empty((layers, 1, my_q, hd), device=dev)
    chunk, chunks = ops.split_geometry(ctx, nH, hd)
    chunks = min(chunks, 128)
    ws = ops.workspace(1, my_q, hd, chunks)
    splitter = sharding.ContextSplitDecoder(my_q, my_kv, hd, my_rows, chunk_slots=64,
                                            exchange=args.exchange) if by_ctx else None
    if by_ctx and world > 1 and args.exchange == "p2p":
        # the library's own exchange must agree with the NCCL all-gather path before anything is timed
        chk = sharding.ContextSplitDecoder(my_q, my_kv, hd, my_rows, chunk_slots=64, exchange="nccl")
        o1, o2 = torch.empty_like(out[0]), torch.empty_like(out[0])
        splitter(q[0], k8[0], v8[0], ks[0], vs[0], o1, my_rows, invSqrt=inv)
        chk(q[0], k8[0], v8[0], ks[0], vs[0], o2, my_rows, invSqrt=inv)
        torch.cuda.synchronize()
        if not torch.allclose(o1, o2, rtol=1e-4, atol=1e-6):
            raise SystemExit("context split: the two exchange paths disagree")
        del chk

    def step_plain():
        for l in range(layers):
            if by_ctx:
                splitter(q[l], k8[l], v8[l], ks[l], vs[l], out[l], my_rows, invSqrt=inv, pdl=True)
            else:
                ops.decode_i8_batch(q[l], k8[l], v8[l], ks[l], vs[l], out[l], ws, None, 1, my_q, my_kv, hd, my_rows,
                                    chunks, invSqrt=inv, pdl=True, prefetch_rows=my_rows - 1)

    step_plain()
    torch.cuda.synchronize()
    if args.no_graph or (by_ctx and args.exchange == "nccl"):
        step = step_plain      # (the NCCL path is timed as plain launches)
    else:
        s_ = torch.cuda.Stream()
        s_.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s_):
            step_plain()
        torch.cuda.current_stream().wait_stream(s_)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            step_plain()
        step = gr.replay

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    flags = ops.device_status()
    if rank == 0:
        total_bytes = layers * algorithmic_bytes(nKV, hd, ctx)       # the whole sequence, all ranks together
        pk = peaks()
        val = total_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": f"decode_attn_kv_gbs_{args.workload}", "value": val, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3 / layers, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 KV, f32 q/out", "data": "synthetic",
            "config": {"workload": f"{args.workload}: 40 q heads / 8 kv heads / head_dim 128, int8 KV, one sequence of "
                                   f"{ctx} rows, {layers} layers per step",
                       "sharding": (("context axis: ctx/N rows per rank; "
                                     + ("each rank's merged partial is stored into every peer over NVLink and merged "
                                        "there, one kernel per rank (no collective library call)"
                                        if args.exchange == "p2p" else
                                        "partials all-gathered over NCCL and merged"))
                                    if by_ctx else "kv-head groups: nKV/N heads per rank, no data-path collective"),
                       "launch": "plain launches" if args.no_graph or (by_ctx and args.exchange == "nccl")
                                 else "cuda_graph",
                       "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": val / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": val / world / pk["hbm_gbs"], "peak_source": pk["source"], "traffic": None,
                         "note": "per-GPU share of the algorithmic bytes over the step time"},
            "gpu_launches": args.steps * layers * 2, "device_error_flags": flags,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode32k", choices=sorted(WORKLOADS) + ["prefill4k", "c4_heads", "c4_ctxsplit", "ragged64"])
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="c4_ctxsplit: partials exchanged by the library's own kernel over peer memory, or by NCCL")
    ap.add_argument("--no-next-prefetch", action="store_true",
                    help="do not hint the next layer's pools to the decode call (L2 prefetch while a layer drains)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary batch-8 measurement of the default line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream order between the kernels of a step")
    ap.add_argument("--partials-only", action="store_true", help="diagnostic: skip the merge launch")
    ap.add_argument("--fused-merge", action="store_true",
                    help="merge the chunk partials inside the decode kernel (last-arriving block) instead of a second launch")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "prefill4k":
        run_prefill(args)
        return
    if args.workload in ("c4_heads", "c4_ctxsplit"):
        run_sharded(args)
        return
    if args.workload == "ragged64":
        run_ragged(args)
        return

    import torch
    import torch.distributed as dist

    from tinycoder_inference_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)

    nH, nKV, hd, ctx, batch, layers = WORKLOADS[args.workload]
    inv = 1.0 / math.sqrt(hd)
    rows = ctx + 16
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE002 + rank)
    # one int8 pool per layer holding `batch` sequences; built by the library's own
    # quantiser from seeded N(0,1) f32 rows (bit-exact with the reference quantiser)
    k8 = torch.empty((layers, batch, rows, nKV, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.zeros((layers, batch, rows, nKV), device=dev)
    vs = torch.zeros_like(ks)
    for l in range(layers):
        for b in range(batch):
            kf = torch.randn((ctx, nKV, hd), generator=g, device=dev)
            vf = torch.randn((ctx, nKV, hd), generator=g, device=dev)
            ops.kv_quantize_i8(kf, vf, k8[l, b], v8[l, b], ks[l, b], vs[l, b], ctx, nKV, hd)
    q = torch.randn((layers, batch, nH, hd), generator=g, device=dev)
    out = torch.empty_like(q)
    chunk, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(batch, nH, hd, chunks)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()

    lens_arg = None  # host lengths: every sequence holds exactly ctx rows
    tickets = torch.zeros(batch * nKV, dtype=torch.int32, device=dev) if args.fused_merge else None

    def step(pdl):
        # rows [0, ctx-1) are old rows; the last row is the one a decode step appends
        for l in range(layers):
            nxt = None if args.no_next_prefetch else (k8[(l + 1) % layers], v8[(l + 1) % layers])
            ops.decode_i8_batch(q[l], k8[l], v8[l], ks[l], vs[l], out[l], ws, lens_arg, batch, nH, nKV, hd, ctx,
                                chunks, rows_per_seq=rows, invSqrt=inv, pdl=pdl, prefetch_rows=ctx - 1,
                                partials_only=args.partials_only, next_kv=nxt, tickets=tickets)

    launches_per_step = layers * 2
    step(False)
    step(True)
    torch.cuda.synchronize()

    def capture(pdl):
        if args.no_graph:
            return lambda: step(pdl)
        s_ = torch.cuda.Stream()
        s_.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s_):
            step(pdl)
        torch.cuda.current_stream().wait_stream(s_)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            step(pdl)
        return gr.replay

    run_plain = capture(False)
    run = capture(True) if not args.no_pdl else run_plain

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    props = torch.cuda.get_device_properties(local)
    gpu_id = str(getattr(props, "uuid", local))
    if "-" in gpu_id and not gpu_id.startswith("GPU-"):
        gpu_id = "GPU-" + gpu_id
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        run()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    # the same step without programmatic dependent launch (no overlap between kernels)
    for _ in range(3):
        run_plain()
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_plain()
    e1.record()
    barrier()
    ms_plain_per_step = e0.elapsed_time(e1) / args.steps
    bytes_per_step_gpu = layers * batch * algorithmic_bytes(nKV, hd, ctx)
    value = world * bytes_per_step_gpu / (ms_per_step * 1e-3) / 1e9
    us_per_layer = ms_per_step * 1e3 / layers

    # ---- end to end through the C ABI with HOST buffers ---------------------------
    # A step: the new token's q, k, v of every layer come from pinned host memory (one
    # asynchronous copy each), then per layer k/v are quantised and appended at the last row
    # and attention runs (the captured launch sequence of the step), and the step's outputs go
    # back to pinned host memory; the host waits for them.
    hq = torch.randn((layers, batch, nH, hd)).pin_memory()
    hk = torch.randn((layers, batch, nKV, hd)).pin_memory()
    hv = torch.randn((layers, batch, nKV, hd)).pin_memory()
    hout = torch.empty((layers, batch, nH, hd)).pin_memory()
    dq = torch.empty((layers, batch, nH, hd), device=dev)
    dk = torch.empty((layers, batch, nKV, hd), device=dev)
    dv = torch.empty((layers, batch, nKV, hd), device=dev)
    dout = torch.empty((layers, batch, nH, hd), device=dev)

    def e2e_layers():
        for l in range(layers):
            ops.kv_quantize_i8_batch(dk[l], dv[l], k8[l], v8[l], ks[l], vs[l], batch, nKV, hd, rows_per_seq=rows,
                                     pos=ctx - 1)
            nxt = None if args.no_next_prefetch else (k8[(l + 1) % layers], v8[(l + 1) % layers])
            ops.decode_i8_batch(dq[l], k8[l], v8[l], ks[l], vs[l], dout[l], ws, lens_arg, batch, nH, nKV, hd, ctx,
                                chunks, rows_per_seq=rows, invSqrt=inv, pdl=not args.no_pdl, prefetch_rows=ctx - 1,
                                next_kv=nxt, tickets=tickets)

    if args.no_graph:
        e2e_run = e2e_layers
    else:
        e2e_layers()
        torch.cuda.synchronize()
        s2 = torch.cuda.Stream()
        s2.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s2):
            e2e_layers()
        torch.cuda.current_stream().wait_stream(s2)
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            e2e_layers()
        e2e_run = g2.replay

    def e2e_step():
        dq.copy_(hq, non_blocking=True)
        dk.copy_(hk, non_blocking=True)
        dv.copy_(hv, non_blocking=True)
        e2e_run()
        hout.copy_(dout, non_blocking=True)
        torch.cuda.synchronize()

    e2e_steps = max(3, min(args.steps, 50))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(t.item()) / e2e_steps
    e2e_value = world * bytes_per_step_gpu / (e2e_ms_per_step * 1e-3) / 1e9
    clocks = sampler.stop() if rank == 0 else None
    dev_flags = ops.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    per_gpu_gbs = bytes_per_step_gpu / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": "decode_attn_kv_gbs_ctx32k" if args.workload == "decode32k" else f"decode_attn_kv_gbs_{args.workload}",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "us_per_layer": us_per_layer,
        "us_per_layer_plain_stream_order": ms_plain_per_step * 1e3 / layers,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 KV, f32 q/out (fp16 hi+lo tensor-core products, f32 accumulate)",
        "data": "synthetic", "config": workload_config(args.workload, world),
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": per_gpu_gbs / pk["hbm_gbs"], "peak_source": pk["source"],
                     # dram__bytes_read + write of one decodeI8Kernel launch, from the ncu capture
                     # summarised in profiles/decode_i8_ctx32k_b1.md (34.65 MB read, 512 B written:
                     # every KV byte leaves DRAM once); scaled by rows for the other decode shapes
                     "traffic": 34650512.0 * (ctx * nKV * batch) / (32768.0 * 4.0),
                     "note": "algorithmic bytes per layer / (step time / layers); split and merge launches both inside; "
                             "traffic per launch from the committed ncu summary, not measured by this run"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms_per_step,
                "h2d_bytes_per_step": layers * batch * (nH + 2 * nKV) * hd * 4,
                "d2h_bytes_per_step": layers * batch * nH * hd * 4},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "device_error_flags": dev_flags,
    }
    if world == 1 and args.workload == "decode32k" and not args.no_extras:
        # the same shape and context with 8 sequences in the batch: enough rows in flight to be
        # bandwidth-bound rather than latency-bound
        del k8, v8, ks, vs
        torch.cuda.empty_cache()
        line["also"] = [quick_decode("decode32k_b8", dev)]
    if not args.no_cpu_baseline and world == 1:
        per_layer, cores, kind, sample = cpu_attention_sample(nH, nKV, hd, ctx)
        line["cpu_baseline"] = {"value": algorithmic_bytes(nKV, hd, ctx) / per_layer / 1e9, "unit": "GB/s",
                                "cores": cores, "kind": kind, "sample": sample, "us_per_layer": per_layer * 1e6}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
