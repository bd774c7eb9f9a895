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


def load_synth():
    """The seeded input generator, loaded by file path: importing it through the package would
    load the CUDA library, which the CPU arms have no business mapping."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("tc_synth", os.path.join(ROOT, "tinycoder_inference_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


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

        synth = load_synth()
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


def cpu_allcores_sample(nH, nKV, hd, lens, budget_s=10.0):
    """The CPU path with the (sequence x kv-head) pairs of a batch flattened into one task list, so
    that every host core has work (the engine's own decode step hands out only nKV tasks per
    sequence, ModelPrimitives.cpp:258).  Returns None where the reference-built library is absent."""
    import numpy as np

    import oracle

    if not (oracle.ref_available() and oracle.ref().has_avx512()):
        return None
    ref = oracle.ref()
    cores = ref.pool_init(0)
    synth = load_synth()
    B, mx = len(lens), int(max(lens))
    q = synth.normal(3, 1, (B, 1, nH, hd))
    k = synth.normal(3, 2, (B, mx, nKV, hd))
    v = synth.normal(3, 3, (B, mx, nKV, hd))
    pos = np.asarray(lens, np.uint32) - 1

    def once():
        ref.attention_fused(q, k, v, pos, 1, nH, nKV, hd, batch=B, flatten=True)

    once()
    t0 = time.perf_counter()
    once()
    one = time.perf_counter() - t0
    reps = max(1, min(50, int(budget_s / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(reps):
        once()
    per = (time.perf_counter() - t0) / reps
    nbytes = algorithmic_bytes(nKV, hd, int(np.sum(lens)))
    return {"value": nbytes / per / 1e9, "unit": "GB/s", "cores": cores, "kind": "reference",
            "sample": f"{B} sequences of one layer, (sequence x kv head) tasks flattened over all cores (labelled "
                      f"variant: the engine itself runs {nKV} tasks per sequence), f32 K/V, {reps} repetitions",
            "ms_per_layer": per * 1e3}


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
        "steps": steps, "warmup": warmup,
        # a step of this arm is the bounded sample below (one layer / one row slice); the time of the
        # GPU arm's whole step at this rate is an extrapolation and is labelled as one
        "ms_per_step": per * 1e3, "ms_per_full_step_extrapolated": per * ms_scale * 1e3,
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

_DIST = {}


def dist_ctx():
    """(world, rank, local rank, device) of this process; the NCCL group is set up once."""
    import torch
    import torch.distributed as dist

    if not _DIST:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        _DIST.update(world=world, rank=rank, local=local, dev=torch.device("cuda", local))
    return _DIST["world"], _DIST["rank"], _DIST["local"], _DIST["dev"]


def dist_done():
    import torch.distributed as dist

    if _DIST and _DIST["world"] > 1 and dist.is_initialized():
        dist.destroy_process_group()


def max_over_ranks(x, dev):
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    if _DIST.get("world", 1) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def rank_barrier():
    import torch
    import torch.distributed as dist

    if _DIST.get("world", 1) > 1:
        dist.barrier()
    torch.cuda.synchronize()


def parity_record(err, tol_ok, checked):
    """The parity entry of a line: every rank compared part of layer 0 with the CPU checker
    (outside the timed region); the worst rank decides."""
    import torch

    dev = _DIST["dev"]
    worst = max_over_ranks(float(err), dev)
    bad = max_over_ranks(0.0 if tol_ok else 1.0, dev)
    return {"max_abs_err": worst, "ok": bad == 0.0, "checked": checked,
            "bar": "|d| <= 1e-4 + 1e-3 |ref| against the CPU restatement of the reference kernels"}


def run_prefill(args, steps=None, warmup=None, chunk=0, with_cpu=True, with_e2e=True):
    """Qwen2.5-7B-shaped causal prefill: 4096 rows, 28 q heads, 4 kv heads, head_dim 128.
    A step = the fp16 twins with the int8 mirror of all 4096 K/V rows (one launch) and the
    tcgen05 attention kernel, for `layers` layers with their own inputs (4 x 126 MB > L2).  chunk > 0
    feeds every layer's prompt in calls of `chunk` rows over the rows already cached, the way
    the engine's caller cuts long prompts (512-token calls)."""
    import torch

    from tinycoder_inference_b200 import ops

    world, rank, local, dev = dist_ctx()
    steps = steps or args.steps
    warmup = max(3, warmup or args.warmup)
    S, nH, nKV, hd, layers = 4096, 28, 4, 128, 4
    C = chunk or S
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
    nbytes = ops.prefill_f16_scratch_bytes(C, nH, nKV, hd, cachePos=S - C)
    scratch = torch.empty(nbytes + 1024, dtype=torch.uint8, device=dev)
    off = (-scratch.data_ptr()) % 1024
    scratch = scratch[off:off + nbytes]

    def layer(ql, kl, vl, ol, l, mirror=True):
        for c0 in range(0, S, C):
            # the int8 mirror of the new rows comes out of the launch that makes the fp16 twins
            ops.prefill_f16(ql[c0:c0 + C], kl, vl, ol[c0:c0 + C], scratch, C, nH, nKV, hd, invSqrt=inv, cachePos=c0,
                            kv8=(k8[l], v8[l], ks[l], vs[l]) if mirror else None)

    def step():
        for l in range(layers):
            layer(q[l], k[l], v[l], out[l], l)

    props = torch.cuda.get_device_properties(local)
    gpu_id = str(getattr(props, "uuid", local))
    if "-" in gpu_id and not gpu_id.startswith("GPU-"):
        gpu_id = "GPU-" + gpu_id
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    ms_per_step = _time_steps(step, steps, warmup, dev)
    # attention launches alone (the dominant kernel with its fp16 twins), same inputs
    def attn_only():
        for l in range(layers):
            layer(q[l], k[l], v[l], out[l], l, mirror=False)

    kern_ms = _time_steps(attn_only, max(3, min(steps, 20)), 3, dev) / layers
    clocks = sampler.stop() if rank == 0 else None
    e2e = None
    if with_e2e:
        # end to end with host buffers: q, k, v of a layer from pinned memory, the output back
        hq, hk, hv = q[0].cpu().pin_memory(), k[0].cpu().pin_memory(), v[0].cpu().pin_memory()
        hout = torch.empty_like(hq).pin_memory()
        dq, dk, dv, dout = torch.empty_like(q[0]), torch.empty_like(k[0]), torch.empty_like(v[0]), torch.empty_like(q[0])

        def e2e_step():
            for l in range(layers):
                dq.copy_(hq, non_blocking=True)
                dk.copy_(hk, non_blocking=True)
                dv.copy_(hv, non_blocking=True)
                layer(dq, dk, dv, dout, l)
                hout.copy_(dout, non_blocking=True)
            torch.cuda.synchronize()

        e2e_step()
        rank_barrier()
        t0 = time.perf_counter()
        n_e2e = max(2, min(steps, 10))
        for _ in range(n_e2e):
            e2e_step()
        rank_barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / n_e2e, dev)
    flags = ops.device_status()
    if rank != 0:
        return None
    flops_layer = 2.0 * hd * nH * S * (S + 1)  # causal count: QK^T and PV over the lower triangle
    pk = peaks()
    tf = world * layers * flops_layer / (ms_per_step * 1e-3) / 1e12
    tf_kernel = flops_layer / (kern_ms * 1e-3) / 1e12
    calls = S // C
    line = {
        "metric": "prefill_attn_tflops_s4096", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3 / layers,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16 operands, f32 accumulate (tcgen05), f32 softmax", "data": "synthetic",
        "config": {"workload": f"prefill4k{'_chunked' + str(C) if chunk else ''}: causal prefill, {S} rows"
                               + (f" in {calls} calls of {C} rows over the rows already cached" if chunk else "")
                               + f", {nH} q heads / {nKV} kv heads / head_dim {hd}, "
                               f"{layers} layers per step, each with fp16 twins + int8 mirror of all rows (one launch) + attention",
                   "l2": f"inputs larger than L2: {layers} layers x 126 MB of q/k/v/out"},
        "roofline": {"bound": "tensor", "achieved": tf_kernel, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tf_kernel / pk["bf16_tflops"], "peak_source": pk["source"] + " (burst)", "traffic": None,
                     "note": "attention launches alone (f32->fp16 twins + tcgen05 kernel), causal flop count"},
        "gpu_launches": steps * layers * 2 * calls, "clocks": clocks, "device_error_flags": flags,
    }
    if with_e2e:
        line["e2e"] = {"value": world * layers * flops_layer / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": layers * (S * nH * hd + 2 * S * nKV * hd) * 4,
                       "d2h_bytes_per_step": layers * S * nH * hd * 4}
    if with_cpu and world == 1:
        rows = 32
        c = CpuAttention(nH, nKV, hd, S, rows)
        c.run()
        per = c.time(max(1, min(20, int(5.0 / max(c.time(1), 1e-6)))))
        fl = sum(4.0 * hd * nH * (S - rows + r + 1) for r in range(rows))
        line["cpu_baseline"] = {"value": fl / per / 1e12, "unit": "TFLOP/s", "cores": c.cores, "kind": c.kind,
                                "sample": f"last {rows} query rows of one layer at the full causal prefix, f32; {c.how}"}
    return line


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
            "unit": "GB/s", "frac_of_peak_per_gpu": gbs / pk["hbm_gbs"], "bound": "hbm", "steps": steps, "warmup": warmup}


def quick_decode_f32(dev, steps=20, warmup=5):
    """The f32-cache shape (14 q heads, 2 kv heads, head_dim 64, 2048 rows, batch 1): 2 MB per launch,
    0.3 us at the HBM roofline -- a launch-latency measurement, reported in us per launch."""
    import torch

    from tinycoder_inference_b200 import ops

    nH, nKV, hd, ctx, layers = 14, 2, 64, 2048, 28
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE001)
    k = torch.randn((layers, ctx, nKV, hd), generator=g, device=dev)
    v = torch.randn((layers, ctx, nKV, hd), generator=g, device=dev)
    q = torch.randn((layers, 1, nH, hd), generator=g, device=dev)
    out = torch.empty_like(q)
    _, chunks = ops.split_geometry(ctx, nH, hd)
    ws = ops.workspace(1, nH, hd, chunks)

    def step():
        for l in range(layers):
            ops.decode_kv(q[l], k[l], v[l], out[l], ws, 1, nH, nKV, hd, ctx - 1, chunks)

    run = _graph_of(step)
    ms = _time_steps(run, steps, warmup, dev)
    nbytes = ctx * nKV * 2 * hd * 4
    gbs = layers * nbytes / (ms * 1e-3) / 1e9
    return {"workload": f"decode2k_f32: {nH} q heads / {nKV} kv heads / head_dim {hd}, f32 KV, context {ctx}, batch 1, "
                        f"{layers} launches per step (56 MB of pools: L2-resident, 2,097,152 algorithmic bytes per launch)",
            "us_per_layer": ms * 1e3 / layers, "value": gbs, "unit": "GB/s",
            "frac_of_peak_per_gpu": gbs / peaks()["hbm_gbs"], "bound": "launch latency (0.32 us at the HBM roofline)",
            "steps": steps, "warmup": warmup}


def _graph_of(step, no_graph=False):
    """Warm the step on a side stream, capture it, return the replay callable."""
    import torch

    step()
    torch.cuda.synchronize()
    if no_graph:
        return step
    s_ = torch.cuda.Stream()
    s_.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s_):
        step()
    torch.cuda.current_stream().wait_stream(s_)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        step()
    return gr.replay


def _time_steps(run, steps, warmup, dev):
    """CUDA-event time of `steps` runs behind `warmup` untimed ones, barrier + synchronise on both
    sides, maximum over the ranks; milliseconds per step."""
    import torch

    for _ in range(warmup):
        run()
    rank_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    rank_barrier()
    return max_over_ranks(e0.elapsed_time(e1), dev) / steps


def _check_rows(got, want):
    import numpy as np

    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    return float(err.max()), bool((err <= 1e-4 + 1e-3 * np.abs(want)).all())


def run_ragged(args, steps=None, warmup=None, layout=None, with_cpu=True):
    """Batched decode serving mix: 64 sequences with context lengths drawn uniformly from
    [512, 32768] by seed (28 q heads, 4 kv heads, head_dim 128, int8 KV), one decode step =
    28 layers.  layout = (sequence groups, kv-head groups), their product the rank count: the
    sequences are dealt to the sequence groups so that the TOKEN counts balance (longest first
    onto the lightest group), the ranks of a group take a block of kv heads each -- strong
    scaling, no collective.  Every rank keeps 4 layer pools of its share resident and cycles
    them 7 times per step.  Before anything is timed every rank checks layer 0 of some of its
    sequences against the CPU checker."""
    import numpy as np
    import torch

    import oracle
    from tinycoder_inference_b200 import ops, sharding

    world, rank, local, dev = dist_ctx()
    steps = steps or args.steps
    warmup = max(3, warmup or args.warmup)
    sp, hp = layout or (world, 1)
    assert sp * hp == world
    nH, nKV, hd, nseq, layers, resident = 28, 4, 128, 64, 28, 4
    sg, hg = rank // hp, rank % hp
    sh = sharding.plan_kv_head_shards(nH, nKV, hp)[hg]
    my_kv, my_q = sh.kv_hi - sh.kv_lo, sh.q_hi - sh.q_lo
    inv = 1.0 / math.sqrt(hd)
    rng = np.random.Generator(np.random.Philox(key=[0x7C0DE005, 0]))
    lens_all = (512 + rng.integers(0, 32257, nseq, dtype=np.uint64)).astype(np.int64)   # 512 + (u64 mod 32257)
    mine = sharding.plan_sequence_shards(lens_all.tolist(), sp)[sg]
    lens = lens_all[mine]
    B = len(mine)
    base = np.zeros(B, dtype=np.uint64)
    base[1:] = np.cumsum(lens[:-1] + 16)      # 16 rows of slack behind every sequence
    rows = int((lens + 16).sum())
    g = torch.Generator(device=dev)
    g.manual_seed(0x7C0DE005 + rank)
    k8 = torch.empty((resident, rows, my_kv, hd), dtype=torch.int8, device=dev)
    v8 = torch.empty_like(k8)
    ks = torch.zeros((resident, rows, my_kv), device=dev)
    vs = torch.zeros_like(ks)
    blk = 32768
    for l in range(resident):
        for r0 in range(0, rows, blk):
            n = min(blk, rows - r0)
            kf = torch.randn((n, my_kv, hd), generator=g, device=dev)
            vf = torch.randn((n, my_kv, hd), generator=g, device=dev)
            ops.kv_quantize_i8(kf, vf, k8[l], v8[l], ks[l], vs[l], n, my_kv, hd, dst_base=r0)
    q = torch.randn((resident, B, my_q, hd), generator=g, device=dev)
    out = torch.empty_like(q)
    dlens = torch.tensor(lens, dtype=torch.int32, device=dev)
    dbase = torch.tensor(base.astype(np.int64), dtype=torch.int64, device=dev)
    maxlen = int(lens.max())
    _, chunks = ops.split_geometry(maxlen, nH, hd)
    chunks = min(chunks, 64)
    ws = ops.workspace(B, my_q, hd, chunks)

    def step():
        for l in range(layers):
            r = l % resident
            ops.decode_i8_batch(q[r], k8[r], v8[r], ks[r], vs[r], out[r], ws, dlens, B, my_q, my_kv, hd, maxlen, chunks,
                                row_base=dbase, invSqrt=inv, pdl=True)

    run = _graph_of(step, args.no_graph)
    # parity of layer 0 (outside the timed region): the longest, the shortest and two more of this
    # rank's sequences against the CPU restatement of the reference's int8 attention
    run()
    torch.cuda.synchronize()
    pick = sorted({int(np.argmax(lens)), int(np.argmin(lens)), 0, B - 1})
    hq, hout = q[0].cpu().numpy(), out[0].cpu().numpy()
    worst, ok = 0.0, True
    for i in pick:
        r0, n = int(base[i]), int(lens[i])
        want = oracle.attention_i8(hq[i:i + 1], k8[0, r0:r0 + n].cpu().numpy(), v8[0, r0:r0 + n].cpu().numpy(),
                                   ks[0, r0:r0 + n].cpu().numpy(), vs[0, r0:r0 + n].cpu().numpy(), 1, my_q, my_kv, hd,
                                   n - 1, inv)
        e, o = _check_rows(hout[i:i + 1], want)
        worst, ok = max(worst, e), ok and o
    parity = parity_record(worst, ok, f"layer 0, {len(pick)} sequences per rank (longest, shortest, first, last)")
    ms_per_step = _time_steps(run, steps, warmup, dev)
    flags = ops.device_status()
    if rank != 0:
        return None
    tokens = int(lens_all.sum())
    total_bytes = layers * algorithmic_bytes(nKV, hd, tokens)
    val = total_bytes / (ms_per_step * 1e-3) / 1e9
    pk = peaks()
    line = {
        "metric": "decode_attn_kv_gbs_ragged64", "value": val, "unit": "GB/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "us_per_layer": ms_per_step * 1e3 / layers, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 KV, f32 q/out", "data": "synthetic",
        "config": {"workload": f"ragged64: {nseq} sequences, context lengths uniform in [512, 32768] by seed "
                               f"({tokens} tokens), 28 q heads / 4 kv heads / head_dim 128, int8 KV, "
                               f"{layers} layers per step ({resident} resident pools cycled)",
                   "sharding": f"{sp} sequence group(s) (whole sequences dealt by token count, longest first) x {hp} "
                               "kv-head group(s), no collective",
                   "rank0_sequences": B, "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": val / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": val / world / pk["hbm_gbs"], "peak_source": pk["source"], "traffic": None,
                     "note": "per-GPU share of the algorithmic bytes over the step time"},
        "parity": parity,
        "gpu_launches": steps * layers * 2, "device_error_flags": flags,
    }
    if with_cpu and world == 1:
        cb = cpu_allcores_sample(nH, nKV, hd, [int(x) for x in lens_all[:8]], budget_s=6.0)
        if cb:
            line["cpu_baseline"] = cb
    return line


def run_sharded(args, steps=None, warmup=None, layout=None, with_cpu=False):
    """Qwen2.5-32B-shaped long-context decode (40 q heads, 8 kv heads, head_dim 128, ctx
    131072, int8 KV), ONE sequence split over the ranks -- strong scaling.  layout = (kv-head
    groups, context ranges), their product the rank count:
      kv-head groups  : each rank holds nKV / groups heads of its rows; disjoint output slices;
      context ranges  : each rank holds its heads of ctx / ranges rows; the ranks of one head
                        group exchange their merged partial -- by the library's own kernel over
                        peer memory (p2p) or by an NCCL all-gather -- and merge.
    8 layers are resident per rank and cycled (a step = 8 layers).  Before anything is timed
    layer 0's output is checked against the CPU checker (the rows of all context ranges of a
    head group are gathered for that)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    from tinycoder_inference_b200 import ops, sharding

    world, rank, local, dev = dist_ctx()
    steps = steps or args.steps
    warmup = max(3, warmup or args.warmup)
    nH, nKV, hd, ctx, layers = 40, 8, 128, 131072, 8
    inv = 1.0 / math.sqrt(hd)
    if layout is None:
        layout = (1, world) if args.workload == "c4_ctxsplit" else (world, 1)
    hp, cp = layout
    assert hp * cp == world
    if nKV % hp != 0:
        raise SystemExit(f"{hp} kv-head groups do not divide {nKV} kv heads")
    hg, cg = rank % hp, rank // hp            # the head axis is the fastest (sharding.GridPlan.coords)
    sh = sharding.plan_kv_head_shards(nH, nKV, hp)[hg]
    lo, hi = sharding.plan_context_ranges(ctx, cp)[cg]
    my_rows, my_kv, my_q = hi - lo, sh.kv_hi - sh.kv_lo, sh.q_hi - sh.q_lo
    by_ctx = cp > 1
    group = None
    if by_ctx and world > 1:
        # every rank creates every group (new_group is collective); mine holds my head group's ranks
        for h in range(hp):
            gr_ = dist.new_group(ranks=[h + hp * c for c in range(cp)])
            if h == hg:
                group = gr_
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
    q = q_all[:, :, sh.q_lo:sh.q_hi].contiguous()
    out = torch.empty((layers, 1, my_q, hd), device=dev)
    chunk, chunks = ops.split_geometry(ctx, nH, hd)
    chunks = min(chunks, 128)
    ws = ops.workspace(1, my_q, hd, chunks)
    splitter = sharding.ContextSplitDecoder(my_q, my_kv, hd, my_rows, group=group, chunk_slots=64,
                                            exchange=args.exchange) if by_ctx else None

    def step_plain():
        for l in range(layers):
            if by_ctx:
                splitter(q[l], k8[l], v8[l], ks[l], vs[l], out[l], my_rows, invSqrt=inv, pdl=True)
            else:
                ops.decode_i8_batch(q[l], k8[l], v8[l], ks[l], vs[l], out[l], ws, None, 1, my_q, my_kv, hd, my_rows,
                                    chunks, invSqrt=inv, pdl=True, prefetch_rows=my_rows - 1)

    plain = args.no_graph or (by_ctx and args.exchange == "nccl")   # the NCCL form is timed as plain launches
    step = _graph_of(step_plain, plain)
    # ---- parity of layer 0 against the CPU checker, before anything is timed ----
    step()
    torch.cuda.synchronize()
    if by_ctx and world > 1:
        # the context ranges of my head group, in range order, onto every rank of the group
        parts = []
        for t in (k8[0, :my_rows], v8[0, :my_rows], ks[0, :my_rows], vs[0, :my_rows]):
            buf = [torch.empty_like(t) for _ in range(cp)]      # equal ranges: ctx is a multiple of 256 * cp
            dist.all_gather(buf, t.contiguous(), group=group)
            parts.append(torch.cat(buf).cpu().numpy())
    else:
        parts = [t[0, :my_rows].cpu().numpy() for t in (k8, v8, ks, vs)]
    worst, ok = 0.0, True
    if cg == 0:                                   # one rank per head group runs the checker
        want = oracle.attention_i8(q[0].cpu().numpy(), parts[0], parts[1], parts[2], parts[3], 1, my_q, my_kv, hd,
                                   ctx - 1, inv)
        worst, ok = _check_rows(out[0].cpu().numpy(), want)
    del parts
    parity = parity_record(worst, ok, "layer 0, every q head, all 131072 rows")
    ms_per_step = _time_steps(step, steps, warmup, dev)
    flags = ops.device_status()
    if rank != 0:
        return None
    total_bytes = layers * algorithmic_bytes(nKV, hd, ctx)       # the whole sequence, all ranks together
    pk = peaks()
    val = total_bytes / (ms_per_step * 1e-3) / 1e9
    name = args.workload if args.workload in ("c4_heads", "c4_ctxsplit") else "c4_32b_128k"
    line = {
        "metric": f"decode_attn_kv_gbs_{name}", "value": val, "unit": "GB/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "us_per_layer": ms_per_step * 1e3 / layers, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 KV, f32 q/out", "data": "synthetic",
        "config": {"workload": f"{name}: 40 q heads / 8 kv heads / head_dim 128, int8 KV, one sequence of "
                               f"{ctx} rows, {layers} layers per step",
                   "sharding": f"{hp} kv-head group(s) x {cp} context range(s)"
                               + ((": each rank's merged partial is stored into the peers of its head group over "
                                   "NVLink and merged there, one kernel per rank (no collective library call)"
                                   if args.exchange == "p2p" else ": partials all-gathered over NCCL and merged")
                                  if by_ctx else ": disjoint output slices, no data-path collective"),
                   "rows_per_rank": my_rows, "kv_heads_per_rank": my_kv,
                   "bytes_per_rank_per_layer": algorithmic_bytes(my_kv, hd, my_rows),
                   "launch": "plain launches" if plain else "cuda_graph",
                   "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": val / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": val / world / pk["hbm_gbs"], "peak_source": pk["source"], "traffic": None,
                     "note": "per-GPU share of the algorithmic bytes over the step time"},
        "parity": parity,
        "gpu_launches": steps * layers * 2, "device_error_flags": flags,
    }
    if with_cpu and world == 1:
        per_layer, cores, kind, sample = cpu_attention_sample(nH, nKV, hd, ctx, budget_s=6.0)
        line["cpu_baseline"] = {"value": algorithmic_bytes(nKV, hd, ctx) / per_layer / 1e9, "unit": "GB/s",
                                "cores": cores, "kind": kind, "sample": sample, "us_per_layer": per_layer * 1e6}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode32k",
                    choices=sorted(WORKLOADS) + ["prefill4k", "prefill4k_chunked512", "c4_heads", "c4_ctxsplit", "ragged64"])
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="c4_ctxsplit: partials exchanged by the library's own kernel over peer memory, or by NCCL")
    ap.add_argument("--no-next-prefetch", action="store_true",
                    help="do not hint the next layer's pools to the decode call (L2 prefetch while a layer drains)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary measurements (`also`) and the sustained replay of the default line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream order between the kernels of a step")
    ap.add_argument("--e2e-plain-copies", action="store_true",
                    help="diagnostic: the end-to-end step's host copies issued around its graph, not as nodes of it")
    ap.add_argument("--partials-only", action="store_true", help="diagnostic: skip the merge launch")
    ap.add_argument("--fused-merge", action="store_true",
                    help="merge the chunk partials inside the decode kernel (last-arriving block) instead of a second launch")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    single = {"prefill4k": lambda: run_prefill(args),
              "prefill4k_chunked512": lambda: run_prefill(args, chunk=512),
              "c4_heads": lambda: run_sharded(args, with_cpu=True), "c4_ctxsplit": lambda: run_sharded(args, with_cpu=True),
              "ragged64": lambda: run_ragged(args)}
    if args.workload in single:
        line = single[args.workload]()
        if line is not None:
            print(json.dumps(line), flush=True)
        dist_done()
        return

    import torch
    import torch.distributed as dist

    from tinycoder_inference_b200 import ops

    world, rank, local, dev = dist_ctx()

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
    # the same graph replayed for about two seconds with the clocks sampled: the short timed region
    # above runs at boost clocks, a latency-bound step depends on them
    sustained = None
    if not args.no_extras:
        s2 = ClockSampler(gpu_id)
        if rank == 0:
            s2.start()
        n_sus = max(args.steps, int(2000.0 / max(ms_per_step, 1e-3)))
        barrier()
        e0.record()
        for _ in range(n_sus):
            run()
        e1.record()
        barrier()
        ms_sus = max_over_ranks(e0.elapsed_time(e1), dev) / n_sus
        ck = s2.stop() if rank == 0 else None
        if rank == 0:
            us = ms_sus * 1e3 / layers
            sustained = {"steps": n_sus, "seconds": ms_sus * n_sus / 1e3, "us_per_layer": us, "sm_mhz": ck["sm_mhz"],
                         "us_x_mhz": us * ck["sm_mhz"] if ck["sm_mhz"] else None, "reasons": ck["reasons"],
                         "samples": ck["samples"]}
    bytes_per_step_gpu = layers * batch * algorithmic_bytes(nKV, hd, ctx)
    value = world * bytes_per_step_gpu / (ms_per_step * 1e-3) / 1e9
    us_per_layer = ms_per_step * 1e3 / layers

    # ---- end to end through the C ABI with HOST buffers ---------------------------
    # A step: the new token's q, k, v of every layer come from one pinned host buffer (one
    # asynchronous copy), then per layer attention runs with k/v quantised into the last row by
    # the decode launch itself, and the step's outputs go back to pinned host memory; the host
    # waits for them.  The two copies are nodes of the step's captured graph, so a step is one
    # graph launch and one wait (--e2e-plain-copies: three input copies and the output copy
    # issued around the graph instead).
    nq, nk = layers * batch * nH * hd, layers * batch * nKV * hd
    hin = torch.randn(nq + 2 * nk).pin_memory()
    din = torch.empty(nq + 2 * nk, device=dev)
    hq, hk, hv = hin[:nq], hin[nq:nq + nk], hin[nq + nk:]
    dq = din[:nq].view(layers, batch, nH, hd)
    dk = din[nq:nq + nk].view(layers, batch, nKV, hd)
    dv = din[nq + nk:].view(layers, batch, nKV, hd)
    hout = torch.empty((layers, batch, nH, hd)).pin_memory()
    dout = torch.empty((layers, batch, nH, hd), device=dev)
    copies_inside = not args.e2e_plain_copies

    def e2e_layers():
        if copies_inside:
            din.copy_(hin, non_blocking=True)
        for l in range(layers):
            nxt = None if args.no_next_prefetch else (k8[(l + 1) % layers], v8[(l + 1) % layers])
            ops.decode_i8_batch(dq[l], k8[l], v8[l], ks[l], vs[l], dout[l], ws, lens_arg, batch, nH, nKV, hd, ctx,
                                chunks, rows_per_seq=rows, invSqrt=inv, pdl=not args.no_pdl, prefetch_rows=ctx - 1,
                                next_kv=nxt, tickets=tickets, append=(dk[l], dv[l]))
        if copies_inside:
            hout.copy_(dout, non_blocking=True)

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
        if not copies_inside:
            din[:nq].copy_(hq, non_blocking=True)
            din[nq:nq + nk].copy_(hk, non_blocking=True)
            din[nq + nk:].copy_(hv, non_blocking=True)
        e2e_run()
        if not copies_inside:
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

    pk = peaks()
    per_gpu_gbs = bytes_per_step_gpu / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": "decode_attn_kv_gbs_ctx32k" if args.workload == "decode32k" else f"decode_attn_kv_gbs_{args.workload}",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "us_per_layer": us_per_layer,
        "us_per_layer_plain_stream_order": ms_plain_per_step * 1e3 / layers,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int8 KV, f32 q/out (exact int8 tensor-core products on integer digit planes of q and p, f32 softmax and accumulation)",
        "data": "synthetic", "config": workload_config(args.workload, world),
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": per_gpu_gbs / pk["hbm_gbs"], "peak_source": pk["source"],
                     "traffic": None,   # not measured by this run (an ncu capture of one launch is summarised separately)
                     "algorithmic_bytes_per_launch": batch * algorithmic_bytes(nKV, hd, ctx),
                     "note": "algorithmic bytes per layer / (step time / layers); split and merge launches both inside"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms_per_step,
                "h2d_bytes_per_step": layers * batch * (nH + 2 * nKV) * hd * 4,
                "d2h_bytes_per_step": layers * batch * nH * hd * 4,
                "copies": ("one H2D and one D2H copy from/to pinned memory as nodes of the step's graph"
                           if copies_inside and not args.no_graph else
                           "H2D copies before and one D2H copy after the step's launches, from/to pinned memory")},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "device_error_flags": dev_flags,
    }
    if sustained is not None:
        line["sustained"] = sustained
    if args.workload == "decode32k" and not args.no_extras:
        del k8, v8, ks, vs
        torch.cuda.empty_cache()
        line["also"] = also_measurements(args, world, rank, dev)
    if rank != 0:
        dist_done()
        return
    if not args.no_cpu_baseline and world == 1:
        per_layer, cores, kind, sample = cpu_attention_sample(nH, nKV, hd, ctx)
        line["cpu_baseline"] = {"value": algorithmic_bytes(nKV, hd, ctx) / per_layer / 1e9, "unit": "GB/s",
                                "cores": cores, "kind": kind, "sample": sample, "us_per_layer": per_layer * 1e6}
    print(json.dumps(line), flush=True)
    dist_done()


def _brief(line, extra=()):
    """The figures of a secondary measurement, without the boilerplate of a full line."""
    keep = ("metric", "value", "unit", "us_per_layer", "ms_per_step", "scaling", "steps", "warmup", "parity", "e2e",
            "cpu_baseline", "device_error_flags") + tuple(extra)
    d = {k: line[k] for k in keep if k in line}
    d["workload"] = line["config"]["workload"]
    if "sharding" in line["config"]:
        d["sharding"] = line["config"]["sharding"]
    for k in ("rows_per_rank", "kv_heads_per_rank", "bytes_per_rank_per_layer"):
        if k in line["config"]:
            d[k] = line["config"][k]
    r = line["roofline"]
    d["frac_of_peak_per_gpu"] = r["frac"]
    d["bound"] = r["bound"]
    if r["bound"] == "tensor":
        d["attention_launch_tflops"] = r["achieved"]
    return d


def also_measurements(args, world, rank, dev):
    """The other configurations next to the headline.  One GPU: the batch-8 twin of the headline, the
    8192-row shapes, the f32 shape, the 32B shape at 131072 rows, the 64-sequence mix, the prefill.
    Several GPUs: the strong-scaling partitions of the 32B sequence and of the 64-sequence mix over
    the ranks of this run."""
    out = []
    k, w = 10, 3

    def add(line, **kw):
        if rank == 0 and line is not None:
            d = _brief(line)
            d.update(kw)
            out.append(d)

    if world == 1:
        for name in ("decode32k_b8", "decode8k_b1", "decode8k_b8", "c4_32b_128k"):
            out.append(quick_decode(name, dev))
        out.append(quick_decode_f32(dev))
        if not args.no_cpu_baseline:
            cb = cpu_allcores_sample(28, 4, 128, [8192] * 8, budget_s=6.0)
            if cb:
                out[2]["cpu_baseline_all_cores"] = cb
        add(run_ragged(args, steps=k, warmup=w, with_cpu=not args.no_cpu_baseline))
        add(run_prefill(args, steps=k, warmup=w, with_cpu=not args.no_cpu_baseline))
        add(run_prefill(args, steps=5, warmup=w, chunk=512, with_cpu=False, with_e2e=False))
        return out
    lat = ("a rank's share of a layer is below about 70 MB: the launch is bounded by the latency chain of the "
           "split-KV kernel and its merge (about 12 us whatever the bytes), not by bandwidth")
    bw = "a rank still streams more than 70 MB per layer: bandwidth-bound"
    layouts = [(h, world // h) for h in (8, 4, 2, 1) if world % h == 0 and h <= world]
    for hp, cp in layouts:
        if cp > 1 and args.exchange != "p2p":
            continue
        line = run_sharded(args, steps=k, warmup=w, layout=(hp, cp))
        if line is not None:
            share = line["config"]["bytes_per_rank_per_layer"]
            add(line, limiter=(lat if share < 70e6 else bw) + ("; plus the exchange of the merged partials over "
                                                                 "NVLink (about 5 us per layer)" if cp > 1 else ""))
    for sp, hp in [(world // h, h) for h in (1, 2, 4) if world % h == 0 and h <= world]:
        line = run_ragged(args, steps=k, warmup=w, layout=(sp, hp), with_cpu=False)
        if line is not None:
            add(line, limiter="token balance between the sequence groups and the tail of the longest sequence; "
                              "with kv-head groups every rank runs all sequences of its group at 1/groups of the bytes")
    return out


if __name__ == "__main__":
    main()
