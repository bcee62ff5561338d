#!/usr/bin/env python
"""Benchmark of the quantized matrix-product path on B200.

Default workload (N=1): the int4 decode step of a Gemma3-1B-shaped decoder -
every MatMulNBits projection of 26 layers (q, k, v, o, gate, up, down) and the
lm_head, M=1, fp16 activations/scales/outputs, block 32 with zero points,
random weights - reported as algorithmic HBM GB/s (bytes = packed weights +
scales + zero points + activations + outputs, each counted once per GEMV).
A "step" is one token: 183 GEMVs over 580 MB of distinct weights (larger than
the 126 MB L2, so no flush is needed between steps).

  python bench.py --gpus N --steps K --warmup W [--impl reference]

One JSON line on stdout (rank 0).  `roofline` is for the dominant kernel, the
lm_head GEMV, timed with CUDA events inside the timed region.  `e2e` runs the
same step through the C ABI with host buffers: pinned-host activations are
uploaded and the logits downloaded every step.  `--impl reference` times the
CPU port of the reference's shader arithmetic (oracle/) on the host cores.
With N > 1 the decode step does not shard (single-GPU by design): each rank
runs one replica ("weak" scaling, no collective in the data path).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.join(ROOT, "onnx-vulkan-rs_b200"),):
    if p not in sys.path:
        sys.path.insert(0, p)

HIDDEN, Q_OUT, KV_OUT, FF, VOCAB, LAYERS, BLOCK = 1152, 1024, 256, 6912, 262144, 26, 32
LAYER_SHAPES = [("q", HIDDEN, Q_OUT), ("k", HIDDEN, KV_OUT), ("v", HIDDEN, KV_OUT), ("o", Q_OUT, HIDDEN),
                ("gate", HIDDEN, FF), ("up", HIDDEN, FF), ("down", FF, HIDDEN)]
LM_HEAD = ("lm_head", HIDDEN, VOCAB)


def nbits_bytes(m, k, n, bs, real_bytes=2, with_zp=True):
    """Algorithmic traffic of one MatMulNBits: every operand once."""
    nb = -(-k // bs)
    return n * nb * bs // 2 + n * nb * real_bytes + (n * ((nb + 1) // 2) if with_zp else 0) + \
        m * k * real_bytes + m * n * real_bytes


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------- GPU arm

def make_weight(torch, ctx, k, n, bs, gen):
    nb = -(-k // bs)
    b = torch.randint(0, 256, (n, nb, bs // 2), dtype=torch.uint8, device="cuda", generator=gen)
    scales = (torch.rand((n * nb,), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.float16)
    zp = torch.randint(0, 256, (n, (nb + 1) // 2), dtype=torch.uint8, device="cuda", generator=gen)
    return ctx.nbits_prepack(b, scales, zp, n, k, bs)


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import ovk_b200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = ovk_b200.Context(local)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xB200 + 0x100 * 2)

    # one distinct weight per projection per layer + the lm_head
    ops = []
    for layer in range(args.layers):
        for name, k, n in LAYER_SHAPES:
            ops.append((f"L{layer}.{name}", k, n, make_weight(torch, ctx, k, n, BLOCK, gen)))
    ops.append((LM_HEAD[0], LM_HEAD[1], LM_HEAD[2], make_weight(torch, ctx, LM_HEAD[1], LM_HEAD[2], BLOCK, gen)))
    acts = {k: torch.randn((1, k), device="cuda", generator=gen).to(torch.float16) for k in {HIDDEN, Q_OUT, FF}}
    outs = {n: torch.empty((1, n), dtype=torch.float16, device="cuda") for n in {Q_OUT, KV_OUT, HIDDEN, FF, VOCAB}}
    step_bytes = sum(nbits_bytes(1, k, n, BLOCK) for _, k, n, _ in ops)
    lm_bytes = nbits_bytes(1, LM_HEAD[1], LM_HEAD[2], BLOCK)
    ctx.flush()

    lm_events = []

    def step(timed: bool):
        for name, k, n, w in ops:
            if timed and name == "lm_head":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ctx.matmul_nbits(w, acts[k], out=outs[n])
                e1.record()
                lm_events.append((e0, e1))
            else:
                ctx.matmul_nbits(w, acts[k], out=outs[n])

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(False)
    sync_all()
    launches0 = ctx.launches
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    launches = ctx.launches - launches0
    ms = torch.tensor([t0.elapsed_time(t1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    lm_ms = statistics.mean(e0.elapsed_time(e1) for e0, e1 in lm_events)
    lm_kernel = ctx.last_kernel

    # ------------------------------------------------------------ end to end
    # the call a user makes: host activations in, logits out, every step
    pinned_in = {k: acts[k].cpu().pin_memory() for k in acts}
    pinned_out = torch.empty((1, VOCAB), dtype=torch.float16).pin_memory()
    h2d = sum(k * 2 for _, k, _, _ in ops)
    d2h = VOCAB * 2

    def e2e_step():
        for name, k, n, w in ops:
            acts[k].copy_(pinned_in[k], non_blocking=True)
            ctx.matmul_nbits(w, acts[k], out=outs[n])
        pinned_out.copy_(outs[VOCAB], non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    sync_all()
    e2e_steps = max(1, min(args.steps, 10))
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    sync_all()
    e2e_s = torch.tensor([time.perf_counter() - w0], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_gbs = world * step_bytes * e2e_steps / float(e2e_s.item()) / 1e9

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        achieved = lm_bytes / (lm_ms * 1e-3) / 1e9
        traffic = None
        prof = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(prof):
            traffic = json.load(open(prof)).get(lm_kernel)
        line = {
            "metric": "int4_decode_gemv_hbm_gbs", "value": world * step_bytes * args.steps / (ms_total * 1e-3) / 1e9,
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "gemma3-1b-int4-decode: %d layers x (q,k,v,o,gate,up,down) + lm_head, M=1, "
                                   "bits=4 block_size=32 zero points, fp16" % args.layers,
                       "gemvs_per_step": len(ops), "bytes_per_step": step_bytes,
                       "l2": "distinct weights per GEMV, %.0f MB per step > 126 MB L2 (no flush needed)" % (step_bytes / 1e6),
                       "parallelism": "replicas" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "kernel": lm_kernel + " (lm_head K=1152 N=262144)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "of": peak_kind, "bytes_per_launch": lm_bytes, "ms_per_launch": lm_ms,
                         "frac_of_nominal_8tbs": achieved / 8000.0, "traffic": traffic},
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------- CPU arm

def cpu_sample(n_cols):
    """The lm_head GEMV restricted to its first n_cols columns, f32 (the only
    form the reference's kernel takes), seeded."""
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(0xB200 + 0x100 * 2))
    nb = HIDDEN // BLOCK
    b = rng.integers(0, 256, size=(n_cols, nb, BLOCK // 2), dtype=np.uint8)
    scales = rng.uniform(0.002, 0.02, size=n_cols * nb).astype(np.float32)
    zp = rng.integers(0, 256, size=(n_cols, (nb + 1) // 2), dtype=np.uint8)
    a = rng.standard_normal((1, HIDDEN), dtype=np.float32)
    return a, b, scales, zp


def cpu_time_once(orc, sample, n_cols):
    a, b, scales, zp = sample
    t = time.perf_counter()
    orc.matmul_nbits_f32_shader_order(a, b, scales, zp, HIDDEN, n_cols, BLOCK)
    return time.perf_counter() - t


def cpu_baseline(budget_s=12.0):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    cores = len(os.sched_getaffinity(0))
    orc.set_num_threads(cores)
    n_cols = VOCAB // 4
    sample = cpu_sample(n_cols)
    cpu_time_once(orc, sample, n_cols)  # warm-up
    times, spent = [], 0.0
    while spent < budget_s and len(times) < 50:
        dt = cpu_time_once(orc, sample, n_cols)
        times.append(dt)
        spent += dt
    byts = nbits_bytes(1, HIDDEN, n_cols, BLOCK, real_bytes=4)
    return {"value": byts / statistics.median(times) / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "lm_head GEMV, first %d of %d columns, f32 (reference shader order, oracle/ovk_oracle.c), "
                      "median of %d runs" % (n_cols, VOCAB, len(times))}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    cores = len(os.sched_getaffinity(0))
    orc.set_num_threads(cores)
    n_cols = VOCAB // 4
    sample = cpu_sample(n_cols)
    for _ in range(max(1, args.warmup)):
        cpu_time_once(orc, sample, n_cols)
    t = time.perf_counter()
    for _ in range(args.steps):
        cpu_time_once(orc, sample, n_cols)
    total = time.perf_counter() - t
    byts = nbits_bytes(1, HIDDEN, n_cols, BLOCK, real_bytes=4)
    value = byts * args.steps / total / 1e9
    desc = ("each step = lm_head GEMV restricted to its first %d of %d columns, f32, reference shader order "
            "(CPU port in oracle/ovk_oracle.c; the reference's own GPU path needs Vulkan: unavailable on this box)"
            % (n_cols, VOCAB))
    print(json.dumps({
        "impl": "reference", "metric": "int4_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemma3-1b-int4-decode (bounded sample)", "sample": desc},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
