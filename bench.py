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


def ovk_int8_code():
    import ovk_b200
    return ovk_b200.INT8


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
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def lines(self) -> int:
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def wait_first_sample(self, keep_busy, limit_s: float = 4.0) -> int:
        """Runs `keep_busy` until nvidia-smi has written its first line; returns the line count."""
        t0 = time.perf_counter()
        while self.proc is not None and self.lines() == 0 and time.perf_counter() - t0 < limit_s:
            keep_busy()
        return self.lines()

    def stop(self, skip: int = 0):
        """Summary of the samples after the first `skip` lines."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in list(open(self.path))[skip:]:
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

def weight_tensors(torch, k, n, bs, gen, scale_lo=0.002, scale_hi=0.02):
    """Random int4 weight in the operator layout (packed nibbles, fp16 scales, packed zero points)."""
    nb = -(-k // bs)
    b = torch.randint(0, 256, (n, nb, bs // 2), dtype=torch.uint8, device="cuda", generator=gen)
    scales = (torch.rand((n * nb,), device="cuda", generator=gen) * (scale_hi - scale_lo) + scale_lo).to(torch.float16)
    zp = torch.randint(0, 256, (n, (nb + 1) // 2), dtype=torch.uint8, device="cuda", generator=gen)
    return b, scales, zp


def make_weight(torch, ctx, k, n, bs, gen, scale_lo=0.002, scale_hi=0.02):
    b, scales, zp = weight_tensors(torch, k, n, bs, gen, scale_lo, scale_hi)
    return ctx.nbits_prepack(b, scales, zp, n, k, bs)


def check_against_port(torch, y, a, b, scales, zp, k, bs, rows, cols):
    """Sampled rows x columns of Y against the CPU port of the operator (outside any timed region)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    nb = -(-k // bs)
    ci, ri = torch.from_numpy(cols).cuda(), torch.from_numpy(rows).cuda()
    want = orc.matmul_nbits(a[ri].cpu().numpy(), b[ci].cpu().numpy(), scales.reshape(-1, nb)[ci].cpu().numpy(),
                            zp[ci].cpu().numpy(), k, cols.size, bs).astype(np.float64)
    got = y[ri][:, ci].cpu().numpy().astype(np.float64)
    return bool(np.all(np.abs(got - want) <= 1e-3 + 1e-3 * np.abs(want)))


def timed(torch, dist, world, fn, iters, warm=3):
    """ms per call of fn, CUDA events on the current stream, max over ranks."""
    for _ in range(warm):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def extra_workloads(torch, dist, ctx, world, rank, gen, peaks):
    """The other operators of the path, one line each.  With more than one GPU
    the prefill is split by weight columns (all-gather of the outputs) and the
    convolution by batch (no exchange)."""
    import numpy as np
    from ovk_b200 import shard
    out = {}
    bf16_peak = peaks["bf16_tflops"]

    # ---- int4 prefill, Qwen2.5-7B-shaped (config 5), M = 4096, block 128
    # One GPU: the plain operator.  More: every rank prepares the SAME seeded weight, keeps its column
    # shard, and the shards are run three ways - the product alone, the product whose store warp writes
    # every tile into every rank's Y (the exchange inside the kernel, peer stores over NVLink), and the
    # product followed by an NCCL all-gather - next to the whole product on rank 0's GPU alone.
    m = 4096
    pg = shard.PeerGroup(ctx, rank, world) if world > 1 else None
    # a second context of this rank for the multicast variant (its own flag blocks and call numbers)
    sg, ctx_mc, mc_error = None, None, None
    if world > 1:
        try:
            import ovk_b200
            ctx_mc = ovk_b200.Context(torch.cuda.current_device())
            sg = shard.SymmetricGroup(ctx_mc, rank, world)
        except Exception as e:
            sg, mc_error = None, "symmetric memory: " + str(e)[:160]
    partitioned = {}
    for name, k, n in (("gate_up", 3584, 18944), ("down", 18944, 3584), ("lm_head", 3584, 152064)):
        if name == "lm_head" and world not in (1, 8):
            continue  # a 1.25 GB output: timed on one GPU and at the full split only
        b, scales, zp = weight_tensors(torch, k, n, 128, gen, 0.001, 0.01)
        a = torch.randn((m, k), device="cuda", generator=gen).to(torch.float16)
        sh = shard.column_shard(n, world, rank)
        bs_, ss_, zs_ = shard.slice_nbits_weight(b, scales, zp, k // 128, sh)
        w = ctx.nbits_prepack(bs_.contiguous(), ss_.contiguous(), zs_.contiguous(), sh.count, k, 128)
        y = torch.empty((m, sh.count), dtype=torch.float16, device="cuda")
        ms_c = timed(torch, dist, world, lambda: ctx.matmul_nbits(w, a, out=y), 5)
        entry = {"M": m, "K": k, "N": n, "block_size": 128, "kernel": ctx.last_kernel, "ms_compute": ms_c,
                 "tflops_compute": 2.0 * m * k * n / (ms_c * 1e-3) / 1e12}
        entry["frac_of_measured_bf16_peak_per_gpu"] = entry["tflops_compute"] / world / bf16_peak
        if world > 1:
            y_ptrs = pg.symmetric(m * n * 2)
            y_full = shard.DeviceBlock(y_ptrs[rank], (m, n), "<f2").tensor("cuda")
            ms_f = timed(torch, dist, world, lambda: ctx.matmul_nbits_nsplit(w, a, sh.start, n, y_ptrs), 5)
            ctx.flush()  # a peer wait that ran out would raise here
            rows = np.arange(7, m, 257)
            cols = np.unique(np.r_[np.arange(5, n, max(1, n // 96)),
                                   [shard.column_shard(n, world, r).start for r in range(world)],
                                   [shard.column_shard(n, world, r).stop - 1 for r in range(world)]])
            ok = check_against_port(torch, y_full, a, b, scales, zp, k, 128, rows, cols) if rank == 0 else True

            # the exchange alone (the column block already in place): what the links take without any product
            ms_x = timed(torch, dist, world, lambda: ctx.allgather_cols(None, m, sh.count, sh.start, n, y_ptrs), 5)
            # the same two through a multicast mapping of the ranks' matrices, where the box offers one: a tile
            # leaves this GPU's links once and the NVSwitch delivers it to every rank
            ms_fm = ms_xm = None
            ok_m = None
            if sg is not None:
                try:
                    ym_ptrs, ym_mc = sg.symmetric(m * n * 2)
                except Exception as e:  # no symmetric memory on this box: say so, keep the peer-store figures
                    ym_mc, mc_error = 0, str(e)[:120]
                if not ym_mc:
                    mc_error = mc_error or "no multicast mapping on this box"
                if ym_mc:
                    ym_full = shard.DeviceBlock(ym_ptrs[rank], (m, n), "<f2").tensor("cuda")
                    ms_fm = timed(torch, dist, world,
                                  lambda: ctx_mc.matmul_nbits_nsplit(w, a, sh.start, n, ym_ptrs, multicast=ym_mc), 5)
                    ctx_mc.flush()
                    ok_m = check_against_port(torch, ym_full, a, b, scales, zp, k, 128, rows, cols) if rank == 0 else True
                    ms_xm = timed(torch, dist, world,
                                  lambda: ctx_mc.allgather_cols(None, m, sh.count, sh.start, n, ym_ptrs, multicast=ym_mc), 5)
                    del ym_full

            def nccl_step():
                ctx.matmul_nbits(w, a, out=y)
                shard.all_gather_columns(y, n, world)
            ms_n = timed(torch, dist, world, nccl_step, 3) if name != "lm_head" else None
            # the whole product on one GPU, in the same run (rank 0 works, the others wait at the barrier)
            ms_1 = torch.zeros(1, device="cuda")
            if rank == 0:
                w1 = ctx.nbits_prepack(b, scales, zp, n, k, 128)
                y1 = torch.empty((m, n), dtype=torch.float16, device="cuda")
                ms_1[0] = timed(torch, dist, 1, lambda: ctx.matmul_nbits(w1, a, out=y1), 5)
                del w1, y1
            dist.broadcast(ms_1, 0)
            ms_1 = float(ms_1.item())
            recv = (world - 1) / world * m * n * 2
            entry.update({"ms_with_exchange_in_kernel": ms_f, "tflops_with_exchange": 2.0 * m * k * n / (ms_f * 1e-3) / 1e12,
                          "ms_with_nccl_all_gather": ms_n, "ms_exchange_alone": ms_x, "ms_one_gpu_same_run": ms_1,
                          "parallelism": ("N-split x%d; the kernel's store warp writes each tile into every rank's Y "
                                          "(peer stores over NVLink), one flag per peer ends the step" % world) if world <= 4 else
                                         ("N-split x%d; beyond four ranks the library runs the product into the rank's own Y and "
                                          "then its all-gather kernel (peer stores over NVLink) - 'ms_with_exchange_in_kernel' "
                                          "is that whole call" % world)})
            partitioned[name] = {"ms_one_gpu": ms_1, "ms_compute": ms_c, "ms_e2e": ms_f, "ms_e2e_nccl": ms_n,
                                 "ms_exchange_alone": ms_x, "exchange_alone_gbs_per_gpu": recv / (ms_x * 1e-3) / 1e9,
                                 "ms_e2e_multicast": ms_fm, "ms_exchange_alone_multicast": ms_xm,
                                 "speedup_e2e_multicast": (ms_1 / ms_fm) if ms_fm else None,
                                 "parity_checked_multicast": ok_m, "multicast_unavailable": mc_error,
                                 "speedup_compute": ms_1 / ms_c, "speedup_e2e": ms_1 / ms_f,
                                 "speedup_e2e_nccl": (ms_1 / ms_n) if ms_n else None,
                                 "received_bytes_per_gpu": recv, "received_gbs_per_gpu": recv / (ms_f * 1e-3) / 1e9,
                                 "parity_checked": ok, "parity_sample": "%d rows x %d columns of the gathered Y on rank 0 "
                                 "against the CPU port, atol = rtol = 1e-3" % (rows.size, cols.size)}
            del y_full
        out["int4_prefill_qwen7b_" + name] = entry
        del w, a, y, b, scales, zp, bs_, ss_, zs_
        torch.cuda.empty_cache()
    if sg is not None:
        sg.close()
    if pg is not None:
        torch.cuda.synchronize()
        pg.close()
        out["partitioned"] = partitioned
    # ---- int4 prefill, Gemma3-1B-shaped lm_head (config 2), M = 512, block 32: rank-local
    if world == 1:
        w = make_weight(torch, ctx, HIDDEN, VOCAB, BLOCK, gen)
        a = torch.randn((512, HIDDEN), device="cuda", generator=gen).to(torch.float16)
        y = torch.empty((512, VOCAB), dtype=torch.float16, device="cuda")
        ms_c = timed(torch, dist, 1, lambda: ctx.matmul_nbits(w, a, out=y), 5)
        out["int4_prefill_gemma3_lm_head"] = {"M": 512, "K": HIDDEN, "N": VOCAB, "block_size": 32,
                                              "kernel": ctx.last_kernel, "ms_compute": ms_c,
                                              "tflops_compute": 2.0 * 512 * HIDDEN * VOCAB / (ms_c * 1e-3) / 1e12}
        del w, a, y
        # ---- the launches either side of the lm_head GEMV in a decode step: greedy ArgMax over the
        # logits and the int4 embedding row of the token it picked (read on the device, no round trip)
        nb = HIDDEN // BLOCK
        table = torch.randint(0, 256, (VOCAB, HIDDEN // 2), dtype=torch.uint8, device="cuda", generator=gen)
        sc = (torch.rand((VOCAB, nb), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.float16)
        zp = torch.randint(0, 256, (VOCAB, (nb + 1) // 2), dtype=torch.uint8, device="cuda", generator=gen)
        logits = torch.randn((1, VOCAB), device="cuda", generator=gen).to(torch.float16)
        tok = torch.empty((1,), dtype=torch.int64, device="cuda")
        row = torch.empty((1, HIDDEN), dtype=torch.float16, device="cuda")

        def neighbours():
            ctx.argmax(logits, out=tok)
            ctx.gather_block_quantized(table, tok, sc, zp, BLOCK, out=row)
        g = torch.cuda.CUDAGraph()
        neighbours()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
            for _ in range(20):
                neighbours()
        ms_n = timed(torch, dist, 1, g.replay, 10) / 20
        out["decode_step_neighbours"] = {"ops": "ArgMax over 262144 fp16 logits + GatherBlockQuantized of one 1152-wide int4 row",
                                         "kernels": ["argmax", ctx.last_kernel], "us_per_pair": ms_n * 1e3,
                                         "bytes": VOCAB * 2 + HIDDEN // 2 + nb * 2 + HIDDEN * 2}
        del g, table, sc, zp, logits

    # ---- dynamic int8 encoder GEMMs, Parakeet-shaped (config 3): replicas
    # One FastConformer layer's six GEMMs in the order the graph runs them, each tensor quantised ONCE:
    #   x -> DynamicQuantizeLinear -> q, k, v (three GEMMs over the same bytes)
    #   attention output -> DynamicQuantizeLinear -> o
    #   FF input -> DynamicQuantizeLinear -> FF1 (1024 -> 4096, f32 out)
    #   FF1 output -> DecomposedGeluQuantize (the f32 GELU is never stored) -> FF2 (4096 -> 1024)
    t = 1000
    layer, layer_step = parakeet_layer(torch, ctx, gen, t)
    before = ctx.launches
    layer_step()
    layer_launches = ctx.launches - before
    layer_kernel = ctx.last_kernel
    torch.cuda.synchronize()
    # a dozen launches of 3-15 us each: replayed from a graph so that the device, not Python, is timed
    # (ten layers per replay, as the layers of an encoder follow each other: one replay of a single layer is
    # half launch latency of the graph itself)
    layers_per_replay = 10
    gl = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gl, stream=torch.cuda.current_stream()):
        for _ in range(layers_per_replay):
            layer_step()
    ms_l = timed(torch, dist, world, gl.replay, 10) / layers_per_replay
    del gl
    ops = sum(2.0 * t * k * n for k, n in layer)
    out["int8_dynamic_parakeet_layer"] = {"T": t, "gemms": len(layer), "launches": layer_launches, "ms_per_layer": ms_l,
                                          "kernel": layer_kernel, "tops": world * ops / (ms_l * 1e-3) / 1e12,
                                          "note": "3 x DynamicQuantizeLinear + DecomposedGeluQuantize + 6 x MatMulInteger with "
                                                  "the fused f32 epilogue (q, k, v share one quantisation and one launch); "
                                                  "2-8 GOP per GEMM, latency/HBM-bound; replicas at N > 1"}
    # the convolution module of the same encoder layer: pointwise 1024 -> 2048, depthwise k=9, pointwise 1024 -> 1024
    # (ConvIntegerScaleBias over [1, C, 1, T]); pointwise layers run as filters x image on the MatMulInteger kernels
    conv_mod = {}
    for name, c_in, c_out, kw, group in (("pointwise_1024_2048", 1024, 2048, 1, 1), ("depthwise_k9", 1024, 1024, 9, 1024),
                                         ("pointwise_1024_1024", 1024, 1024, 1, 1)):
        wc = ctx.qconv_prepack(torch.randint(-127, 128, (c_out, c_in // group, 1, kw), dtype=torch.int8, device="cuda",
                                             generator=gen), group=group)
        xc = torch.randint(0, 256, (1, c_in, 1, t), dtype=torch.uint8, device="cuda", generator=gen)
        sc_c = torch.rand((c_out,), device="cuda", generator=gen) * 0.009 + 0.001
        bi_c = torch.zeros((c_out,), device="cuda")
        pads_c = (0, kw // 2, 0, kw // 2)
        fn_c = lambda: ctx.conv_integer_scale_bias(wc, xc, 128, 0, sc_c, bi_c, pads=pads_c)
        fn_c()
        kern_c = ctx.last_kernel
        torch.cuda.synchronize()
        gc_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gc_, stream=torch.cuda.current_stream()):
            for _ in range(10):
                fn_c()
        conv_mod[name] = {"us": timed(torch, dist, world, gc_.replay, 10) / 10 * 1e3, "kernel": kern_c}
        del gc_, wc, xc
    out["int8_parakeet_conv_module"] = {"T": t, **conv_mod}
    big = ctx.mmi_prepack(torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device="cuda", generator=gen))
    xa = torch.randint(0, 256, (8192, 8192), dtype=torch.uint8, device="cuda", generator=gen)
    zp8 = torch.full((1,), 128, dtype=torch.uint8, device="cuda")
    ms_b = timed(torch, dist, world, lambda: ctx.matmul_integer(big, xa, zp8, None), 5)
    tops_b = 2.0 * 8192 ** 3 / (ms_b * 1e-3) / 1e12
    out["int8_gemm_8192"] = {"ms": ms_b, "kernel": ctx.last_kernel, "tops_per_gpu": tops_b,
                             "frac_of_2x_measured_bf16_peak": tops_b / (2 * bf16_peak)}
    del layer_step  # and with it the layer's weights

    # ---- static int8 QLinearConv, ResNet block (config 4): batch 64 split over the ranks
    bsh = shard.batch_shard(64, world, rank)
    x = torch.randint(0, 256, (bsh.count, 64, 56, 56), dtype=torch.uint8, device="cuda", generator=gen)
    wc = ctx.qconv_prepack(torch.randint(-127, 128, (64, 64, 3, 3), dtype=torch.int8, device="cuda", generator=gen))
    bias = torch.randint(-1000, 1001, (64,), dtype=torch.int32, device="cuda", generator=gen)
    ratio = (0.02 * np.random.default_rng(4).uniform(0.001, 0.01, 64) / 0.05).astype(np.float32)
    yq = torch.empty((bsh.count, 64, 56, 56), dtype=torch.uint8, device="cuda")
    conv = lambda: ctx.qlinear_conv(wc, x, 128, 0, ratio, bias, 128, pads=(1, 1, 1, 1), out=yq)
    conv()
    torch.cuda.synchronize()
    conv_kernel = ctx.last_kernel
    # 25 us of GPU work against ~25 us of Python per call: replayed from a graph so that the device is timed
    gq = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gq, stream=torch.cuda.current_stream()):
        for _ in range(10):
            conv()
    ms_q = timed(torch, dist, world, gq.replay, 10) / 10
    if world == 1:
        # the residual add that follows a quantized block (resnet50: 256 x 56 x 56), one byte per element and side
        qa = torch.randint(0, 256, (64, 256, 56, 56), dtype=torch.uint8, device="cuda", generator=gen)
        qb = torch.randint(0, 256, (64, 256, 56, 56), dtype=torch.uint8, device="cuda", generator=gen)
        ctx.qlinear_add(qa, 0.02, 128, qb, 0.05, 100, 0.03, 30)
        add_kernel = ctx.last_kernel
        torch.cuda.synchronize()
        ga = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ga, stream=torch.cuda.current_stream()):
            for _ in range(5):
                ctx.qlinear_add(qa, 0.02, 128, qb, 0.05, 100, 0.03, 30)
        ms_a = timed(torch, dist, 1, ga.replay, 5) / 5
        del ga
        out["int8_qlinear_add_resnet"] = {"shape": [64, 256, 56, 56], "ms": ms_a, "kernel": add_kernel,
                                          "algorithmic_gbs": 3.0 * qa.numel() / (ms_a * 1e-3) / 1e9,
                                          "frac_of_measured_hbm": 3.0 * qa.numel() / (ms_a * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del qa, qb
    # the same layer inside a chain of quantized layers: activations stay channels-last in a frame that
    # holds the zero point (the layout the kernel computes from), so a layer is ONE launch - no layout
    # pass - and stores 16 channels per instruction into the next layer's input
    frame = (1, 1, 1, 1)
    cl_a = ctx.to_padded_nhwc(x, frame, 128)
    cl_b = torch.full_like(cl_a, 128)
    conv_cl = lambda src, dst: ctx.qlinear_conv_channels_last(wc, src, 128, 0, ratio, bias, 128, dst, frame, pads=frame)
    conv_cl(cl_a, cl_b)
    torch.cuda.synchronize()
    cl_kernel = ctx.last_kernel
    gc = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gc, stream=torch.cuda.current_stream()):
        for _ in range(5):
            conv_cl(cl_a, cl_b)
            conv_cl(cl_b, cl_a)
    ms_cl = timed(torch, dist, world, gc.replay, 10) / 10
    del gc, gq
    # (before the half-second loop below, which leaves the GPU at its power-capped clock for a while)
    resnet = resnet50_convolutions(torch, dist, ctx, gen) if world == 1 else None
    # the dense int8 peak, measured here: what back-to-back kind::i8 MMAs deliver per clock per SM, times
    # the SMs, times the clock the GPU held while this GEMM ran (sampled by nvidia-smi during a second run)
    mac_rate = ctx.probe_mma_rate(ovk_int8_code())
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    skip = sampler.wait_first_sample(lambda: (ctx.matmul_integer(big, xa, zp8, None), torch.cuda.synchronize()))
    w0 = time.perf_counter()
    while time.perf_counter() - w0 < 0.5:
        for _ in range(4):
            ctx.matmul_integer(big, xa, zp8, None)
        torch.cuda.synchronize()
    int8_clocks = sampler.stop(skip)
    sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    mhz_sustained = int8_clocks.get("sm_mhz") or 1965.0
    mhz_max = int8_clocks.get("sm_max_mhz") or 1965.0
    # fractions below are against the rate at the MAXIMUM clock, which the short timed bursts run at (the
    # smaller, stricter fraction); the rate at the clock a seconds-long run settles to is given beside it
    int8_peak = 2.0 * mac_rate * sm_count * mhz_max * 1e6 / 1e12
    out["int8_peak_tops_measured"] = {"value": int8_peak, "mac_per_clk_per_sm": mac_rate, "sms": sm_count, "sm_mhz": mhz_max,
                                      "sustained": {"value": 2.0 * mac_rate * sm_count * mhz_sustained * 1e6 / 1e12,
                                                    "sm_mhz": mhz_sustained, "clock_reasons": int8_clocks.get("reasons")},
                                      "how": "2 x MAC/clk/SM of back-to-back 128x256x32 tcgen05.mma kind::i8 (ovk_probe_mma_rate) "
                                             "x SMs x SM clock: the maximum clock, and the median sampled while the 8192^3 "
                                             "GEMM ran for half a second"}
    out["int8_gemm_8192"]["frac_of_measured_int8_peak"] = out["int8_gemm_8192"]["tops_per_gpu"] / int8_peak
    del big, xa
    ops = 2.0 * 64 * 64 * 56 * 56 * 576
    conv_bytes = 2.0 * 64 * 64 * 56 * 56
    out["int8_qlinear_conv_resnet_block"] = {"batch": 64, "ms": ms_q, "kernel": conv_kernel,
                                             "tops": ops / (ms_q * 1e-3) / 1e12,
                                             "frac_of_measured_int8_peak": ops / (ms_q * 1e-3) / 1e12 / (world * int8_peak),
                                             "frac_of_measured_hbm": conv_bytes / (ms_q * 1e-3) / 1e9 / (world * peaks["hbm_gbs"]),
                                             "channels_last_chain": {
                                                 "ms": ms_cl, "kernel": cl_kernel, "tops": ops / (ms_cl * 1e-3) / 1e12,
                                                 "frac_of_measured_int8_peak": ops / (ms_cl * 1e-3) / 1e12 / (world * int8_peak),
                                                 "frac_of_measured_hbm": conv_bytes / (ms_cl * 1e-3) / 1e9 / (world * peaks["hbm_gbs"]),
                                                 "note": "padded-NHWC in and out (ovk_qlinear_conv_layout): one launch per layer"},
                                             "algorithmic_gbs": 2.0 * 64 * 64 * 56 * 56 / (ms_q * 1e-3) / 1e9,
                                             "parallelism": "batch-split x%d, no exchange" % world if world > 1 else "single"}
    if resnet is not None:
        out["int8_resnet50_convolutions"] = resnet
    return out


# (input channels, output channels, filter, stride, input height = width, how many such layers) of ResNet-50 v1.5
RESNET50_LAYERS = [
    (3, 64, 7, 2, 224, 1),
    (64, 64, 1, 1, 56, 1), (64, 64, 3, 1, 56, 3), (64, 256, 1, 1, 56, 4), (256, 64, 1, 1, 56, 2),
    (256, 128, 1, 1, 56, 1), (128, 128, 3, 2, 56, 1), (128, 512, 1, 1, 28, 4), (512, 128, 1, 1, 28, 3), (128, 128, 3, 1, 28, 3),
    (256, 512, 1, 2, 56, 1),
    (512, 256, 1, 1, 28, 1), (256, 256, 3, 2, 28, 1), (256, 1024, 1, 1, 14, 6), (1024, 256, 1, 1, 14, 5), (256, 256, 3, 1, 14, 5),
    (512, 1024, 1, 2, 28, 1),
    (1024, 512, 1, 1, 14, 1), (512, 512, 3, 2, 14, 1), (512, 2048, 1, 1, 7, 3), (2048, 512, 1, 1, 7, 2), (512, 512, 3, 1, 7, 2),
    (1024, 2048, 1, 2, 14, 1),
]


def parakeet_layer(torch, ctx, gen, t=1000):
    """The six GEMMs of one FastConformer layer (d = 1024, FF = 4096) in the order the graph runs them, each tensor
    quantised once; returns the (K, N) list and a function that enqueues the layer."""
    import numpy as np
    layer = [(1024, 1024)] * 4 + [(1024, 4096), (4096, 1024)]
    ws, scs, bis = [], [], []
    for k, n in layer:
        ws.append(ctx.mmi_prepack(torch.randint(-127, 128, (k, n), dtype=torch.int8, device="cuda", generator=gen)))
        scs.append(torch.rand((n,), device="cuda", generator=gen) * 0.009 + 0.001)
        bis.append(torch.zeros((n,), device="cuda"))
    x_in, a_in, f_in = (torch.randn((t, 1024), device="cuda", generator=gen) for _ in range(3))
    gelu_c = (float(np.float32(np.sqrt(2.0))), 1.0, 0.5)

    def gemm(i, q):
        xq, a_scale, a_zp = q
        return ctx.matmul_integer_scale_bias(ws[i], xq, a_zp, None, scs[i], bis[i], product=a_scale.reshape(1))

    def layer_step():
        xq, a_scale, a_zp = ctx.dynamic_quantize(x_in)
        ctx.matmul_integer_scale_bias_group(ws[:3], xq, a_zp, None, scs[:3], bis[:3], product=a_scale.reshape(1))
        gemm(3, ctx.dynamic_quantize(a_in))
        h = gemm(4, ctx.dynamic_quantize(f_in))
        gemm(5, ctx.decomposed_gelu_quantize(h, *gelu_c))
    return layer, layer_step


def resnet50_convolutions(torch, dist, ctx, gen, batch=64):
    """Every convolution layer of a ResNet-50 as QLinearConv (uint8 in and out, int8 symmetric per-channel weights),
    batch 64, each shape timed from a graph replay and weighted by how often the network has it: the layers beyond
    config 4's block - large filter banks, strides, 7 x 7 planes, the 3-channel stem."""
    import numpy as np
    total_us, layers, slowest = 0.0, 0, ("", 0.0)
    kernels = {}
    for c_in, c_out, k, stride, hw, count in RESNET50_LAYERS:
        w = ctx.qconv_prepack(torch.randint(-127, 128, (c_out, c_in, k, k), dtype=torch.int8, device="cuda", generator=gen))
        x = torch.randint(0, 256, (batch, c_in, hw, hw), dtype=torch.uint8, device="cuda", generator=gen)
        bias = torch.zeros((c_out,), dtype=torch.int32, device="cuda")
        ratio = np.full(c_out, 0.002, dtype=np.float32)
        pad = k // 2
        ho = (hw + 2 * pad - k) // stride + 1
        y = torch.empty((batch, c_out, ho, ho), dtype=torch.uint8, device="cuda")
        fn = lambda: ctx.qlinear_conv(w, x, 128, 0, ratio, bias, 128, pads=(pad,) * 4, strides=(stride, stride), out=y)
        fn()
        kern = ctx.last_kernel
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
            for _ in range(3):
                fn()
        us = timed(torch, dist, 1, g.replay, 5) / 3 * 1e3
        del g, w, x, y
        total_us += us * count
        layers += count
        kernels[kern] = kernels.get(kern, 0) + count
        if us > slowest[1]:
            slowest = ("%d->%d %dx%d s%d on %dx%d" % (c_in, c_out, k, k, stride, hw, hw), us)
    return {"batch": batch, "layers": layers, "ms_all_layers": total_us / 1e3, "slowest_layer": slowest[0],
            "slowest_layer_us": slowest[1], "layers_by_last_kernel": kernels}


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
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        _run_gpu_on_stream(args, torch, dist, ovk_b200, world, rank, local, stream)
    if world > 1:
        dist.destroy_process_group()


def _run_gpu_on_stream(args, torch, dist, ovk_b200, world, rank, local, stream):
    ctx = ovk_b200.Context(local)  # bound to the current (side) stream: events and graph capture share it
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xB200 + 0x100 * 2)

    # one distinct weight per projection per layer + the lm_head
    ops = []
    for layer in range(args.layers):
        for name, k, n in LAYER_SHAPES:
            ops.append((f"L{layer}.{name}", k, n, make_weight(torch, ctx, k, n, BLOCK, gen)))
    lm = make_weight(torch, ctx, LM_HEAD[1], LM_HEAD[2], BLOCK, gen)
    acts = {k: torch.randn((1, k), device="cuda", generator=gen).to(torch.float16) for k in {HIDDEN, Q_OUT, FF}}
    # one output buffer per projection of a layer (k/v and gate/up run side by side) + the logits
    outs = {name: torch.empty((1, n), dtype=torch.float16, device="cuda") for name, _, n in LAYER_SHAPES}
    outs[VOCAB] = torch.empty((1, VOCAB), dtype=torch.float16, device="cuda")
    step_bytes = sum(nbits_bytes(1, k, n, BLOCK) for _, k, n, _ in ops) + nbits_bytes(1, LM_HEAD[1], LM_HEAD[2], BLOCK)
    lm_bytes = nbits_bytes(1, LM_HEAD[1], LM_HEAD[2], BLOCK)
    n_gemv = len(ops) + 1
    ctx.flush()

    # A decoder layer's data flow: q, k and v read the same hidden state, and so
    # do gate and up, so those launches are independent and are put on parallel
    # branches (side streams that fork from and join the main one: in the
    # captured graph these are just edges); o waits for q/k/v, down for gate/up.
    side = []
    if args.launch == "branches":
        for _ in range(2):
            s_side = torch.cuda.Stream()
            with torch.cuda.stream(s_side):
                side.append((s_side, ovk_b200.Context(local)))
    BRANCHES = {"k": 0, "v": 1, "up": 0}   # projection -> side branch; the rest stay on the main stream
    FORK_BEFORE = {"q": (0, 1), "gate": (0,)}
    JOIN_BEFORE = {"o": (0, 1), "down": (0,)}

    GROUPS = {"q": ("q", "k", "v"), "gate": ("gate", "up")}   # members that read the same activations
    by_label = {label: (k, n, w) for label, k, n, w in ops}

    def layers_grouped():
        """q|k|v and gate|up as one launch each: one serial chain of four dependent launches per layer,
        every launch overlapping its predecessor's tail (programmatic dependent launch)."""
        for label, k, n, w in ops:
            layer, name = label.split(".", 1)
            if name in GROUPS:
                members = GROUPS[name]
                ctx.matmul_nbits_group([by_label[f"{layer}.{mname}"][2] for mname in members], acts[k],
                                       outs=[outs[mname] for mname in members])
            elif not any(name in g[1:] for g in GROUPS.values()):
                ctx.matmul_nbits(w, acts[k], out=outs[name])

    def layers_eager():
        if args.launch == "grouped":
            return layers_grouped()
        for label, k, n, w in ops:
            name = label.split(".", 1)[1]
            if side:
                for b in FORK_BEFORE.get(name, ()):
                    side[b][0].wait_stream(stream)
                for b in JOIN_BEFORE.get(name, ()):
                    stream.wait_stream(side[b][0])
            if side and name in BRANCHES:
                side[BRANCHES[name]][1].matmul_nbits(w, acts[k], out=outs[name])
            else:
                ctx.matmul_nbits(w, acts[k], out=outs[name])

    # The per-layer GEMVs are launch-bound (0.2-4.6 MB each): the step replays
    # them from a CUDA graph, as the reference replays its captured decode step
    # (crates/onnx-vulkan-core/src/plan.rs, vk-compute stream.rs:537-629).
    layers_eager()
    torch.cuda.synchronize()
    # The whole step is one CUDA graph.  A second graph of the same step has the
    # lm_head launch between two event-record nodes: it is replayed after the
    # timed region to read that launch's duration from inside a step.
    graph, probe, layers_only, replay = None, None, None, "eager launches"
    g0 = torch.cuda.Event(enable_timing=True, external=True)
    g1 = torch.cuda.Event(enable_timing=True, external=True)
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                layers_eager()
                ctx.matmul_nbits(lm, acts[HIDDEN], out=outs[VOCAB])
            probe = torch.cuda.CUDAGraph()
            with torch.cuda.graph(probe, stream=stream):
                layers_eager()
                g0.record(stream)
                ctx.matmul_nbits(lm, acts[HIDDEN], out=outs[VOCAB])
                g1.record(stream)
            # the step without its last launch: the difference of the two replays is what the lm_head costs
            # inside a step with nothing fencing it (the event-record nodes above forbid the overlap of its
            # weight streaming with the previous launch's tail, which the step really has)
            layers_only = torch.cuda.CUDAGraph()
            with torch.cuda.graph(layers_only, stream=stream):
                layers_eager()
            replay = "one CUDA graph replay per step (%s)" % {
                "grouped": "q|k|v and gate|up as one launch each", "branches": "q|k|v and gate|up on parallel branches",
                "serial": "one launch per GEMV in one chain"}[args.launch]
        except Exception as e:  # capture refused: fall back to eager launches, say so
            graph, layers_only, replay = None, None, "eager launches (graph capture failed: %s)" % str(e)[:80]
            torch.cuda.synchronize()

    lm_samples = []

    def step(timed_step: bool):
        if graph is not None:
            graph.replay()
            return
        layers_eager()
        if timed_step:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ctx.matmul_nbits(lm, acts[HIDDEN], out=outs[VOCAB])
            e1.record()
            lm_samples.append((e0, e1))
        else:
            ctx.matmul_nbits(lm, acts[HIDDEN], out=outs[VOCAB])

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(False)
    sync_all()
    # clocks are sampled while the GPU runs these steps: nvidia-smi takes a few
    # hundred ms to produce its first line, so the same steps keep running
    # (untimed) until it has, and for 0.4 s after the timed region; only lines
    # written from the start of the timed region on are summarised
    sampler = ClockSampler(local)
    skip = 0
    if rank == 0:
        sampler.start()

        def busy():
            for _ in range(20):
                step(False)
            torch.cuda.synchronize()
        skip = sampler.wait_first_sample(busy)
    sync_all()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(True)
    t1.record()
    if rank == 0:
        w0 = time.perf_counter()
        while time.perf_counter() - w0 < 0.4:
            for _ in range(20):
                step(False)
            torch.cuda.synchronize()
    sync_all()
    clocks = sampler.stop(skip) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "the timed steps and 0.4 s of the same steps after them"
    per_step = n_gemv if args.launch != "grouped" else n_gemv - 3 * args.layers  # q|k|v and gate|up share a launch
    launches = per_step * args.steps  # kernels of this library (graph replays launch them too)
    ms = torch.tensor([t0.elapsed_time(t1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    # ---- the dominant launch on its own: the lm_head GEMV (30 % of the step's bytes)
    # (a) inside a step, between two event-record nodes (which also keep it from
    #     overlapping its neighbours): the record nodes hold the last replay's stamps
    if probe is not None:
        lm_times = []
        for _ in range(8):
            probe.replay()
            torch.cuda.synchronize()
            lm_times.append(g0.elapsed_time(g1))
        lm_in_step_ms = statistics.median(lm_times)
    else:
        lm_in_step_ms = statistics.mean(e0.elapsed_time(e1) for e0, e1 in lm_samples)
    # (a') the step with and without the lm_head launch, unfenced
    lm_marginal_ms = None
    if graph is not None and layers_only is not None:
        def replay_ms(g, n=20):
            g.replay()
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record()
            for _ in range(n):
                g.replay()
            r1.record()
            torch.cuda.synchronize()
            return r0.elapsed_time(r1) / n
        lm_marginal_ms = replay_ms(graph) - replay_ms(layers_only)
    # (b) back to back: a graph of launches over distinct copies of the weight (3 x 175 MB > L2),
    #     one event pair around the replays; consecutive launches overlap their ramps
    lm_copies = [lm] + [make_weight(torch, ctx, LM_HEAD[1], LM_HEAD[2], BLOCK, gen) for _ in range(2)]
    ctx.flush()
    lm_reps = 8

    def lm_run():
        for _ in range(lm_reps):
            for w in lm_copies:
                ctx.matmul_nbits(w, acts[HIDDEN], out=outs[VOCAB])
    lm_run()
    torch.cuda.synchronize()
    lm_how = "%d launches back to back over 3 copies of the weight" % (lm_reps * len(lm_copies))
    lm_graph = None
    if not args.no_graph:
        try:
            lm_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(lm_graph, stream=stream):
                lm_run()
            lm_how += ", replayed from a CUDA graph"
        except Exception:
            lm_graph = None
            torch.cuda.synchronize()
    fn = lm_graph.replay if lm_graph is not None else lm_run
    fn()
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    b0.record()
    for _ in range(3):
        fn()
    b1.record()
    torch.cuda.synchronize()
    lm_ms = b0.elapsed_time(b1) / (3 * lm_reps * len(lm_copies))
    del lm_graph
    del lm_copies
    lm_kernel = ctx.last_kernel

    # ------------------------------------------------------------ end to end
    # the call a user makes, every step: the step's inputs (the three activation
    # vectors the GEMVs read; the weights are resident, as in any decode loop)
    # come from pinned host memory, the step runs, the logits go back to the host
    pinned_in = {k: acts[k].cpu().pin_memory() for k in acts}
    pinned_out = torch.empty((1, VOCAB), dtype=torch.float16).pin_memory()
    h2d = sum(k * 2 for k in acts)
    d2h = VOCAB * 2

    def e2e_step():
        for k in acts:
            acts[k].copy_(pinned_in[k], non_blocking=True)
        step(False)
        pinned_out.copy_(outs[VOCAB], non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(3):
        e2e_step()
    sync_all()
    e2e_steps = max(1, min(args.steps, 20))
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    sync_all()
    e2e_s = torch.tensor([time.perf_counter() - w0], device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_gbs = world * step_bytes * e2e_steps / float(e2e_s.item()) / 1e9

    peaks, peak_kind = measured_peaks()
    extra = None
    if not args.no_extra:
        del ops, lm, graph, probe, layers_only
        torch.cuda.empty_cache()
        extra = extra_workloads(torch, dist, ctx, world, rank, gen, peaks)

    if rank == 0:
        achieved = lm_bytes / (lm_ms * 1e-3) / 1e9
        # dram__bytes_read.sum + dram__bytes_write.sum of one lm_head launch (174.62 MB + 4.70 MB) from an ncu
        # capture of `bench.py --one lm_head`; the weight layout that sets it has not changed since
        traffic = 179.32e6
        line = {
            "metric": "int4_decode_gemv_hbm_gbs", "value": world * step_bytes * args.steps / (ms_total * 1e-3) / 1e9,
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD % args.layers,
                       "gemvs_per_step": n_gemv, "bytes_per_step": step_bytes, "launch": replay,
                       "l2": "distinct weights per GEMV, %.0f MB per step > 126 MB L2 (no flush needed)" % (step_bytes / 1e6),
                       "parallelism": "replicas (the decode GEMV is single-GPU by design)" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "kernel": lm_kernel + " (lm_head K=1152 N=262144)", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "of": peak_kind, "bytes_per_launch": lm_bytes, "ms_per_launch": lm_ms,
                         "timing": lm_how + ", one CUDA event pair",
                         "ms_per_launch_inside_step": lm_in_step_ms,
                         "frac_inside_step": lm_bytes / (lm_in_step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "ms_marginal_inside_step": lm_marginal_ms,
                         "frac_marginal_inside_step": (lm_bytes / (lm_marginal_ms * 1e-3) / 1e9 / peaks["hbm_gbs"])
                         if lm_marginal_ms and lm_marginal_ms > 0 else None,
                         "whole_step_frac": world * step_bytes * args.steps / (ms_total * 1e-3) / 1e9 / (world * peaks["hbm_gbs"]),
                         "frac_of_nominal_8tbs": achieved / 8000.0, "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on "
                                           "this shape, captured separately (not measured in this run); 1.02 x bytes_per_launch"},
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks,
        }
        if extra is not None:
            if "partitioned" in extra:
                line["partitioned"] = extra.pop("partitioned")
            line["extra"] = extra
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.layers, budget_s=args.cpu_seconds)
        print(json.dumps(line), flush=True)


def run_one(which):
    """One operator, three launches, no timing: a bounded target for ncu."""
    import numpy as np
    import torch
    import ovk_b200
    torch.cuda.set_device(0)
    ctx = ovk_b200.Context(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xB200)
    if which == "lm_head":
        w = make_weight(torch, ctx, HIDDEN, VOCAB, BLOCK, gen)
        a = torch.randn((1, HIDDEN), device="cuda", generator=gen).to(torch.float16)
        fn = lambda: ctx.matmul_nbits(w, a)
    elif which == "prefill":
        w = make_weight(torch, ctx, 3584, 18944, 128, gen, 0.001, 0.01)
        a = torch.randn((1024, 3584), device="cuda", generator=gen).to(torch.float16)
        fn = lambda: ctx.matmul_nbits(w, a)
    elif which == "prefill32":
        w = make_weight(torch, ctx, HIDDEN, VOCAB, BLOCK, gen)
        a = torch.randn((512, HIDDEN), device="cuda", generator=gen).to(torch.float16)
        y = torch.empty((512, VOCAB), dtype=torch.float16, device="cuda")
        fn = lambda: ctx.matmul_nbits(w, a, out=y)
    elif which in ("int8", "int8big"):
        d = 4096 if which == "int8" else 8192
        w = ctx.mmi_prepack(torch.randint(-127, 128, (d, d), dtype=torch.int8, device="cuda", generator=gen))
        a = torch.randint(0, 256, (d, d), dtype=torch.uint8, device="cuda", generator=gen)
        zp = torch.full((1,), 128, dtype=torch.uint8, device="cuda")
        fn = lambda: ctx.matmul_integer(w, a, zp, None)
    elif which == "parakeet":
        _, fn = parakeet_layer(torch, ctx, gen)
    else:
        w = ctx.qconv_prepack(torch.randint(-127, 128, (64, 64, 3, 3), dtype=torch.int8, device="cuda", generator=gen))
        x = torch.randint(0, 256, (64, 64, 56, 56), dtype=torch.uint8, device="cuda", generator=gen)
        bias = torch.zeros((64,), dtype=torch.int32, device="cuda")
        ratio = np.full(64, 0.002, dtype=np.float32)
        fn = lambda: ctx.qlinear_conv(w, x, 128, 0, ratio, bias, 128, pads=(1, 1, 1, 1))
        if which == "conv_cl":  # the same layer channels-last in and out: one launch
            frame = (1, 1, 1, 1)
            xa = ctx.to_padded_nhwc(x, frame, 128)
            xb = torch.full_like(xa, 128)
            fn = lambda: ctx.qlinear_conv_channels_last(w, xa, 128, 0, ratio, bias, 128, xb, frame, pads=frame)
    for _ in range(3):
        fn()
    ctx.flush()
    print("ran", which, ctx.last_kernel)


# --------------------------------------------------------------------- CPU arm

WORKLOAD = ("gemma3-1b-int4-decode: %d layers x (q,k,v,o,gate,up,down) + lm_head, M=1, "
            "bits=4 block_size=32 zero points")


def cpu_step_inputs(layers):
    """The decode step's 7 x layers + 1 GEMVs with distinct seeded weights, in f32 (the only form the
    reference's kernel takes): 0.5 GB of nibbles, 0.13 GB of scales."""
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(0xB200 + 0x100 * 2))
    acts = {k: rng.standard_normal((1, k), dtype=np.float32) for k in (HIDDEN, Q_OUT, FF)}
    ops = []
    for name, k, n in [s for _ in range(layers) for s in LAYER_SHAPES] + [LM_HEAD]:
        nb = k // BLOCK
        b = rng.integers(0, 256, size=(n, nb, BLOCK // 2), dtype=np.uint8)
        scales = rng.random(n * nb, dtype=np.float32) * np.float32(0.018) + np.float32(0.002)
        zp = rng.integers(0, 256, size=(n, (nb + 1) // 2), dtype=np.uint8)
        ops.append((acts[k], b, scales, zp, k, n))
    byts = sum(nbits_bytes(1, k, n, BLOCK, real_bytes=4) for *_, k, n in ops)
    return ops, byts


def cpu_step(orc, ops):
    t = time.perf_counter()
    for a, b, scales, zp, k, n in ops:
        orc.matmul_nbits_f32_shader_order(a, b, scales, zp, k, n, BLOCK)
    return time.perf_counter() - t


def cpu_describe(layers, cores):
    return ("each step = the whole decode step, %d GEMVs over distinct weights, f32, the reference's shader "
            "arithmetic order (its CPU port, oracle/ovk_oracle.c, %d OpenMP threads); the reference's own GPU "
            "path needs Vulkan: unavailable on this box" % (7 * layers + 1, cores))


def cpu_baseline(layers, budget_s=12.0):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    cores = len(os.sched_getaffinity(0))
    orc.set_num_threads(cores)
    ops, byts = cpu_step_inputs(layers)
    cpu_step(orc, ops)  # warm-up
    times, spent = [], 0.0
    while spent < budget_s and len(times) < 50:
        dt = cpu_step(orc, ops)
        times.append(dt)
        spent += dt
    return {"value": byts / statistics.median(times) / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": cpu_describe(layers, cores) + "; median of %d steps" % len(times)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    cores = len(os.sched_getaffinity(0))
    orc.set_num_threads(cores)
    ops, byts = cpu_step_inputs(args.layers)
    for _ in range(max(1, args.warmup)):
        cpu_step(orc, ops)
    total = sum(cpu_step(orc, ops) for _ in range(args.steps))
    value = byts * args.steps / total / 1e9
    desc = cpu_describe(args.layers, cores)
    print(json.dumps({
        "impl": "reference", "metric": "int4_decode_gemv_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD % args.layers, "gemvs_per_step": len(ops), "bytes_per_step": byts,
                   "sample": desc},
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
    ap.add_argument("--no-extra", action="store_true", help="skip the prefill / int8 / conv lines")
    ap.add_argument("--no-graph", action="store_true", help="launch the per-layer GEMVs eagerly")
    ap.add_argument("--launch", default="grouped", choices=["grouped", "branches", "serial"],
                    help="how the independent GEMVs of a layer (q|k|v, gate|up) are launched: one launch per group, "
                         "parallel graph branches, or one launch per GEMV in a single chain")
    ap.add_argument("--one", default=None, choices=["lm_head", "prefill", "prefill32", "int8", "int8big", "conv", "conv_cl", "parakeet"],
                    help="run one operator three times and exit (small target for an ncu capture)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.one:
        run_one(args.one)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
