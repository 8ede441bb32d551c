#!/usr/bin/env python
"""Benchmark of the denoise hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (configuration 2 of the benchmark definition): the full Pi0.5-shape action expert — 18 blocks, width 1024, 8 x 256 query
heads over one KV head, 768-token prefix KV per layer + 50 action tokens, GeGLU 1024-4096-1024, FP8 E4M3 weights
and activations with static per-tensor scales, 10 Euler steps captured as ONE CUDA graph, batch 1.  Synthetic
random-init weights / prefix / noise of those shapes (seeded).  One benchmark "step" = one whole 10-step denoise
loop.  Multi-GPU: the path does not shard (M = 50 is latency-bound) -> N independent replicas, one per rank.

Prints ONE JSON line.  `value` = milliseconds per loop with the noise already on the device (graph replay only,
CUDA events, max over ranks); `e2e` = the same through ``load_model(...).predict(noise)`` with the noise in host
memory and the actions copied back to the host inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bs1 10-step action-expert denoise ms"
WORKLOAD = ("pi05 action expert: 18 blocks x 10 Euler steps, 50 action tokens, 768-token prefix KV, FP8 E4M3 "
            "weights+activations, one CUDA graph, batch 1")
WORKLOAD_NVFP4 = ("pi05 action expert (benchmark configuration 3): 18 blocks x 10 Euler steps, 50 action tokens, 768-token "
                  "prefix KV, NVFP4 weights (FP32 global scale) + activations in all four projections, bf16 "
                  "attention, one CUDA graph, batch %d")


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
def cpu_reference_loop(steps: int, warmup: int, layers: int = 18):
    """The reference's torch math for this path (fp32, CPU): oracle.block_ref.denoise_loop on all host cores."""
    import torch
    from oracle import block_ref as R
    from flashrt_b200.pi05_decoder import synthetic_state_dict
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sd = synthetic_state_dict(0, layers)
    ck = R.from_hf_state_dict(sd, layers)
    pk, pv = R.synthetic_prefix_kv(1, layers)
    noise = R.synthetic_noise(1)
    for _ in range(warmup):
        R.denoise_loop(noise, ck, pk, pv, layers=layers)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        R.denoise_loop(noise, ck, pk, pv, layers=layers)
        ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts), cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    ms, cores = cpu_reference_loop(steps, min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ms, 3), "unit": "ms", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": round(ms, 3), "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "reference torch math of the path (fp32) on the host CPU cores"},
        "cpu_baseline": {"value": round(ms, 3), "unit": "ms", "cores": cores, "kind": "port",
                         "sample": f"{steps} full 10-step loops, median"},
        "e2e": {"value": round(ms, 3), "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
def gemm_roofline(fe, reps: int = 20):
    """Average duration of the dominant kernel (the small-M FP8 GEMM that streams the weights): a graph holding
    exactly the 4 x 18 GEMM launches of one Euler step, each on its own layer's weights (311 MB > L2), timed with
    CUDA events on the launching stream."""
    import torch
    p, s = fe.pipeline, fe.stream
    S, L = fe.chunk_size * fe.batch, fe.layers
    nv = fe.precision == "nvfp4"
    if nv:
        shapes = [("qkv", None, (p.act4, p.act4_sf), p.qkv, 2560, 1024), ("o", None, (p.ctx4, p.ctx4_sf), p.xn, 1024, 2048),
                  ("gu", None, (p.act4, p.act4_sf), p.merged, 8192, 1024), ("d", None, (p.hid4, p.hid4_sf), p.xn, 1024, 4096)]
    else:
        shapes = [("w_qkv", "ws_qkv_t", p.act8, p.qkv, 2560, 1024), ("w_o", "ws_o_t", p.attn8, p.xn, 1024, 2048),
                  ("w_gu", "ws_gu_t", p.act8, p.merged, 8192, 1024), ("w_d", "ws_d_t", p.hid8, p.xn, 1024, 4096)]

    def enqueue():
        for i in range(L):
            for wn, sn, a8, out, N, K in shapes:
                if nv:
                    p._gemm(a8[0], a8[1], fe.w4[i][wn], out, s.cuda_stream, fe.use_pdl)
                else:
                    p._gemm(a8, getattr(fe, wn)[i], getattr(fe, sn)[i], out, S, N, K, p._scale_ptr(0, i, "qkv"),
                            s.cuda_stream, fe.use_pdl)

    with torch.cuda.stream(s):
        enqueue()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s, capture_error_mode="relaxed"):
            enqueue()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            g.replay()
        e1.record(s)
        s.synchronize()
    launches = len(shapes) * L
    us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
    eb = 0.5625 if nv else 1.0          # bytes per operand element (NVFP4: 4 bits + one scale byte per 16)
    bytes_per_launch = sum(eb * (N * K + S * K) + 2 * S * N for *_, N, K in shapes) / len(shapes)
    return us, bytes_per_launch, launches


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from flashrt_b200 import load_model
    from flashrt_b200.pi05_decoder import ACTION_DIM
    gsd = torch.Generator().manual_seed(1)
    nv = args.precision == "nvfp4"
    model = load_model("synthetic:0", config="pi05", device=local, use_pdl=not args.no_pdl,
                       precision=args.precision, batch=args.batch, persistent_loop=args.persistent_loop)
    fe = model.frontend
    L, P = fe.layers, fe.prefix_len
    model.set_prefix(torch.randn(L, P, 256, generator=gsd), torch.randn(L, P, 256, generator=gsd))
    cal = [torch.randn(fe.chunk_size, ACTION_DIM, generator=torch.Generator().manual_seed(100 + j)) for j in range(args.calib_samples)]
    model.calibrate(cal)                  # no-op for NVFP4 (block scales are computed at run time)
    nshape = (fe.chunk_size, ACTION_DIM) if fe.batch == 1 else (fe.batch, fe.chunk_size, ACTION_DIM)
    noise = torch.randn(*nshape, generator=torch.Generator().manual_seed(7)).numpy()
    model.predict(noise=noise)            # captures the graph

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    s = fe.stream
    # ---- device-resident timing: graph replay only
    for _ in range(max(args.warmup, 3)):
        fe.forward_decode_only()
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    torch.cuda.profiler.start()      # no-op unless a profiler was attached with --profile-from-start off
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s)
    for _ in range(args.steps):
        fe.forward_decode_only()
    e1.record(s)
    barrier()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    # ---- end to end through the public API: host noise in, host actions out
    for _ in range(3):
        model.predict(noise=noise)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = model.predict(noise=noise)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    barrier()

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        from flashrt_b200 import flash_rt_kernels as fvk
        status = fvk.tensor_core_status()
        peak, peak_src = _peaks()
        if args.loop_trace:
            loop_trace_report(ms)
        if args.lean:
            print(json.dumps({"metric": METRIC, "value": round(ms, 4), "unit": "ms", "lean": True,
                              "e2e_ms": round(e2e_ms, 4), "tensor_core_status": status}), flush=True)
            if world > 1:
                dist.destroy_process_group()
            return
        gemm_us, gemm_bytes, _ = gemm_roofline(fe)
        alt = (persistent_loop_ms(local, args.calib_samples)
               if (not nv and fe.batch == 1 and not args.persistent_loop) else None)
        M = fe.batch * fe.chunk_size
        gemm_out_bytes = 2 * M * (2560 + 1024 + 8192 + 1024) / 4
        achieved = gemm_bytes / (gemm_us * 1e-6) / 1e9
        # algorithmic HBM bytes of one loop: weights (FP8: 1 byte, NVFP4: 0.5625 byte per element with the
        # block scales) + prefix/fresh KV per layer per step (per batch element)
        wbytes = 17301504 * (0.5625 if nv else 1.0)
        loop_bytes = int(fe.num_steps * L * (wbytes + fe.batch * 2 * (P + fe.chunk_size) * 256 * 2))
        cpu_ms, cores = cpu_reference_loop(3, 1, L)
        line = {
            "metric": METRIC, "value": round(ms, 4), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None,
            "dtype": ("nvfp4_e2m1 (ue4m3 block scales, fp32 accumulate, bf16 residual stream)" if nv
                      else "fp8_e4m3 (fp32 accumulate, bf16 residual stream)"),
            "data": "synthetic",
            "config": {"workload": (WORKLOAD_NVFP4 % fe.batch) if nv else WORKLOAD,
                       "parallelism": f"replicas x{world} (no collective)",
                       "l2": ("working set %d MB per Euler step exceeds the 126 MB L2; no explicit flush"
                              % (loop_bytes // fe.num_steps // 1000000)),
                       "kernels_per_loop": fe.kernels_per_loop(), "pdl": fe.use_pdl,
                       "calibration_samples": args.calib_samples,
                       "tensor_core_status": status, "actions_finite": bool((out == out).all())},
            "e2e": {"value": round(e2e_ms, 4), "unit": "ms", "h2d_bytes_per_step": int(noise.nbytes),
                    "d2h_bytes_per_step": int(out.nbytes)},
            "gpu_launches": fe.kernels_per_loop() * args.steps,
            "aggregate_loops_per_s": round(world * 1e3 / ms, 2),
            # the same loop as ONE persistent cooperative kernel (opt-in composition, reported beside the default)
            "persistent_loop": alt,
            "loop_hbm_floor": {"algorithmic_bytes": loop_bytes, "floor_ms": round(loop_bytes / (peak * 1e9) * 1e3, 4),
                               "frac": round(loop_bytes / (peak * 1e9) * 1e3 / ms, 4)},
            "roofline": {"bound": "hbm", "kernel": ("gemm_fp8_kernel<..,true,..,NVFP4> (M=%d weight streaming)" % M
                                                    if nv else "gemm_fp8_kernel<64,true> (M=50 weight streaming)"),
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # dram read+write of one launch from the ncu capture in profiles/ (1.005 x the algorithmic
                         # read bytes; the bf16 result stays in L2), scaled to the average launch by bytes
                         "traffic": int(1.005 * (gemm_bytes - gemm_out_bytes)), "peak_source": peak_src,
                         "avg_launch_us": round(gemm_us, 3), "algorithmic_bytes_per_launch": int(gemm_bytes)},
            "cpu_baseline": {"value": round(cpu_ms, 2), "unit": "ms", "cores": cores, "kind": "port",
                             "sample": "3 full 10-step loops of the fp32 torch oracle, median"},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
WAN_METRIC = "video-DiT step ms"
WAN_WORKLOAD = ("wan2.2-5B-shape DiT step: 30 blocks, width 3072, 24 heads x 128, FFN 14336 GELU-tanh, adaLN, "
                "cross-attention to 512 text tokens of width 4096, 13x30x52 = 20280 latent tokens, batch 2, "
                "FP8 E4M3 GEMMs + bf16 attention")


def run_wan(args):
    """Benchmark configuration 4: one denoise step of the video DiT, tensor-parallel over the N GPUs (strong scaling)."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from flashrt_b200.wan_dit import WanDiTB200, synthetic_wan_state
    layers = args.wan_layers
    state = synthetic_wan_state(0, layers=1)
    grid, B, T = (13, 30, 52), 2, 512
    model = WanDiTB200(state, grid=grid, batch=B, text_len=T, device=local, tp_rank=rank, tp_size=world,
                       repeat_blocks=layers, overlap_chunks=args.wan_overlap_chunks)
    L, D = model.L, model.dim
    g = torch.Generator().manual_seed(1)
    x_host = torch.randn(B, L, D, generator=g).to(torch.bfloat16).pin_memory()
    ctx = torch.randn(B, T, 4096, generator=g)
    tproj = torch.randn(B, 6, D, generator=g) * 0.3
    x_dev = x_host.to(f"cuda:{local}")
    model.set_context(ctx)
    model.calibrate(x_dev, tproj)
    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        model.step(x_dev, tproj)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = model.step(x_dev, tproj)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    t0 = time.perf_counter()
    for _ in range(steps):
        xd = x_host.to(f"cuda:{local}", non_blocking=True)
        out_host = model.step(xd, tproj).cpu()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    clocks = sampler.stop()
    barrier()
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        from flashrt_b200 import flash_rt_kernels as fvk
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
            os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops_sustained": 1400.0}
        gemm_flop = 2.0 * B * L * (3072 * 9216 + 3 * 3072 * 3072 + 2 * 3072 * 14336) * layers
        attn_flop = 4.0 * L * L * 3072 * B * layers + 4.0 * L * T * 3072 * B * layers
        achieved = (gemm_flop + attn_flop) / world / (ms * 1e-3) / 1e12
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        line = {
            "metric": WAN_METRIC, "value": round(ms, 2), "unit": "ms", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": round(ms, 2), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 GEMMs (fp32 accumulate), bf16 attention", "data": "synthetic",
            "config": {"workload": WAN_WORKLOAD, "layers": layers, "parallelism": f"tp{world} (heads + FFN columns, "
                       "NCCL all-reduce after attention-out, cross-attention-out and FFN-down)",
                       "l2": "activations of one step (> 1 GB) exceed the 126 MB L2; no explicit flush",
                       "tensor_core_status": fvk.tensor_core_status(), "finite": bool(torch.isfinite(out.float()).all())},
            "e2e": {"value": round(e2e_ms, 2), "unit": "ms", "h2d_bytes_per_step": int(x_host.numel() * 2),
                    "d2h_bytes_per_step": int(out_host.numel() * 2)},
            "gpu_launches": model.launches_per_step * steps,
            "roofline": {"bound": "tensor", "kernel": "whole step (FP8 GEMMs + bf16 attention), per GPU",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                         "frac": round(achieved / peak, 4), "traffic": None,
                         "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (bf16 peak; FP8 GEMMs can exceed it)",
                         "flop_per_step": gemm_flop + attn_flop},
            "cpu_baseline": None, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
def run_ops(args):
    """Operator sweep (benchmark configuration 1) on one GPU: fused residual + RMSNorm + FP8 quantise over row widths,
    FP8 and NVFP4 GEMMs over M x (N, K).  Every case is timed as a CUDA graph of launches that cycle through
    enough distinct buffers to exceed L2, with CUDA events around the replays.  One JSON line; the table is in
    ``config.table`` (GB/s for the norm, TFLOP/s for the GEMMs, with the fraction of the measured peak)."""
    import torch
    from flashrt_b200 import _lib
    from flashrt_b200 import flash_rt_fp4 as fp4
    torch.cuda.set_device(0)
    peak_hbm, _ = _peaks()
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            bf16_tf = float(json.load(f)["bf16_tflops"])
    except Exception:
        bf16_tf = 1590.0
    fp8_peak, fp4_peak = 2 * bf16_tf, 4 * bf16_tf
    s = torch.cuda.Stream()
    L2 = 160e6
    launches = 0

    def timed(enqueue, n_launch, reps=5):
        with torch.cuda.stream(s):
            enqueue()
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s, capture_error_mode="relaxed"):
                enqueue()
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            for _ in range(reps):
                g.replay()
            e1.record(s)
            s.synchronize()
        nonlocal launches
        launches += n_launch * (1 + 3 + reps)
        return e0.elapsed_time(e1) * 1e-3 / (reps * n_launch)

    table = []
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    # ---- K3 fused residual + RMSNorm + FP8 quantise
    for W in (1024, 2048, 3072, 4096):
        rows = 81920
        nbuf = max(2, int(L2 // (rows * W * 7)) + 1)
        res = [torch.randn(rows, W, device="cuda").bfloat16() for _ in range(nbuf)]
        x = [torch.randn(rows, W, device="cuda").bfloat16() for _ in range(nbuf)]
        out = [torch.empty(rows, W, dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
        wt = torch.ones(W, device="cuda").bfloat16()
        def enq():
            for i in range(nbuf):
                _lib.call("frt_b200_norm_fp8", res[i].data_ptr(), x[i].data_ptr(), None, 0, wt.data_ptr(), None, 0,
                          out[i].data_ptr(), None, rows, W, 1e-6, one.data_ptr(), 0, s.cuda_stream)
        t = timed(enq, nbuf)
        gbs = rows * W * 7 / t / 1e9
        table.append({"op": "residual_add_rms_norm_fp8", "rows": rows, "width": W, "us": round(t * 1e6, 2),
                      "GB/s": round(gbs, 1), "frac_hbm": round(gbs / peak_hbm, 3)})
        del res, x, out
    # ---- GEMMs
    NK = [(1024, 1024), (4096, 1024), (1024, 4096), (3072, 3072), (14336, 3072), (3072, 14336)]
    gemm_flags = 8 if args.cta_pair else 0       # bit 3: the 256 x 256-tile kernel on CTA pairs for M > 256
    for kind in ("fp8", "nvfp4"):
        for M in (16, 50, 256, 2048, 8192, 20480):
            for N, K in NK:
                eb = 1.0 if kind == "fp8" else 0.5
                wbytes = N * K * eb
                nbuf = max(1, min(160, int(L2 // wbytes) + 1)) if M <= 256 else 2
                A = torch.randint(0, 256, (M, int(K * eb)), dtype=torch.uint8, device="cuda")
                Ws = [torch.randint(0, 120, (N, int(K * eb)), dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
                D = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                if kind == "fp8":
                    A &= 0x77                      # finite E4M3 codes
                    def enq():
                        for w in Ws:
                            _lib.call("frt_b200_gemm_fp8_nt", A.data_ptr(), w.data_ptr(), D.data_ptr(), M, N, K,
                                      one.data_ptr(), one.data_ptr(), 1.0, None, 0, gemm_flags if M > 256 else 0,
                                      s.cuda_stream)
                else:
                    sfa = torch.full((fp4.sfa_size_bytes(M, K),), 0x38, dtype=torch.uint8, device="cuda")
                    sfw = torch.full((fp4.sfa_size_bytes(N, K),), 0x30, dtype=torch.uint8, device="cuda")
                    def enq():
                        for w in Ws:
                            _lib.call("frt_b200_gemm_nvfp4_nt", A.data_ptr(), sfa.data_ptr(), w.data_ptr(),
                                      sfw.data_ptr(), D.data_ptr(), M, N, K, 1.0, None, None, 0, 0, s.cuda_stream)
                t = timed(enq, nbuf, reps=3 if M >= 2048 else 10)
                tf = 2.0 * M * N * K / t / 1e12
                ob = 0.5625 if kind == "nvfp4" else 1.0
                gbs = (ob * (N * K + M * K) + 2 * M * N) / t / 1e9
                table.append({"op": "gemm_" + kind, "M": M, "N": N, "K": K, "us": round(t * 1e6, 2),
                              "TFLOP/s": round(tf, 1),
                              "frac_tensor": round(tf / (fp8_peak if kind == "fp8" else fp4_peak), 3),
                              "GB/s": round(gbs, 1), "frac_hbm": round(gbs / peak_hbm, 3)})
                del A, Ws, D
    from flashrt_b200 import flash_rt_kernels as fvk
    big = [r for r in table if r["op"] == "gemm_fp8" and r["M"] >= 2048]
    line = {"metric": "operator sweep (configs[1])", "value": round(statistics.mean(r["frac_tensor"] for r in big), 4),
            "unit": "mean fraction of 2 x measured bf16 peak over the FP8 GEMMs with M >= 2048", "n_gpus": 1,
            "steps": 1, "warmup": 3, "higher_is_better": True, "data": "synthetic", "dtype": "fp8_e4m3 / nvfp4 / bf16",
            "config": {"workload": "configs[1] operator sweep", "peaks": {"hbm_gbs": peak_hbm, "fp8_tflops": fp8_peak,
                                                                           "nvfp4_tflops": fp4_peak,
                                                                           "note": "tensor peaks = 2x / 4x the measured cuBLAS bf16 burst"},
                       "l2": ("norm and M <= 256 GEMM cases cycle through distinct row / weight buffers totalling more than "
                              "L2; M >= 2048 GEMM cases alternate two weight buffers (tensor-bound)"),
                       "large_m_fp8_kernel": "cta pair (256 x 256 tiles)" if args.cta_pair else "persistent, one CTA per tile",
                       "tensor_core_status": fvk.tensor_core_status(), "table": table},
            "gpu_launches": launches}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
def run_prefix(args):
    """The step in front of the denoise path: 18 Gemma-2B encoder layers (FP8) turning a 768-token prefix into the
    per-layer K / V of the action expert.  One "step" = one encode() of the whole prefix."""
    import torch
    from flashrt_b200.pi05_prefix import ENC_D, ENC_H, ENC_L, Pi05PrefixEncoderB200, QKV_N
    torch.cuda.set_device(0)
    seq, L = 768, ENC_L
    enc = Pi05PrefixEncoderB200("synthetic:0", layers=L, max_seq=seq)
    g = torch.Generator().manual_seed(3)
    embeds = torch.randn(seq, ENC_D, generator=g).to(torch.bfloat16)
    enc.calibrate([embeds])
    k = torch.zeros(L, seq + 50, 256, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    emb_dev = embeds.cuda()
    st = enc.stream
    for _ in range(max(args.warmup, 3)):
        enc.encode(emb_dev, k, v)
    sampler = ClockSampler(0)
    sampler.start()
    steps = max(1, min(args.steps, 50))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(st):
        enc.x[:seq].copy_(emb_dev)
        e0.record(st)
        for _ in range(steps):
            enc.transformer_encoder(seq, k, v, st.cuda_stream, False)
        e1.record(st)
    st.synchronize()
    ms = e0.elapsed_time(e1) / steps
    embeds_pin = embeds.pin_memory()
    t0 = time.perf_counter()
    for _ in range(steps):
        enc.encode(embeds_pin, k, v)
        probe = k[L - 1, seq - 1, :8].cpu()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    clocks = sampler.stop()
    from flashrt_b200 import flash_rt_kernels as fvk
    flop = (L - 1) * (2.0 * seq * ENC_D * (QKV_N + 2048 + 2 * ENC_H + ENC_H) + 4.0 * seq * seq * 2048) \
        + 2.0 * seq * ENC_D * QKV_N
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            bf16_tf = float(json.load(f)["bf16_tflops"])
    except Exception:
        bf16_tf = 1590.0
    launches = (L - 1) * 9 + 3
    line = {"metric": "prefix encoder ms (768 tokens, 18 Gemma-2B layers, FP8)", "value": round(ms, 4), "unit": "ms",
            "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 GEMMs, bf16 attention",
            "data": "synthetic",
            "config": {"workload": "pi05 prefix producer: 768 x 2048 embeddings -> per-layer K/V (18 layers, FFN 16384)",
                       "l2": "2.0 GB of FP8 weights per pass exceed L2", "tensor_core_status": fvk.tensor_core_status(),
                       "finite": bool(torch.isfinite(probe.float()).all())},
            "e2e": {"value": round(e2e_ms, 4), "unit": "ms", "h2d_bytes_per_step": int(embeds.numel() * 2),
                    "d2h_bytes_per_step": 16},
            "gpu_launches": launches * steps,
            "roofline": {"bound": "tensor", "kernel": "whole pass (FP8 GEMMs at M = 768 + attention)",
                         "achieved": round(flop / (ms * 1e-3) / 1e12, 1), "peak": 2 * bf16_tf, "unit": "TFLOP/s",
                         "frac": round(flop / (ms * 1e-3) / 1e12 / (2 * bf16_tf), 4), "traffic": None,
                         "peak_source": "2 x measured bf16 burst (MEASURED_PEAKS.json)"},
            "clocks": clocks}
    print(json.dumps(line), flush=True)


def persistent_loop_ms(local: int, calib_samples: int):
    """The same workload through ``persistent_loop=True`` (one cooperative launch per loop), timed by a child process
    (``bench.py --persistent-loop --lean``) on the same GPU so that nothing it does can disturb this process's
    measurement.  Never fails the bench: errors are reported in the value."""
    env = dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK=str(local))
    for k in ("MASTER_ADDR", "MASTER_PORT", "GROUP_RANK", "LOCAL_WORLD_SIZE", "TORCHELASTIC_RUN_ID"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.abspath(__file__), "--persistent-loop", "--lean", "--steps", "50", "--warmup", "5",
           "--calib-samples", str(calib_samples)]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
        rec = json.loads(r.stdout.strip().splitlines()[-1])
        return {"ms": rec["value"], "e2e_ms": rec["e2e_ms"], "launches_per_loop": 1,
                "tensor_core_status": rec["tensor_core_status"]}
    except Exception as e:  # noqa: BLE001
        return {"error": f"{type(e).__name__}: {e}"[:200]}


def loop_trace_report(ms: float) -> None:
    """Phase timing of the persistent loop kernel from its device-side stamps (library built with
    ``FRT_NVCC_EXTRA=-DFRT_LOOP_TRACE``): worker thread 0 of every CTA stamps %globaltimer at the start and end of each
    phase of two decoder blocks of the second Euler step, the MMA thread when it sees its operands and when it has
    issued its last MMA.  Printed to stderr; the JSON line on stdout is unchanged."""
    import ctypes
    import numpy as np
    from flashrt_b200 import _lib
    lib = _lib.load()
    if not hasattr(lib, "frt_loop_trace_read"):
        print("loop trace: the library was built without -DFRT_LOOP_TRACE", file=sys.stderr)
        return
    buf = (ctypes.c_ulonglong * (160 * 128))()
    lib.frt_loop_trace_read.argtypes = [ctypes.c_void_p]
    lib.frt_loop_trace_read(ctypes.addressof(buf))
    t = np.frombuffer(buf, dtype=np.uint64).reshape(160, 128).astype(np.int64)
    names = ["A rows", "B qkv", "C attention", "D combine", "E o-proj", "F rows", "G gate|up", "H down"]
    tr = {1: 40, 4: 42, 6: 44, 7: 46}
    out = [f"persistent loop: {ms:.3f} ms per loop; phase times in us (second Euler step, blocks 0 and 1)"]
    for blk in range(2):
        tt = t[:148, blk * 64: blk * 64 + 64]
        out.append(f"block {blk}: {(tt[:, 32].max() - tt[:, 0].min()) / 1e3:.2f} us")
        out.append("  phase         whole  slowest-CTA work  barrier (last arrival -> first release)  owners: operands in smem | MMA issue | epilogue")
        for k, nm in enumerate(names):
            st, en, nx = tt[:, 4 * k], tt[:, 4 * k + 3], tt[:, 4 * k + 4]
            line = (f"  {nm:12s} {(nx.max() - st.min()) / 1e3:6.2f} {(en - st).max() / 1e3:10.2f} "
                    f"{(nx.min() - en.max()) / 1e3:18.2f}")
            if k in tr:
                own = (tt[:, tr[k]] > st) & (tt[:, tr[k]] < st + 100000)
                if own.any():
                    med = lambda a, b: float(np.median((tt[:, a] - tt[:, b])[own])) / 1e3  # noqa: E731
                    line += (f"{'':22s}{int(own.sum()):3d}: {med(tr[k], 4 * k):.2f} | {med(tr[k] + 1, tr[k]):.2f} | "
                             f"{med(4 * k + 3, 4 * k + 2):.2f}")
            out.append(line)
    print("\n".join(out), file=sys.stderr, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--calib-samples", type=int, default=8, help="calibration noises (8 = the named config)")
    ap.add_argument("--no-pdl", action="store_true",
                    help="chain kernels with plain stream order instead of programmatic dependent launch "
                         "(Nsight Compute cannot profile programmatically dependent launches)")
    ap.add_argument("--persistent-loop", action="store_true",
                    help="pi05 / fp8: run the whole denoise loop as one persistent cooperative kernel")
    ap.add_argument("--cta-pair", action="store_true",
                    help="--workload ops: run the FP8 GEMMs with M > 256 through the CTA-pair kernel")
    ap.add_argument("--loop-trace", action="store_true",
                    help="with --persistent-loop and a library built with FRT_NVCC_EXTRA=-DFRT_LOOP_TRACE: print the "
                         "kernel's phase timing to stderr")
    ap.add_argument("--lean", action="store_true",
                    help="skip the CPU baseline and the GEMM roofline leg (for short runs under a profiler)")
    ap.add_argument("--workload", default="pi05", choices=["pi05", "wan", "ops", "prefix"],
                    help="pi05 = the headline action-expert loop (default); wan = the video-DiT step (configs[4]); "
                         "ops = the operator sweep of configs[1] (norm / FP8 GEMM / NVFP4 GEMM)")
    ap.add_argument("--precision", default="fp8", choices=["fp8", "nvfp4"],
                    help="pi05 workload: fp8 = configs[2] (default, the headline), nvfp4 = configs[3]")
    ap.add_argument("--batch", type=int, default=1, help="pi05 workload with --precision nvfp4: chunks per loop (1 or 4)")
    ap.add_argument("--wan-layers", type=int, default=30)
    ap.add_argument("--wan-overlap-chunks", type=int, default=int(os.environ.get("FRT_WAN_CHUNKS", "4")),
                    help="wan workload under TP: pieces per row-parallel GEMM whose all-reduce overlaps the next piece")
    args = ap.parse_args()
    if args.workload == "wan" and args.impl != "reference":
        run_wan(args)
        return
    if args.workload == "ops" and args.impl != "reference":
        run_ops(args)
        return
    if args.workload == "prefix" and args.impl != "reference":
        run_prefix(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
