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
def cpu_reference_loop(steps: int, warmup: int, layers: int = 18, inputs=None):
    """The reference's torch math for this path (fp32, CPU): oracle.block_ref.denoise_loop on all host cores.
    ``inputs`` = (prefix_k, prefix_v, noise) of the device arm (so that the two outputs can be compared); seeded
    stand-ins otherwise.  Returns (median ms, cores, actions of the last run)."""
    import torch
    from oracle import block_ref as R
    from flashrt_b200.pi05_decoder import synthetic_state_dict
    torch.set_num_threads(os.cpu_count() or 1)    # a launcher may have exported OMP_NUM_THREADS=1
    cores = torch.get_num_threads()
    sd = synthetic_state_dict(0, layers)
    ck = R.from_hf_state_dict({k: v.to(torch.bfloat16).float() for k, v in sd.items()}, layers)
    if inputs is None:
        pk, pv = R.synthetic_prefix_kv(1, layers)
        noise = R.synthetic_noise(1)
    else:
        pk, pv, noise = (t.to(torch.bfloat16).float() for t in inputs)
    for _ in range(warmup):
        R.denoise_loop(noise, ck, pk, pv, layers=layers)
    ts, out = [], None
    for _ in range(steps):
        t0 = time.perf_counter()
        out = R.denoise_loop(noise, ck, pk, pv, layers=layers)
        ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts), cores, out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    ms, cores, _ = cpu_reference_loop(steps, min(args.warmup, 1))
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
    """Average duration of the dominant kernel family (the small-M FP8 projections that stream the weights): a graph
    holding exactly the 4 x 18 projection launches of one Euler step as the loop issues them (folded norms and fused
    epilogues included), each on its own layer's weights (311 MB > L2), timed with CUDA events on the launching
    stream.  Returns (us per launch, algorithmic bytes per launch, launches)."""
    import torch
    p, s = fe.pipeline, fe.stream
    S, L = fe.chunk_size * fe.batch, fe.layers
    nv = fe.precision == "nvfp4"
    st = s.cuda_stream
    if nv:
        shapes = [("qkv", None, (p.act4, p.act4_sf), p.qkv, 2560, 1024), ("o", None, (p.ctx4, p.ctx4_sf), p.xn, 1024, 2048),
                  ("gu", None, (p.act4, p.act4_sf), p.merged, 8192, 1024), ("d", None, (p.hid4, p.hid4_sf), p.xn, 1024, 4096)]
    else:
        shapes = [("w_qkv", "ws_qkv_t", p.act8, p.qkv, 2560, 1024), ("w_o", "ws_o_t", p.attn8, p.xn, 1024, 2048),
                  ("w_gu", "ws_gu_t", p.act8, p.merged, 8192, 1024), ("w_d", "ws_d_t", p.hid8, p.xn, 1024, 4096)]
    folded = (not nv) and p._folds_norms()

    def enqueue():
        if folded:
            p._folded_layers(0, st, fe.use_pdl, attention=False)
            return
        for i in range(L):
            for wn, sn, a8, out, N, K in shapes:
                if nv:
                    p._gemm(a8[0], a8[1], fe.w4[i][wn], out, st, fe.use_pdl)
                else:
                    p._gemm(a8, getattr(fe, wn)[i], getattr(fe, sn)[i], out, S, N, K, p._scale_ptr(0, i, "qkv"),
                            st, fe.use_pdl)

    with torch.cuda.stream(s):
        if folded:
            keep = p.x.clone()
            p.row_stats.fill_(64.0)
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
        if folded:
            p.x.copy_(keep)
    launches = len(shapes) * L
    us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
    eb = 0.5625 if nv else 1.0          # bytes per operand element (NVFP4: 4 bits + one scale byte per 16)
    bytes_per_launch = sum(eb * (N * K + S * K) + 2 * S * N for *_, N, K in shapes) / len(shapes)
    return us, bytes_per_launch, launches


def _pctl(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(q * (len(xs) - 1))))]


def run_ours(args):
    import torch
    import torch.distributed as dist
    t_start = time.perf_counter()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))

    from flashrt_b200 import load_model
    from flashrt_b200.pi05_decoder import ACTION_DIM
    gsd = torch.Generator().manual_seed(1)
    nv = args.precision == "nvfp4"
    model = load_model("synthetic:0", config="pi05", device=local, use_pdl=not args.no_pdl,
                       precision=args.precision, batch=args.batch, persistent_loop=args.persistent_loop)
    fe = model.frontend
    L, P = fe.layers, fe.prefix_len
    prefix_k, prefix_v = torch.randn(L, P, 256, generator=gsd), torch.randn(L, P, 256, generator=gsd)
    model.set_prefix(prefix_k, prefix_v)
    cal = [torch.randn(fe.chunk_size, ACTION_DIM, generator=torch.Generator().manual_seed(100 + j)) for j in range(args.calib_samples)]
    model.calibrate(cal)                  # no-op for NVFP4 (block scales are computed at run time)
    nshape = (fe.chunk_size, ACTION_DIM) if fe.batch == 1 else (fe.batch, fe.chunk_size, ACTION_DIM)
    noise_t = torch.randn(*nshape, generator=torch.Generator().manual_seed(7))
    noise = noise_t.numpy()
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
    # ---- distribution of single replays (events around every replay; the mean above stays the value)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in evs:
        a.record(s)
        fe.forward_decode_only()
        b.record(s)
    s.synchronize()
    per = [a.elapsed_time(b) for a, b in evs]
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

    from flashrt_b200 import flash_rt_kernels as fvk
    status = fvk.tensor_core_status()
    if args.lean:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": round(ms, 4), "unit": "ms", "lean": True,
                              "e2e_ms": round(e2e_ms, 4), "tensor_core_status": status}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    M = fe.batch * fe.chunk_size
    kernels_per_loop, num_steps, batch, use_pdl = fe.kernels_per_loop(), fe.num_steps, fe.batch, fe.use_pdl
    gemm_us = gemm_bytes = None
    if rank == 0:
        gemm_us, gemm_bytes, _ = gemm_roofline(fe)
    # ---- the other configurations of the benchmark definition, measured after the headline (never inside it).
    # Whether an extra runs is decided on rank 0 and told to every rank: the video-DiT step is a collective.
    extras = {}
    if not args.no_extras:
        del model, fe
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        go = torch.tensor([1 if time.perf_counter() - t_start < args.extras_budget_s else 0], device=f"cuda:{local}")
        if world > 1:
            dist.broadcast(go, src=0)
        if int(go[0]):
            try:
                w = measure_wan(args, rank, world, local, steps=3, warm=1)
                extras["video_dit"] = {"ms": w["ms"], "e2e_ms": w["e2e_ms"], "tp": world, "layers": w["layers"],
                                       "frac_weighted": w["frac_weighted"], "finite": w["finite"],
                                       "tensor_core_status": w["status"], "launches_per_step": w["launches"]}
            except Exception as e:  # noqa: BLE001
                extras["video_dit"] = {"error": f"{type(e).__name__}: {e}"[:200]}
        else:
            extras["video_dit"] = {"skipped": "time budget of the default run"}
        if world == 1 and rank == 0:
            for name, fn in (("ops", lambda: ops_summary(args)), ("nvfp4", lambda: nvfp4_summary(args, local))):
                if time.perf_counter() - t_start > args.extras_budget_s:
                    extras[name] = {"skipped": "time budget of the default run"}
                    continue
                try:
                    extras[name] = fn()
                except Exception as e:  # noqa: BLE001
                    extras[name] = {"error": f"{type(e).__name__}: {e}"[:200]}
    if rank == 0:
        peak, peak_src = _peaks()
        gemm_out_bytes = 2 * M * (2560 + 1024 + 8192 + 1024) / 4
        achieved = gemm_bytes / (gemm_us * 1e-6) / 1e9
        # algorithmic HBM bytes of one loop: weights (FP8: 1 byte, NVFP4: 0.5625 byte per element with the
        # block scales) + prefix/fresh KV per layer per step (per batch element)
        wbytes = 17301504 * (0.5625 if nv else 1.0)
        loop_bytes = int(num_steps * L * (wbytes + batch * 2 * (P + M // batch) * 256 * 2))
        # the CPU port of the reference math on the SAME prefix and noise: the baseline time, and the check that the
        # timed output is right (last, so that no other rank waits on it)
        cpu_ms, cores, ref = cpu_reference_loop(3, 1, L, inputs=(prefix_k, prefix_v, noise_t if batch == 1 else noise_t[0]))
        got = torch.from_numpy(out if batch == 1 else out[0]).double().flatten()
        refd = ref.double().flatten()
        rms = float(refd.pow(2).mean().sqrt())
        parity = {"cosine": round(float(got @ refd / (got.norm() * refd.norm())), 6),
                  "max_abs_over_rms": round(float((got - refd).abs().max()) / rms, 4),
                  "rms_err_over_rms": round(float((got - refd).pow(2).mean().sqrt()) / rms, 4),
                  "layers": L, "steps": num_steps,
                  "against": "fp32 torch oracle (oracle.block_ref.denoise_loop) on the same weights, prefix and noise"}
        line = {
            "metric": METRIC, "value": round(ms, 4), "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None,
            "dtype": ("nvfp4_e2m1 (ue4m3 block scales, fp32 accumulate, bf16 residual stream)" if nv
                      else "fp8_e4m3 (fp32 accumulate, bf16 residual stream)"),
            "data": "synthetic",
            "config": {"workload": (WORKLOAD_NVFP4 % batch) if nv else WORKLOAD,
                       "parallelism": f"replicas x{world} (no collective)",
                       "l2": ("working set %d MB per Euler step exceeds the 126 MB L2; no explicit flush"
                              % (loop_bytes // num_steps // 1000000)),
                       "kernels_per_loop": kernels_per_loop, "pdl": use_pdl,
                       "calibration_samples": args.calib_samples,
                       "tensor_core_status": status, "actions_finite": bool((out == out).all())},
            "e2e": {"value": round(e2e_ms, 4), "unit": "ms", "h2d_bytes_per_step": int(noise.nbytes),
                    "d2h_bytes_per_step": int(out.nbytes)},
            "gpu_launches": kernels_per_loop * args.steps,
            "aggregate_loops_per_s": round(world * 1e3 / ms, 2),
            "p50_ms": round(_pctl(per, 0.5), 4), "p95_ms": round(_pctl(per, 0.95), 4),
            "parity": parity,
            "loop_hbm_floor": {"algorithmic_bytes": loop_bytes, "floor_ms": round(loop_bytes / (peak * 1e9) * 1e3, 4),
                               "frac": round(loop_bytes / (peak * 1e9) * 1e3 / ms, 4)},
            "roofline": {"bound": "hbm",
                         "kernel": ("gemm_fp8_kernel<..,true,..,NVFP4> (M=%d weight streaming)" % M if nv else
                                    "gemm_tok_kernel (M=%d projections of the loop: weight streaming)" % M),
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # not measured in this run: dram read + write of one launch from the ncu capture under
                         # profiles/ (1.005 x the algorithmic read bytes; the result stays in L2), scaled by bytes
                         "traffic": int(1.005 * (gemm_bytes - gemm_out_bytes)),
                         "traffic_source": "carried over from the ncu capture in profiles/, scaled by bytes",
                         "peak_source": peak_src,
                         "avg_launch_us": round(gemm_us, 3), "algorithmic_bytes_per_launch": int(gemm_bytes)},
            "cpu_baseline": {"value": round(cpu_ms, 2), "unit": "ms", "cores": cores, "kind": "port",
                             "sample": "3 full 10-step loops of the fp32 torch oracle, median"},
            "clocks": clocks,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def nvfp4_summary(args, local: int) -> dict:
    """configs[3] in short: the NVFP4 loop at batch 1 and batch 4, graph replay only (ms per loop)."""
    import torch
    from flashrt_b200 import load_model
    from flashrt_b200.pi05_decoder import ACTION_DIM
    res = {}
    for batch in (1, 4):
        model = load_model("synthetic:0", config="pi05", device=local, precision="nvfp4", batch=batch)
        fe = model.frontend
        g = torch.Generator().manual_seed(1)
        model.set_prefix(torch.randn(fe.layers, fe.prefix_len, 256, generator=g),
                         torch.randn(fe.layers, fe.prefix_len, 256, generator=g))
        shape = (fe.chunk_size, ACTION_DIM) if batch == 1 else (batch, fe.chunk_size, ACTION_DIM)
        out = model.predict(noise=torch.randn(*shape, generator=g).numpy())
        s = fe.stream
        for _ in range(3):
            fe.forward_decode_only()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(20):
            fe.forward_decode_only()
        e1.record(s)
        s.synchronize()
        res[f"b{batch}_ms"] = round(e0.elapsed_time(e1) / 20, 4)
        res[f"b{batch}_finite"] = bool((out == out).all())
        del model, fe
        torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------------------------------------------
WAN_METRIC = "video-DiT step ms"
WAN_WORKLOAD = ("wan2.2-5B-shape DiT step: 30 blocks, width 3072, 24 heads x 128, FFN 14336 GELU-tanh, adaLN, "
                "cross-attention to 512 text tokens of width 4096, 13x30x52 = 20280 latent tokens, batch 2, "
                "FP8 E4M3 GEMMs + bf16 attention")


def measure_wan(args, rank, world, local, steps, warm):
    """One denoise step of the video DiT, tensor-parallel over the ``world`` ranks of the already initialised process
    group (strong scaling).  Returns the timings (max over ranks) and the roofline inputs on every rank."""
    import torch
    import torch.distributed as dist
    from flashrt_b200.wan_dit import WanDiTB200, synthetic_wan_state
    from flashrt_b200 import flash_rt_kernels as fvk
    layers = args.wan_layers
    state = synthetic_wan_state(0, layers=1)
    grid, B, T = (13, 30, 52), 2, 512
    model = WanDiTB200(state, grid=grid, batch=B, text_len=T, device=local, tp_rank=rank, tp_size=world,
                       repeat_blocks=layers, overlap_chunks=args.wan_overlap_chunks,
                       sequence_parallel=not args.wan_replicated, fast_gelu=not args.wan_exact_gelu)
    L, D = model.L, model.dim
    g = torch.Generator().manual_seed(1)
    x_host = torch.randn(B, L, D, generator=g).to(torch.bfloat16).pin_memory()
    ctx = torch.randn(B, T, 4096, generator=g)
    tproj = torch.randn(B, 6, D, generator=g) * 0.3
    x_dev = x_host.to(f"cuda:{local}")
    model.set_context(ctx)
    model.calibrate(x_dev, tproj)

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
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops_sustained": 1400.0}
    bf16_peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    gemm_flop = 2.0 * B * L * (3072 * 9216 + 3 * 3072 * 3072 + 2 * 3072 * 14336) * layers      # FP8 projections
    attn_flop = 4.0 * L * L * 3072 * B * layers + 4.0 * L * T * 3072 * B * layers              # bf16 attention
    # time-weighted floor per GPU: the FP8 part against 2 x the measured bf16 rate, the attention against 1 x
    floor_ms = (gemm_flop / (2 * bf16_peak) + attn_flop / bf16_peak) / world / 1e12 * 1e3
    res = {"ms": round(ms, 2), "e2e_ms": round(e2e_ms, 2), "layers": layers, "clocks": clocks,
           "finite": bool(torch.isfinite(out.float()).all()), "status": fvk.tensor_core_status(),
           "launches": model.launches_per_step, "gemm_flop": gemm_flop, "attn_flop": attn_flop,
           "bf16_peak": bf16_peak, "floor_ms": round(floor_ms, 2), "frac_weighted": round(floor_ms / ms, 4),
           "h2d": int(x_host.numel() * 2), "d2h": int(out_host.numel() * 2), "steps": steps, "warm": warm}
    del model
    torch.cuda.empty_cache()
    return res


def wan_cpu_baseline(tokens: int = 512, text: int = 128):
    """One block of the fp32 torch restatement of the video-DiT block (oracle.wan_ref.block) on the host cores at a
    reduced token count, scaled to the 30-block step at 2 x 20280 tokens by FLOPs (projections linear, attention
    quadratic in the tokens): an extrapolation, flagged as such."""
    import torch
    from oracle import wan_ref
    from flashrt_b200.wan_dit import synthetic_wan_state
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    st = synthetic_wan_state(0, layers=1)
    bw = st["blocks"][0]
    D, hd, B = 3072, 128, 2
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, tokens, D, generator=g)
    ctx = torch.randn(B, text, 4096, generator=g)
    tp = torch.randn(B, 6, D, generator=g) * 0.3
    cos, sin = (torch.ones(tokens, hd // 2), torch.zeros(tokens, hd // 2))
    t0 = time.perf_counter()
    wan_ref.block(x, bw, tp, ctx, cos, sin, hd)
    sec = time.perf_counter() - t0
    Lf, Tf = 20280, 512
    small = 2.0 * B * tokens * (3072 * 9216 + 3 * 3072 * 3072 + 2 * 3072 * 14336) + 4.0 * tokens * tokens * 3072 * B \
        + 4.0 * tokens * text * 3072 * B
    full = 2.0 * B * Lf * (3072 * 9216 + 3 * 3072 * 3072 + 2 * 3072 * 14336) + 4.0 * Lf * Lf * 3072 * B \
        + 4.0 * Lf * Tf * 3072 * B
    return {"value": round(sec * full / small * 30 * 1e3, 1), "unit": "ms", "cores": cores, "kind": "port",
            "sample": (f"one block of the fp32 torch restatement at {tokens} latent + {text} text tokens "
                       f"({sec:.2f} s), EXTRAPOLATED by FLOPs to 30 blocks at 20280 + 512 tokens")}


def run_wan(args):
    """Benchmark configuration 4: one denoise step of the video DiT, tensor-parallel over the N GPUs (strong scaling)."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))
    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    w = measure_wan(args, rank, world, local, steps, warm)
    if rank == 0:
        try:
            cpu = wan_cpu_baseline()
        except Exception as e:  # noqa: BLE001
            cpu = {"error": f"{type(e).__name__}: {e}"[:200]}
        achieved = (w["gemm_flop"] + w["attn_flop"]) / world / (w["ms"] * 1e-3) / 1e12
        line = {
            "metric": WAN_METRIC, "value": w["ms"], "unit": "ms", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": w["ms"], "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3 GEMMs (fp32 accumulate), bf16 attention", "data": "synthetic",
            "config": {"workload": WAN_WORKLOAD, "layers": w["layers"], "parallelism": f"tp{world} (heads + FFN columns; " + (
                           "replicated residual stream, NCCL all-reduce after attention-out, cross-attention-out and "
                           "FFN-down)" if args.wan_replicated or world == 1 else
                           "sequence-parallel residual stream: NCCL all-gather of the FP8 operand in front of QKV / "
                           "cross-Q / FFN-up, reduce-scatter after attention-out, cross-attention-out and FFN-down)"),
                       "l2": "activations of one step (> 1 GB) exceed the 126 MB L2; no explicit flush",
                       "tensor_core_status": w["status"], "finite": w["finite"]},
            "e2e": {"value": w["e2e_ms"], "unit": "ms", "h2d_bytes_per_step": w["h2d"], "d2h_bytes_per_step": w["d2h"]},
            "gpu_launches": w["launches"] * steps,
            "roofline": {"bound": "tensor", "kernel": "whole step (FP8 GEMMs + bf16 attention), per GPU",
                         # time-weighted: FP8 FLOPs against 2 x the measured bf16 rate, attention FLOPs against 1 x
                         "achieved": round(achieved, 1), "peak": round((w["gemm_flop"] + w["attn_flop"]) / world /
                                                                       (w["floor_ms"] * 1e-3) / 1e12, 1),
                         "unit": "TFLOP/s", "frac": w["frac_weighted"], "traffic": None,
                         "peak_source": ("time-weighted from MEASURED_PEAKS.json bf16_tflops_sustained: FP8 projections "
                                         "at 2 x, bf16 attention at 1 x"),
                         "floor_ms": w["floor_ms"], "flop_per_step": w["gemm_flop"] + w["attn_flop"]},
            "cpu_baseline": cpu, "clocks": w["clocks"],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
def ops_table(args, quick: bool):
    """Operator sweep (benchmark configuration 1) on one GPU: fused residual + RMSNorm + FP8 quantise over row widths,
    FP8 and NVFP4 GEMMs over M x (N, K).  Every case is timed as a CUDA graph of launches that cycle through
    enough distinct buffers to exceed L2, with CUDA events around the replays.  ``quick``: the norm rows and the FP8
    GEMMs with M >= 2048 only.  The FP8 GEMMs with M >= 2048 carry a LIBRARY column beside them: the same product
    through ``torch._scaled_mm`` (cuBLASLt FP8, per-tensor scales) on the same tensors -- the stated baseline, since
    the reference's own sm_100 CUTLASS kernels cannot be built here; never on the hot path.
    Returns (table, launches, peaks)."""
    import torch
    from flashrt_b200 import _lib
    from flashrt_b200 import flash_rt_fp4 as fp4
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

    def timed(enqueue, n_launch, reps=5, count=True):
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
        if count:
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
    for kind in (("fp8",) if quick else ("fp8", "nvfp4")):
        for M in ((2048, 8192, 20480) if quick else (16, 50, 256, 2048, 8192, 20480)):
            for N, K in NK:
                eb = 1.0 if kind == "fp8" else 0.5
                wbytes = N * K * eb
                nbuf = max(1, min(160, int(L2 // wbytes) + 1)) if M <= 256 else 2
                A = torch.randint(0, 256, (M, int(K * eb)), dtype=torch.uint8, device="cuda")
                Ws = [torch.randint(0, 120, (N, int(K * eb)), dtype=torch.uint8, device="cuda") for _ in range(nbuf)]
                D = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
                lib_us = None
                if kind == "fp8":
                    A &= 0x77                      # finite E4M3 codes
                    def enq():
                        for w in Ws:
                            _lib.call("frt_b200_gemm_fp8_nt", A.data_ptr(), w.data_ptr(), D.data_ptr(), M, N, K,
                                      one.data_ptr(), one.data_ptr(), 1.0, None, 0, gemm_flags if M > 256 else 0,
                                      s.cuda_stream)
                    if M >= 2048:
                        a8 = A.view(torch.float8_e4m3fn)
                        w8 = [w.view(torch.float8_e4m3fn).t() for w in Ws]
                        def enq_lib():
                            for w in w8:
                                torch._scaled_mm(a8, w, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                        try:
                            lib_us = timed(enq_lib, nbuf, reps=3, count=False) * 1e6
                        except Exception:  # noqa: BLE001
                            lib_us = None
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
                row = {"op": "gemm_" + kind, "M": M, "N": N, "K": K, "us": round(t * 1e6, 2),
                       "TFLOP/s": round(tf, 1),
                       "frac_tensor": round(tf / (fp8_peak if kind == "fp8" else fp4_peak), 3),
                       "frac_datasheet": round(tf / (4500.0 if kind == "fp8" else 9000.0), 3),
                       "GB/s": round(gbs, 1), "frac_hbm": round(gbs / peak_hbm, 3)}
                if lib_us is not None:
                    row["cublaslt_us"] = round(lib_us, 2)
                    row["vs_cublaslt"] = round(lib_us / (t * 1e6), 3)      # > 1: this library is faster
                table.append(row)
                del A, Ws, D
    # ---- long-sequence bidirectional attention (the video-DiT shape) beside torch's fused SDPA, full sweep only
    if not quick:
        from flashrt_b200 import flash_rt_fa2 as fa2
        B, Sq, H, Dh = 2, 20280, 24, 128
        q = torch.randn(B, Sq, H, Dh, device="cuda").bfloat16()
        k, v, o = torch.randn_like(q), torch.randn_like(q), torch.empty_like(q)
        st3 = (Sq * H * Dh, H * Dh, Dh)
        def enq_a():
            fa2.fwd_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 0, 0, 0, B, Sq, Sq, H, H, Dh, st3, st3,
                         st3, st3, Dh ** -0.5, 148, s.cuda_stream)
        t = timed(enq_a, 1, reps=3)
        qt, kt, vt = (z.transpose(1, 2) for z in (q, k, v))
        def enq_s():
            torch.nn.functional.scaled_dot_product_attention(qt, kt, vt)
        try:
            tl = timed(enq_s, 1, reps=3, count=False)
        except Exception:  # noqa: BLE001
            tl = None
        fl = 4.0 * B * H * Sq * Sq * Dh
        row = {"op": "attention_bf16", "B": B, "S": Sq, "H": H, "D": Dh, "us": round(t * 1e6, 1),
               "TFLOP/s": round(fl / t / 1e12, 1), "frac_tensor": round(fl / t / 1e12 / bf16_tf, 3)}
        if tl:
            row["torch_sdpa_us"] = round(tl * 1e6, 1)
            row["vs_torch_sdpa"] = round(tl / t, 3)
        table.append(row)
    return table, launches, {"hbm_gbs": peak_hbm, "fp8_tflops": fp8_peak, "nvfp4_tflops": fp4_peak,
                             "fp8_datasheet_tflops": 4500.0,
                             "note": "tensor peaks = 2x / 4x the measured cuBLAS bf16 burst; the 4.5 PF dense "
                                     "FP8 datasheet figure beside it"}


def ops_summary(args) -> dict:
    """configs[1] in short for the default line: worst norm fraction of HBM peak, the FP8 GEMM fractions at M >= 2048
    (of 2 x the measured bf16 burst), how many of the 18 reach 0.60, and the ratio to cuBLASLt per shape."""
    table, _, _ = ops_table(args, quick=True)
    norm = [r for r in table if r["op"] == "residual_add_rms_norm_fp8"]
    big = [r for r in table if r["op"] == "gemm_fp8"]
    key = lambda r: f"{r['M']}x{r['N']}x{r['K']}"  # noqa: E731
    return {"norm_frac_min": min(r["frac_hbm"] for r in norm),
            "gemm_fp8_frac": {key(r): r["frac_tensor"] for r in big},
            "n_at_target": sum(1 for r in big if r["frac_tensor"] >= 0.60), "n_shapes": len(big),
            "vs_cublaslt": {key(r): r.get("vs_cublaslt") for r in big}}


def run_ops(args):
    import torch
    torch.cuda.set_device(0)
    table, launches, peaks = ops_table(args, quick=False)
    from flashrt_b200 import flash_rt_kernels as fvk
    big = [r for r in table if r["op"] == "gemm_fp8" and r["M"] >= 2048]
    line = {"metric": "operator sweep (configs[1])", "value": round(statistics.mean(r["frac_tensor"] for r in big), 4),
            "unit": "mean fraction of 2 x measured bf16 peak over the FP8 GEMMs with M >= 2048", "n_gpus": 1,
            "steps": 1, "warmup": 3, "higher_is_better": True, "data": "synthetic", "dtype": "fp8_e4m3 / nvfp4 / bf16",
            "config": {"workload": "configs[1] operator sweep", "peaks": peaks,
                       "l2": ("norm and M <= 256 GEMM cases cycle through distinct row / weight buffers totalling more than "
                              "L2; M >= 2048 GEMM cases alternate two weight buffers (tensor-bound)"),
                       "large_m_fp8_kernel": ("cta pair (256 x 256 tiles) forced" if args.cta_pair else
                                              "library's choice: cta pair for >= 2 waves of 256 x 256 tiles at "
                                              "K >= 2048, else persistent one-CTA tiles"),
                       "library_baseline": "torch._scaled_mm (cuBLASLt FP8) and torch SDPA on the same tensors",
                       "tensor_core_status": fvk.tensor_core_status(), "table": table},
            "gpu_launches": launches}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
def run_timeline(args):
    """Per-hop timeline of the operator graph (diagnostic; needs a library built with -DFRT_PHASE_STAMPS): two decoder
    blocks (QKV, attention, attention-out, gate|up, FFN-down -- the loop's own calls) captured as one graph; every CTA
    stamps %globaltimer at its phases, and the medians over the CTAs of a launch are printed on a common clock."""
    import ctypes
    import numpy as np
    import torch
    from flashrt_b200 import _lib, load_model
    from flashrt_b200.pi05_decoder import ACTION_DIM
    torch.cuda.set_device(0)
    model = load_model("synthetic:0", config="pi05", device=0)
    fe = model.frontend
    p, L = fe.pipeline, fe.layers
    g = torch.Generator().manual_seed(1)
    model.set_prefix(torch.randn(L, fe.prefix_len, 256, generator=g), torch.randn(L, fe.prefix_len, 256, generator=g))
    model.calibrate([torch.randn(fe.chunk_size, ACTION_DIM, generator=g)])
    gb = (ctypes.c_ulonglong * (8 * 160 * 16))()
    ab = (ctypes.c_ulonglong * (8 * 128 * 16))()

    def read(reset=1):
        rc = _lib.call_status("frt_b200_phase_stamps_read", ctypes.addressof(gb), ctypes.addressof(ab), reset)
        if rc != 0:
            raise SystemExit("timeline: the library was built without -DFRT_PHASE_STAMPS "
                             "(FRT_NVCC_EXTRA=-DFRT_PHASE_STAMPS python -m flashrt_b200._build --force)")
        return (np.frombuffer(gb, dtype=np.uint64).reshape(8, 160, 16).astype(np.int64),
                np.frombuffer(ab, dtype=np.uint64).reshape(8, 128, 16).astype(np.int64))

    s = fe.stream
    calls = {"n": 0}
    orig = p._folded_layers

    def two_blocks(step, stream, pdl):
        fe.layers = 2
        try:
            orig(step, stream, pdl)
        finally:
            fe.layers = L

    with torch.cuda.stream(s):
        p.noise.normal_()
        p._step_in(s.cuda_stream, True)
        p._norm(None, None, "attn", 0, 0, "qkv", s.cuda_stream, True, False)
        two_blocks(0, s.cuda_stream, True)
        s.synchronize()
        read()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s, capture_error_mode="relaxed"):
            two_blocks(0, s.cuda_stream, True)
        for _ in range(3):
            gr.replay()
        s.synchronize()
    tt, ta = read(0)
    kinds = ["qkv (layer 0)", "attention", "attention-out", "gate|up", "FFN-down",
             "qkv", "attention", "attention-out", "gate|up", "FFN-down"]
    rows, gi, ai = [], 0, 0
    for k in kinds:
        if k == "attention":
            a = ta[ai % 8]
            ai += 1
            a = a[a[:, 0] > 0]
            pub = 9 if (a[:, 9] > 0).all() else 8      # cluster exchange: no fence + barrier stamp, "pushed" instead
            cols = (a[:, 0].min(), np.median(a[:, 1]), np.median(a[:, 7]), np.median(a[:, pub]), np.median(a[:, 10]),
                    a[:, 12].max())
        else:
            a = tt[gi % 8]
            gi += 1
            a = a[a[:, 0] > 0]
            cols = (a[:, 0].min(), np.median(a[:, 3]), np.median(a[:, 4]), np.median(a[:, 6]), np.median(a[:, 7]),
                    a[:, 9].max())
        rows.append({"kernel": k, "ctas": int(len(a)), "ns": [float(v) for v in cols]})
    t0 = rows[0]["ns"][0]
    for r in rows:
        r["us"] = [round((v - t0) / 1e3, 2) for v in r.pop("ns")]
    hdr = ("kernel                     CTAs  first CTA start | dependency wait returned (GEMM: + operand produced) | "
           "accumulator complete | GEMM: slots received / attention: partial published | GEMM: finish done / "
           "attention: all splits arrived | last CTA end   [us, common clock, medians over the CTAs]")
    print(hdr, file=sys.stderr)
    for r in rows:
        print(f"{r['kernel']:26s} {r['ctas']:4d}  " + "  ".join(f"{v:8.2f}" for v in r["us"]), file=sys.stderr)
    # the last attention launch per kv split: medians over the CTAs of a split (4 row tiles x 4 head-dim parts), us since
    # the launch's first CTA.  Stamps: dependency wait returned, first Q block landed, first S complete, first P written,
    # P.V complete, partial in registers, partial stored, fenced + CTA barrier, all CTAs of the tile seen, combined, end.
    a = ta[(ai - 1) % 8]
    splits, cols = [], (1, 2, 4, 5, 7, 13, 14, 9, 10, 11, 12)
    n_cta = int((a[:, 0] > 0).sum())
    if n_cta in (112, 128) and not (a[:n_cta, 9] > 0).any():
        # cluster exchange (no scratch): CTA (x, z) is row z * gx + x.  Ragged launch (gx = 14): x 0 and 1 are the two
        # parts of the short last tile.  Stamps: dependency wait returned, first Q block landed, first S complete, first
        # P written, P.V complete, partial packed in registers, pushed to the peers, all peers' slices received,
        # combined + stored, end.
        gx, a, a0 = n_cta // 8, a[:n_cta], a[:n_cta, 0].min()
        xs = np.arange(n_cta) % gx
        groups = ([("last tile, 2 parts", xs < 2), ("full tiles, 4 parts", xs >= 2)] if gx % 4 == 2
                  else [("all", xs >= 0)])
        for z in (0, 1, 7):
            groups.append((f"kv split {z}", np.arange(n_cta) // gx == z))
        groups.append(("slowest", None))
        print("attention launch (us): wait returned | Q block | first S | first P | P.V done | packed | pushed | "
              "received | combined | end", file=sys.stderr)
        for name, m in groups:
            blk = a if m is None else a[m]
            f = np.max if m is None else np.median
            us = [round(float(f(blk[:, c]) - a0) / 1e3, 2) for c in (1, 2, 4, 5, 7, 13, 14, 10, 11, 12)]
            splits.append({"ctas": name, "us": us})
            print(f"  {name:20s} " + "  ".join(f"{v:6.2f}" for v in us), file=sys.stderr)
    elif n_cta == 128:
        a0 = a[:, 0].min()
        print("attention launch per kv split (us): wait returned | Q block | first S | first P | P.V done | in registers | "
              "stored | fenced | all seen | combined | end", file=sys.stderr)
        for z in list(range(8)) + ["slowest"]:
            blk = a if z == "slowest" else a[z * 16:(z + 1) * 16]
            f = np.max if z == "slowest" else np.median
            us = [round(float(f(blk[:, c]) - a0) / 1e3, 2) for c in cols]
            splits.append({"split": z, "us": us})
            print(f"  split {z!s:8s} " + "  ".join(f"{v:6.2f}" for v in us), file=sys.stderr)
    print(json.dumps({"metric": "operator-graph phase timeline (diagnostic)", "unit": "us", "rows": rows,
                      "block_us": rows[-1]["us"][-1] - rows[4]["us"][-1], "attention_splits": splits}), flush=True)


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
    ap.add_argument("--no-extras", action="store_true",
                    help="pi05 workload: skip the short runs of the other configurations (video-DiT step, operator "
                         "sweep, NVFP4 loop) that the default line carries as extra keys")
    ap.add_argument("--extras-budget-s", type=float, default=150.0,
                    help="an extra is started only while the whole run has taken less than this many seconds")
    ap.add_argument("--lean", action="store_true",
                    help="skip the CPU baseline and the GEMM roofline leg (for short runs under a profiler)")
    ap.add_argument("--workload", default="pi05", choices=["pi05", "wan", "ops", "prefix", "timeline"],
                    help="pi05 = the headline action-expert loop (default); wan = the video-DiT step (configs[4]); "
                         "ops = the operator sweep of configs[1] (norm / FP8 GEMM / NVFP4 GEMM)")
    ap.add_argument("--precision", default="fp8", choices=["fp8", "nvfp4"],
                    help="pi05 workload: fp8 = configs[2] (default, the headline), nvfp4 = configs[3]")
    ap.add_argument("--batch", type=int, default=1, help="pi05 workload with --precision nvfp4: chunks per loop (1 or 4)")
    ap.add_argument("--wan-layers", type=int, default=30)
    ap.add_argument("--wan-exact-gelu", action="store_true",
                    help="wan workload: the exactly rounded GELU in the fused FFN-up epilogue instead of the hardware tanh")
    ap.add_argument("--wan-replicated", action="store_true",
                    help="wan workload under TP: replicated residual stream with an all-reduce per row-parallel "
                         "projection instead of the sequence-parallel stream (all-gather / reduce-scatter)")
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
    if args.workload == "timeline" and args.impl != "reference":
        run_timeline(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
