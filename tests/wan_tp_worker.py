"""Worker of the tensor-parallel video-DiT GPU test (launched with torch.distributed.run, one rank per GPU):
runs the reduced Wan-shape step at TP = world size and checks rank 0's result against the fp32 restatement."""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main():
    from test_f_wan_dit_gpu import _setup
    from flashrt_b200.wan_dit import WanDiTB200
    from oracle import wan_ref
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    state, grid, B, T, x, ctx, tproj, cos, sin = _setup()
    # exact GELU everywhere: pieces of 192 rows run GEMM -> bias_gelu_quantize, whole tensors the fused epilogue
    m = WanDiTB200(state, grid=grid, batch=B, text_len=T, device=local, tp_rank=rank, tp_size=world, fast_gelu=False)
    m.set_context(ctx)
    m.calibrate(x, tproj)
    assert m.sp and m.C >= 2, "the reduced shape must exercise the sequence-parallel pieces"
    got = m.step(x, tproj).float().cpu()                 # sequence-parallel residual stream (the default)
    again = m.step(x, tproj).float().cpu()
    ok = bool(torch.equal(got, again))
    if not ok:
        print(f"rank {rank}: two sequence-parallel steps differ", flush=True)
    # two pieces (whole batch elements) with the attention launched per piece: same arithmetic, other launch shapes
    m2 = WanDiTB200(state, grid=grid, batch=B, text_len=T, device=local, tp_rank=rank, tp_size=world, overlap_chunks=2,
                    split_attention=True, fast_gelu=False)
    m2.set_context(ctx)
    m2.scales.copy_(m.scales)
    m2.calibrated = True
    got2 = m2.step(x, tproj).float().cpu()
    assert m2.sp and m2.C == 2
    d2 = float((got2 - got).abs().max() / got.pow(2).mean().sqrt())
    if d2 > 0.1:
        ok = False
        print(f"rank {rank}: per-piece attention differs from the whole launch: {d2:.4f} x RMS", flush=True)
    del m2
    # replicated residual stream with an all-reduce per row-parallel projection: the chunked form (all-reduce of one
    # row piece overlapping the GEMM of the next, on a side stream) must give the same bytes as GEMM -> all-reduce
    m.sp = False
    m.overlap_chunks = 3
    m._min_chunk_rows = 128
    got_chunked = m.step(x, tproj).float().cpu()
    m.overlap_chunks = 1
    got_plain = m.step(x, tproj).float().cpu()
    if not torch.equal(got_chunked, got_plain):
        ok = False
        print(f"rank {rank}: chunked all-reduce differs from the plain one", flush=True)
    # both forms compute the same sums, but a piece of 192 rows runs through the small-M GEMM kernels (split-K: another
    # fp32 summation order), so single bf16 results -- and FP8 codes behind them -- differ in the last place
    rms_plain = got_plain.pow(2).mean().sqrt()
    d_max = float((got - got_plain).abs().max() / rms_plain)
    d_rms = float((got - got_plain).pow(2).mean().sqrt() / rms_plain)
    if rank == 0:
        print(f"sequence-parallel vs replicated: rms {d_rms:.5f} max {d_max:.4f} (x RMS)", flush=True)
    if d_rms > 1e-2 or d_max > 0.1:
        ok = False
    if rank == 0:
        ref = wan_ref.step(x, state, tproj, ctx, cos, sin)
        rms = float(ref.pow(2).mean().sqrt())
        err = (got - ref).abs()
        cosv = float((got.double().flatten() @ ref.double().flatten()) / (got.double().norm() * ref.double().norm()))
        print(f"TP={world} cos={cosv:.6f} err_rms={float(err.pow(2).mean().sqrt()):.5f} max={float(err.max()):.4f}",
              flush=True)
        ok = ok and cosv >= 0.999 and float(err.pow(2).mean().sqrt()) <= 1e-2 * rms and float(err.max()) <= 0.1 * rms
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
