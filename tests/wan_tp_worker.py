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
    m = WanDiTB200(state, grid=grid, batch=B, text_len=T, device=local, tp_rank=rank, tp_size=world)
    m.set_context(ctx)
    m.calibrate(x, tproj)
    got = m.step(x, tproj).float().cpu()
    ok = True
    if rank == 0:
        ref = wan_ref.step(x, state, tproj, ctx, cos, sin)
        rms = float(ref.pow(2).mean().sqrt())
        err = (got - ref).abs()
        cosv = float((got.double().flatten() @ ref.double().flatten()) / (got.double().norm() * ref.double().norm()))
        print(f"TP={world} cos={cosv:.6f} err_rms={float(err.pow(2).mean().sqrt()):.5f} max={float(err.max()):.4f}",
              flush=True)
        ok = cosv >= 0.999 and float(err.pow(2).mean().sqrt()) <= 1e-2 * rms and float(err.max()) <= 0.1 * rms
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
