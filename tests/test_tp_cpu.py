"""CPU suite (gloo, world size 2): the host-side tensor-parallel logic of the video-DiT path — weight sharding,
the all-reduce of row-parallel partial products and of the per-row sums of squares for the full-width q/k RMSNorm —
reproduces the unsharded arithmetic."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flashrt_b200.wan_dit import shard_cols, shard_rows
    g = torch.Generator().manual_seed(0)
    M, D, F = 12, 64, 96
    x = torch.randn(M, D, generator=g)
    w1, w2 = torch.randn(F, D, generator=g), torch.randn(D, F, generator=g)
    wq, nq = torch.randn(D, D, generator=g), torch.rand(D, generator=g) + 0.5
    # column-parallel then row-parallel: partial products summed by all-reduce
    h = torch.nn.functional.gelu(x @ shard_rows(w1, rank, world).t(), approximate="tanh")
    y = h @ shard_cols(w2, rank, world).t()
    dist.all_reduce(y)
    ref = torch.nn.functional.gelu(x @ w1.t(), approximate="tanh") @ w2.t()
    ok1 = torch.allclose(y, ref, atol=1e-4)
    # full-width RMSNorm of a column-sharded projection: local sum of squares + all-reduce of one float per row
    q_loc = x @ shard_rows(wq, rank, world).t()
    ssq = q_loc.pow(2).sum(-1)
    dist.all_reduce(ssq)
    qn_loc = q_loc * torch.rsqrt(ssq[:, None] / D + 1e-6) * shard_rows(nq, rank, world)
    q = x @ wq.t()
    qn = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6) * nq
    n = D // world
    ok2 = torch.allclose(qn_loc, qn[:, rank * n:(rank + 1) * n], atol=1e-5)
    ret[rank] = bool(ok1 and ok2)
    dist.destroy_process_group()


def test_tensor_parallel_host_logic_world_size_2():
    world = 2
    port = 29500 + (os.getpid() % 1000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world))
