"""CPU suite (gloo, world size 2): the host-side tensor-parallel logic of the video-DiT path — weight sharding,
the all-reduce of row-parallel partial products and of the per-row sums of squares for the full-width q/k RMSNorm,
and the sequence-parallel form (interleaved row ownership, all-gather in front of a column-parallel layer,
reduce-scatter behind a row-parallel one) — reproduces the unsharded arithmetic."""
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
    # sequence-parallel residual stream: interleaved row ownership (block c * world + r of Mb rows belongs to rank r),
    # all-gather of piece c in front of a column-parallel layer, reduce-scatter of piece c behind a row-parallel one
    C, Mb = 2, M // (world * 2)
    xl = torch.stack([x[(c * world + rank) * Mb:(c * world + rank + 1) * Mb] for c in range(C)])      # (C, Mb, D)
    out_l = torch.empty(C, Mb, D)
    for c in range(C):
        piece = torch.empty(world * Mb, D)
        dist.all_gather_into_tensor(piece, xl[c].contiguous())
        ok_piece = torch.equal(piece, x[c * world * Mb:(c + 1) * world * Mb])
        part = torch.nn.functional.gelu(piece @ shard_rows(w1, rank, world).t(), approximate="tanh") \
            @ shard_cols(w2, rank, world).t()
        dist.reduce_scatter_tensor(out_l[c], part)
        ok1 = ok1 and ok_piece
    mine = torch.stack([ref[(c * world + rank) * Mb:(c * world + rank + 1) * Mb] for c in range(C)])
    ok3 = torch.allclose(out_l, mine, atol=1e-4)
    ret[rank] = bool(ok1 and ok2 and ok3)
    dist.destroy_process_group()


def test_tensor_parallel_host_logic_world_size_2():
    world = 2
    port = 29500 + (os.getpid() % 1000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world))


def test_sequence_parallel_row_ownership():
    """Host logic of the sequence-parallel stream: every row is owned exactly once, a block never straddles a batch
    element, a piece is one contiguous range on every rank, and the shapes of the benchmark pick the expected layout."""
    from flashrt_b200.wan_dit import sp_block_rows, sp_layout
    L = 13 * 30 * 52
    assert sp_layout(2 * L, L, 2, 4) == (4, 2 * L // 8)
    assert sp_layout(2 * L, L, 4, 4) == (4, 2 * L // 16)
    assert sp_layout(2 * L, L, 8, 4) == (2, 2 * L // 16)         # 40 560 rows divide by 16, not by 32
    assert sp_layout(2 * 384, 384, 2, 4) == (4, 96)
    assert sp_layout(2 * 384, 384, 2, 2) == (2, 192)
    assert sp_layout(2 * 385, 385, 4, 4) is None                  # rows that do not divide: replicated stream
    for rows, per_batch, tp, want in ((2 * L, L, 8, 4), (2 * L, L, 4, 4), (768, 384, 2, 4), (768, 384, 2, 1)):
        C, mb = sp_layout(rows, per_batch, tp, want)
        seen = [0] * rows
        for c in range(C):
            piece_first = c * tp * mb
            for r in range(tp):
                a, b = sp_block_rows(c, r, tp, mb)
                assert a == piece_first + r * mb and b - a == mb          # rank order inside the contiguous piece
                assert a // per_batch == (b - 1) // per_batch              # one batch element per block
                for i in range(a, b):
                    seen[i] += 1
        assert all(v == 1 for v in seen)
