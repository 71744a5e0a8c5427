"""Multi-rank host logic on CPU: two gloo ranks.  Sequence assignment, the max-over-ranks
timing reduction, and the column-sharded mm8 (each rank multiplies its column slice of a
packed matrix with the oracle's arithmetic, slices are all-gathered) against the unsharded
result."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from chatrwkv_b200 import shard
        from oracle import rwkv_oracle as orc
        ok = True
        # sequences: a partition of range(n)
        mine = shard.assign_sequences(11, world, rank)
        counts = torch.zeros(11, dtype=torch.int64)
        counts[mine] = 1
        dist.all_reduce(counts)
        ok &= bool((counts == 1).all())
        # timing: max over ranks
        t = shard.max_over_ranks([1.0 + rank, 5.0 - rank])
        ok &= t == [float(world), 5.0]
        # column-sharded mm8 == unsharded mm8, for an M that does not divide evenly
        g = torch.Generator().manual_seed(7)
        for (N, M) in ((64, 300), (48, 50)):
            w = torch.randn(N, M, generator=g) * 0.02
            q, mx, rx, my, ry = orc.quantize_weight(w, torch.float32)
            x1 = torch.randn(N, generator=g)
            xs = torch.randn(5, N, generator=g)
            ql, mxl, rxl = shard.column_shard(q, mx, rx, world, rank)
            mw = shard.shard_width(M, world)
            for x in (x1, xs):
                full = orc.mm8_kernel(x, q, mx, rx, my, ry)
                loc = torch.zeros(x.shape[:-1] + (mw,))
                if ql.shape[1] > 0:
                    loc[..., :ql.shape[1]] = orc.mm8_kernel(x, ql, mxl, rxl, my, ry)
                got = shard.gather_columns(loc, M, world)
                ok &= got.shape == full.shape and torch.allclose(got, full, rtol=1e-6, atol=1e-6)
        lo, hi = shard.column_range(50277, world, rank)
        ok &= (hi - lo) > 0 and lo % 16 == 0
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_rank_host_logic_gloo():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_geometry():
    from chatrwkv_b200 import shard
    for M, world in ((50277, 8), (5120, 4), (20480, 2), (300, 8), (16, 8)):
        ranges = [shard.column_range(M, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and max(hi for _, hi in ranges) == M
        for (lo0, hi0), (lo1, hi1) in zip(ranges, ranges[1:]):
            assert hi0 == lo1 or (hi0 == M and lo1 == M)
        assert shard.shard_width(M, world) % 16 == 0
