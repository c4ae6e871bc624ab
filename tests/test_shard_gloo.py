"""The N > 1 path on CPU: two gloo ranks each take their shard of a workload,
compute it with the oracle, and the gathered result equals the unsharded one.
Also covers the max-over-ranks timing reduction bench.py uses."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lego_b200 import shard


def test_split_range_covers_everything_once():
    for n, world, align in [(16384, 8, 1), (4096, 8, 32), (1000, 3, 128), (5, 8, 1), (0, 4, 1), (8192, 8, 128)]:
        seen = []
        for r in range(world):
            b, e = shard.split_range(n, r, world, align)
            assert b <= e and (b % align == 0)
            seen += list(range(b, e))
        assert seen == list(range(n)), (n, world, align)
    with pytest.raises(ValueError):
        shard.split_range(10, 4, 4)


def test_grouped_gemm_shards_balance_ragged_groups():
    mnk = [(2048, 1024, 4096), (1024, 4096, 4096), (4096, 4096, 4096)]
    loads = []
    for r in range(8):
        blocks = shard.shard_grouped_gemm(mnk, r, 8)
        loads.append(sum((e - b) * n for (b, e), (_m, n, _k) in zip(blocks, mnk)))
    assert max(loads) == min(loads)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from oracle import lego_oracle as O
        g = torch.Generator().manual_seed(1)
        x = (torch.randn(64, 256, generator=g) * 2).half()          # every rank builds the same input
        b, e = shard.shard_rows(64, rank, world)
        mine = O.softmax(x[b:e]).float()
        parts = [torch.empty(shard.shard_rows(64, r, world)[1] - shard.shard_rows(64, r, world)[0], 256)
                 for r in range(world)]
        dist.all_gather(parts, mine)
        full = torch.cat(parts)
        ok = torch.equal(full, O.softmax(x).float())
        # GEMM split by M: B replicated, C row blocks concatenated
        a = torch.randn(256, 64, generator=g).half()
        bm = torch.randn(64, 128, generator=g).half()
        mb, me = shard.shard_gemm_m(256, rank, world)
        c_parts = [torch.empty(shard.shard_gemm_m(256, r, world)[1] - shard.shard_gemm_m(256, r, world)[0], 128)
                   for r in range(world)]
        dist.all_gather(c_parts, O.matmul(a[mb:me], bm))
        ok = ok and torch.allclose(torch.cat(c_parts), O.matmul(a, bm), atol=1e-5)
        # timing reduction: the slowest rank decides
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok = ok and t.item() == float(world)
        dist.barrier()
        if rank == 0:
            out.put(bool(ok))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=10) is True
