"""bench.py's multi-GPU bookkeeping on the CPU: the way each workload's shards are laid
end to end, gathered and handed to its parity check.  The shards here come from the oracle
(no GPU), cut exactly as the ranks cut them; a wrong offset in the assembly arithmetic
fails the check just as a wrong kernel would."""
import importlib.util
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
sys.modules["bench"] = bench
spec.loader.exec_module(bench)

from lego_b200 import shard  # noqa: E402
from oracle import lego_oracle as O  # noqa: E402


class _NoOps:
    @staticmethod
    def device_status():
        return 0


def test_grouped_gemm_shards_assemble_for_the_check():
    world = 4
    w = bench.GroupedGemm()
    w.groups, w.k = 5, 64
    bench._cpu_setup(w)
    w.world, w.ops = world, _NoOps
    w.packing = shard.pack_grouped_gemm_blocks(w.sizes, world, 512)
    w.slot = max(sum((e - b) * w.sizes[g][1] for g, b, e in p) for p in w.packing)
    per_rank = []
    for rank in range(world):
        cs = [(w.A_host[g][b:e].float() @ w.B_host[g].float()).half().reshape(-1) for g, b, e in w.packing[rank]]
        slot = torch.zeros(w.slot, dtype=torch.float16)
        flat = torch.cat(cs)
        slot[:flat.numel()] = flat
        per_rank.append(slot)
    ok, text = w.check(torch.cat(per_rank))
    assert ok, text
    per_rank[1][:] = 0                                        # one rank's result lost: must be noticed
    ok, _ = w.check(torch.cat(per_rank))
    assert not ok


def test_grouped_gemm_blocks_pack_evenly():
    from lego_b200 import configs
    sizes, _ = configs.grouped_sizes()
    for world in (2, 4, 8):
        packing = shard.pack_grouped_gemm_blocks(sizes, world, 512)
        seen = sorted((g, b, e) for p in packing for g, b, e in p)
        assert seen == sorted((g, b, min(m, b + 512)) for g, (m, _n, _k) in enumerate(sizes) for b in range(0, m, 512))
        loads = [sum((e - b) * sizes[g][1] for g, b, e in p) for p in packing]
        assert max(loads) <= 1.03 * sum(loads) / world, (world, loads)


def test_layernorm_backward_partial_column_sums_assemble():
    world = 2
    w = bench.LayerNormBwd()
    w.rows, w.cols = 514 * 2, 1024
    bench._cpu_setup(w)
    w.world = world
    _, mean, rstd = O.layernorm_fwd(w.x_host, w.g_host, w.b_host, 1e-5)
    parts = []
    for rank in range(world):
        r0, r1 = shard.shard_rows(w.rows, rank, world)
        w.r0, w.r1 = shard.shard_rows(w.rows, 0, world)
        dx, dw, db = O.layernorm_bwd(w.dy_host[r0:r1], w.x_host[r0:r1], w.g_host, mean[r0:r1], rstd[r0:r1])
        parts.append(torch.cat([dx.half(), dw.half()[None], db.half()[None]]))
    ok, text = w.check(torch.cat(parts))
    assert ok, text


def test_transpose_slabs_are_ranges_of_the_column_major_tile_order():
    import lego_b200 as L
    n, t, world = 256, 32, 4
    nt = n // t
    order = L.OrderBy(L.Col(nt, nt)).TileBy([nt, nt])
    for rank in range(world):
        r0, r1 = shard.shard_transpose(n, n, rank, world, t)
        begin, count = r0 // t * nt, (r1 - r0) // t * nt
        cols = {int(order.inv(i)[1]) for i in range(begin, begin + count)}
        assert cols == set(range(r0 // t, r1 // t))       # source tile columns = output row slab
