"""Splitting a named workload across the GPUs of one box.

The hot path shards with no exchange step: rows of the row-wise kernels, output
row slabs of a transpose, row blocks of A and C for a GEMM and row blocks of
every group's A and C for a grouped GEMM are independent.  These helpers are
pure host arithmetic (no torch.distributed calls): rank ``r`` of ``world``
learns which contiguous slab is its own.  Slabs are aligned so that each rank's
piece still satisfies the kernels' tile and vector constraints.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def split_range(n: int, rank: int, world: int, align: int = 1) -> Tuple[int, int]:
    """``[begin, end)`` of rank's share of ``n`` items, in units of ``align``;
    the first ``(n / align) % world`` ranks get one extra unit and every item is
    covered exactly once."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if align < 1 or n < 0:
        raise ValueError("align must be >= 1 and n >= 0")
    units, tail = divmod(n, align)
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    begin, end = begin_u * align, end_u * align
    if rank == world - 1:
        end += tail  # a ragged remainder smaller than one unit stays with the last rank
    return begin, end


def shard_rows(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Row block of a row-wise kernel (softmax, LayerNorm)."""
    return split_range(n_rows, rank, world)


def shard_transpose(n_rows: int, n_cols: int, rank: int, world: int, tile: int = 32) -> Tuple[int, int]:
    """Slab of *output* rows (= input columns) of a 2-D transpose, whole tiles."""
    return split_range(n_cols, rank, world, tile)


def shard_gemm_m(m: int, rank: int, world: int, tile_m: int = 128) -> Tuple[int, int]:
    """Row block of A and C; B is replicated."""
    return split_range(m, rank, world, tile_m)


def shard_grouped_gemm(mnk: Sequence[Tuple[int, int, int]], rank: int, world: int,
                       tile_m: int = 128) -> List[Tuple[int, int]]:
    """Every group's M is split across the ranks (whole-group assignment cannot
    balance ragged groups); returns one ``[begin, end)`` row block per group."""
    return [split_range(m, rank, world, tile_m) for m, _n, _k in mnk]


def pack_grouped_gemm_blocks(mnk: Sequence[Tuple[int, int, int]], world: int,
                             block_m: int = 512) -> List[List[Tuple[int, int, int]]]:
    """Every group's M is cut into blocks of ``block_m`` rows (the last one of a group may be
    shorter) and the blocks are packed onto the ranks, heaviest first onto the least loaded
    rank (weight = rows x N x K).  Returns, per rank, its ``(group, row_begin, row_end)`` list
    in group order.  Blocks of 512 rows keep every rank's problems on the GEMM's 512 x 256
    tiles, where an even split of every group's M (128 rows per rank for M = 1024 on eight
    ranks) would fall back to one 128-row tile per SM; ragged groups still balance to within
    one block.  Deterministic: every rank computes the same packing."""
    if world < 1 or block_m < 1:
        raise ValueError("world and block_m must be >= 1")
    blocks = []
    for g, (m, n, k) in enumerate(mnk):
        for b in range(0, m, block_m):
            e = min(m, b + block_m)
            blocks.append(((e - b) * n * k, g, b, e))
    blocks.sort(key=lambda t: (-t[0], t[1], t[2]))
    load = [0] * world
    out: List[List[Tuple[int, int, int]]] = [[] for _ in range(world)]
    for w, g, b, e in blocks:
        r = min(range(world), key=lambda i: (load[i], i))
        load[r] += w
        out[r].append((g, b, e))
    for lst in out:
        lst.sort()
    return out
