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
