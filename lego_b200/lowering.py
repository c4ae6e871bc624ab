"""Layout objects -> the C-ABI descriptor (``lego_layout_t``).

Lowering is a plain serialisation of ``GroupBy.objects`` (stage by stage, block
by block); validation, constant folding and strength reduction happen in the
native library (``lego_layout_check`` / ``lego_layout_fold``), so every binding
gets the same treatment.  This replaces the reference's printers
(``lego/lego_python.py:10-37``, ``lego/lego_c.py:9-38``,
``lego/lego_mlir.py:180-272``), which serialise the layout as expression text.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from . import _abi
from .layout import GenP, GroupBy, OrderBy, RegP, unflatten_index

_GENP_KINDS = {"antidiag": _abi.BLOCK_ANTIDIAG, "reverse": _abi.BLOCK_REVERSE}


def genp_tables(blk: GenP):
    """Tabulate a GenP block over its whole domain: ``(apply_table, inv_table)`` as int64
    arrays of ``prod(dims)`` entries.  ``apply_table[r]`` is ``f_apply`` at the index whose
    row-major id over ``dims`` is ``r``; it must be a permutation of ``0 .. size-1`` (that is
    what makes the block a bijection, and what the reference silently assumes,
    ``lego/lego.py:150-178``).  ``inv_table`` is its inverse; when the block carries an
    ``f_inv`` it is checked against the table on a sample."""
    dims = blk.dims()
    size = 1
    for d in dims:
        size *= int(d)
    if size > _abi.MAX_LUT:
        raise ValueError(f"GenP block of {size} entries is beyond the table limit of {_abi.MAX_LUT}; "
                         "give it a `kind` the device evaluator computes in closed form")
    ids = np.arange(size, dtype=np.int64)
    idx = unflatten_index(ids, dims)
    try:
        table = np.asarray(blk.f_apply(tuple(idx)), dtype=np.int64)
        if table.shape != (size,):
            raise TypeError
    except Exception:  # the callable is scalar-only (SymPy Piecewise, Python branches): one id at a time
        table = np.fromiter((int(blk.f_apply(tuple(int(c[i]) for c in idx))) for i in range(size)),
                            dtype=np.int64, count=size)
    inv = np.full(size, -1, dtype=np.int64)
    ok = (table >= 0) & (table < size)
    if not ok.all():
        raise ValueError("GenP f_apply leaves the block's index range: not a permutation")
    inv[table] = ids
    if (inv < 0).any():
        raise ValueError("GenP f_apply is not a bijection over the block's dims")
    if blk.f_inv is not None:
        probe = np.unique(np.linspace(0, size - 1, num=min(size, 257)).astype(np.int64))
        for f in probe:
            got = tuple(int(v) for v in blk.f_inv(int(f)))
            want = tuple(int(c[inv[f]]) for c in idx)
            if got != want:
                raise ValueError(f"GenP f_inv({int(f)}) = {got} disagrees with f_apply, whose inverse there is {want}")
    return table, inv


def _device_tables(blk: GenP):
    """The block's tables on the current CUDA device (kept on the block, per device)."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("lego_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    dev = torch.cuda.current_device()
    cache = blk.__dict__.setdefault("_tables", {})
    if dev not in cache:
        host = blk.__dict__.get("_host_tables")
        if host is None:
            host = blk.__dict__["_host_tables"] = genp_tables(blk)
        cache[dev] = tuple(torch.from_numpy(t).to(torch.device("cuda", dev)) for t in host)
    return cache[dev]


def lower(layout: GroupBy, host_only: bool = False) -> _abi.Layout:
    """Serialise a layout.  Raises ValueError for shapes beyond the ABI limits.  A GenP block
    with a known ``kind`` lowers to its closed form; any other GenP is tabulated on the host
    once and lowers to a pair of device tables (``LEGO_BLOCK_LUT``).  ``host_only`` is for the
    host services (validation, folding), which never read a table: the descriptor then points
    at the host copies and must not reach a kernel."""
    if not isinstance(layout, GroupBy):
        raise TypeError(f"expected a GroupBy layout (from .TileBy/.GroupBy), got {type(layout).__name__}")
    uses_tables = any(isinstance(b, GenP) and b.kind not in _GENP_KINDS for o in layout.objects for b in o.perms)
    key = "_lowered"
    if uses_tables and host_only:
        key = "_lowered_host"
    elif uses_tables:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("lego_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
        key = f"_lowered_dev{torch.cuda.current_device()}"
    cached = layout.__dict__.get(key)
    if cached is not None:
        return cached
    dims = layout.dims()
    if not 1 <= len(dims) <= _abi.MAX_RANK:
        raise ValueError(f"layout rank {len(dims)} outside 1..{_abi.MAX_RANK}")
    stages = [o for o in layout.objects if o.dims()]
    if len(stages) > _abi.MAX_STAGES:
        raise ValueError(f"layout has {len(stages)} stages, limit is {_abi.MAX_STAGES}")
    out = _abi.Layout()
    out.rank = len(dims)
    out.n_stages = len(stages)
    for k, d in enumerate(dims):
        out.dims[k] = int(d)
    for s, obj in enumerate(stages):
        if not isinstance(obj, OrderBy):
            raise TypeError("GroupBy.objects must be OrderBy stages")
        if len(obj.perms) > _abi.MAX_BLOCKS:
            raise ValueError(f"OrderBy has {len(obj.perms)} blocks, limit is {_abi.MAX_BLOCKS}")
        st = out.stages[s]
        st.n_blocks = len(obj.perms)
        for b, blk in enumerate(obj.perms):
            bd = blk.dims()
            if not 1 <= len(bd) <= _abi.MAX_RANK:
                raise ValueError(f"block rank {len(bd)} outside 1..{_abi.MAX_RANK}")
            dst = st.blocks[b]
            dst.rank = len(bd)
            for i, d in enumerate(bd):
                dst.dims[i] = int(d)
            if isinstance(blk, RegP):
                dst.kind = _abi.BLOCK_REGP
                for i, p in enumerate(blk.permutation):
                    dst.perm[i] = int(p)
            elif isinstance(blk, GenP):
                for i in range(len(bd)):
                    dst.perm[i] = i
                if blk.kind in _GENP_KINDS:
                    dst.kind = _GENP_KINDS[blk.kind]
                else:
                    dst.kind = _abi.BLOCK_LUT
                    if host_only:
                        host = blk.__dict__.get("_host_tables")
                        if host is None:
                            host = blk.__dict__["_host_tables"] = genp_tables(blk)
                        dst.lut_apply, dst.lut_inv = host[0].ctypes.data, host[1].ctypes.data
                    else:
                        t_apply, t_inv = _device_tables(blk)
                        dst.lut_apply, dst.lut_inv = t_apply.data_ptr(), t_inv.data_ptr()
            else:
                raise TypeError(f"unknown permutation block {type(blk).__name__}")
    _abi.check(_abi.lib().lego_layout_check(C.byref(out)), "lego_layout_check")
    layout.__dict__[key] = out
    return out


def lower_optional(layout: Optional[GroupBy]):
    return None if layout is None else C.byref(lower(layout))


@dataclass(frozen=True)
class FoldedTerm:
    src: int
    div: int
    mod: int
    stride: int


@dataclass(frozen=True)
class FoldedLayout:
    foldable: bool
    size: int
    terms: List[FoldedTerm]


def fold(layout: GroupBy) -> FoldedLayout:
    """The library's constant-folded form of a layout:
    ``flat = sum_j ((idx[src_j] // div_j) % mod_j) * stride_j``."""
    desc = lower(layout, host_only=True)
    raw = _abi.Folded()
    _abi.check(_abi.lib().lego_layout_fold(C.byref(desc), C.byref(raw)), "lego_layout_fold")
    terms = [FoldedTerm(t.src, t.div, t.mod, t.stride) for t in raw.terms[:raw.n_terms]]
    return FoldedLayout(bool(raw.foldable), int(raw.size), terms)
