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

from . import _abi
from .layout import GenP, GroupBy, OrderBy, RegP

_GENP_KINDS = {"antidiag": _abi.BLOCK_ANTIDIAG, "reverse": _abi.BLOCK_REVERSE}


def lower(layout: GroupBy) -> _abi.Layout:
    """Serialise a layout.  Raises ValueError for shapes beyond the ABI limits
    and for GenP blocks whose body the device evaluator does not know."""
    if not isinstance(layout, GroupBy):
        raise TypeError(f"expected a GroupBy layout (from .TileBy/.GroupBy), got {type(layout).__name__}")
    cached = getattr(layout, "_lowered", None)
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
                if blk.kind not in _GENP_KINDS:
                    raise ValueError(
                        "GenP block without a known `kind` cannot be lowered: the device evaluator "
                        f"knows {sorted(_GENP_KINDS)}")
                dst.kind = _GENP_KINDS[blk.kind]
                for i in range(len(bd)):
                    dst.perm[i] = i
            else:
                raise TypeError(f"unknown permutation block {type(blk).__name__}")
    _abi.check(_abi.lib().lego_layout_check(C.byref(out)), "lego_layout_check")
    layout._lowered = out
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
    desc = lower(layout)
    raw = _abi.Folded()
    _abi.check(_abi.lib().lego_layout_fold(C.byref(desc), C.byref(raw)), "lego_layout_fold")
    terms = [FoldedTerm(t.src, t.div, t.mod, t.stride) for t in raw.terms[:raw.n_terms]]
    return FoldedLayout(bool(raw.foldable), int(raw.size), terms)
