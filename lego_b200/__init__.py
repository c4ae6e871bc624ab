"""lego_b200: B200 (sm_100a) back end for LEGO layouts.

The layout vocabulary of the reference (``Row``, ``Col``, ``RegP``, ``GenP``,
``OrderBy(...).TileBy(...)``, ``GroupBy``) is the Python API; ops lower a layout
to a C-ABI descriptor and run hand-written CUDA kernels.  There is no CPU or
Triton fallback behind any op.
"""
from .layout import (Col, GenP, GroupBy, OrderBy, RegP, Row, antidiag, antidiag_inv,
                     flatten_index, get_sigma_perm, inverse_permutation, unflatten_index)
from .lowering import fold, lower

__all__ = [
    "Row", "Col", "RegP", "GenP", "OrderBy", "GroupBy", "flatten_index", "unflatten_index",
    "get_sigma_perm", "inverse_permutation", "antidiag", "antidiag_inv", "lower", "fold",
]
