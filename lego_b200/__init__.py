"""lego_b200: B200 (sm_100a) back end for LEGO layouts.

The layout vocabulary of the reference (``Row``, ``Col``, ``RegP``, ``GenP``,
``OrderBy(...).TileBy(...)``, ``GroupBy``) is the Python API; ops lower a layout
to a C-ABI descriptor and run hand-written CUDA kernels.  There is no CPU or
Triton fallback behind any op.
"""
from .layout import (Col, GenP, GroupBy, OrderBy, RegP, Row, antidiag, antidiag_inv,
                     divisibility_constraint, equal_constraint, flatten_index, get_arange,
                     get_sigma_perm, inverse_permutation, le_constraint, new_antidiag,
                     new_antidiag_inv, unflatten_index)
from .lowering import fold, lower

__all__ = [
    "Row", "Col", "RegP", "GenP", "OrderBy", "GroupBy", "flatten_index", "unflatten_index",
    "get_sigma_perm", "inverse_permutation", "antidiag", "antidiag_inv", "new_antidiag",
    "new_antidiag_inv", "get_arange", "divisibility_constraint", "le_constraint", "equal_constraint",
    "lower", "fold",
]
