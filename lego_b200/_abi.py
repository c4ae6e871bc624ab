"""ctypes view of ``include/lego_b200.h`` and the loader of the shared library.

The library is the product: there is no Python or CPU fallback behind any op.
If ``liblego_b200.so`` has not been built, loading raises with the build
command instead of degrading.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

MAX_RANK = 12
MAX_BLOCKS = 4
MAX_STAGES = 8
MAX_TERMS = 32
MAX_GROUPS = 256

BLOCK_REGP = 0
BLOCK_ANTIDIAG = 1
BLOCK_REVERSE = 2
BLOCK_LUT = 3
MAX_LUT = 1 << 24

ACT_NONE = 0
ACT_LEAKY_RELU = 1

TUNE_GEMM_BLOCKS = 1
TUNE_GEMM_STREAMK = 2
TUNE_GEMM_LAG = 3
TUNE_LNBWD_SPLIT = 4
TUNE_PERMUTE_TILE_VECS = 5
TUNE_PERMUTE_DMA_TILE = 6
TUNE_PERMUTE_DMA_CTAS = 7
TUNE_PDL_LAST_WAVE = 8
TUNE_LNBWD_LANES = 9
TUNE_PERMUTE_DMA_LONG = 10
TUNE_LNBWD_MIN_ROWS = 11
TUNE_LNBWD_FOLD_WARP = 12

ERR_UNSUPPORTED = -8
ERR_CUDA_BASE = 1000
ERR_DEVICE_TIMEOUT = 2001


class Block(C.Structure):
    _fields_ = [("rank", C.c_int32), ("kind", C.c_int32),
                ("dims", C.c_int64 * MAX_RANK), ("perm", C.c_int32 * MAX_RANK),
                ("lut_apply", C.c_void_p), ("lut_inv", C.c_void_p)]


class Stage(C.Structure):
    _fields_ = [("n_blocks", C.c_int32), ("reserved", C.c_int32), ("blocks", Block * MAX_BLOCKS)]


class Layout(C.Structure):
    _fields_ = [("rank", C.c_int32), ("n_stages", C.c_int32),
                ("dims", C.c_int64 * MAX_RANK), ("stages", Stage * MAX_STAGES)]


class Term(C.Structure):
    _fields_ = [("src", C.c_int32), ("reserved", C.c_int32),
                ("div", C.c_int64), ("mod", C.c_int64), ("stride", C.c_int64)]


class Folded(C.Structure):
    _fields_ = [("foldable", C.c_int32), ("n_terms", C.c_int32), ("size", C.c_int64),
                ("terms", Term * MAX_TERMS)]


class DmaSide(C.Structure):
    _fields_ = [("rank", C.c_int32), ("reserved", C.c_int32),
                ("size", C.c_int64 * 5), ("stride", C.c_int64 * 5), ("box", C.c_int64 * 5)]


class DmaOuter(C.Structure):
    _fields_ = [("radix", C.c_int64), ("ld_dim", C.c_int32), ("ld_mul", C.c_int32),
                ("st_dim", C.c_int32), ("st_mul", C.c_int32), ("reserved", C.c_int32)]


class DmaPlan(C.Structure):
    _fields_ = [("elem_bytes", C.c_int32), ("n_outer", C.c_int32), ("n_tiles", C.c_int64),
                ("tile_bytes", C.c_int64), ("load", DmaSide), ("store", DmaSide), ("outer", DmaOuter * 8)]


LayoutP = C.POINTER(Layout)

# name -> (restype, argtypes); must list every function include/lego_b200.h declares.
SIGNATURES = {
    "lego_layout_check": (C.c_int32, [LayoutP]),
    "lego_layout_fold": (C.c_int32, [LayoutP, C.POINTER(Folded)]),
    "lego_permute_plan": (C.c_int32, [C.c_int32, LayoutP, LayoutP, LayoutP, C.POINTER(C.c_int32),
                                      C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "lego_permute_dma_plan": (C.c_int32, [C.c_int32, LayoutP, LayoutP, C.c_int64, C.POINTER(DmaPlan)]),
    "lego_eval_apply": (C.c_int32, [LayoutP, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "lego_eval_inv": (C.c_int32, [LayoutP, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "lego_eval_range": (C.c_int32, [LayoutP, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "lego_permute": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, LayoutP, LayoutP, LayoutP, C.c_void_p]),
    "lego_permute_tiles": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, LayoutP, LayoutP, LayoutP, C.c_int64,
                                       C.c_int64, C.c_void_p]),
    "lego_permute_slab_info": (C.c_int32, [C.c_int32, LayoutP, LayoutP, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "lego_permute_slabs": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, LayoutP, LayoutP, C.c_int64, C.c_void_p]),
    "lego_softmax_f16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, LayoutP, C.c_void_p]),
    "lego_softmax_f32": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, LayoutP, C.c_void_p]),
    "lego_layernorm_fwd_f16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int64, C.c_int64, C.c_float, LayoutP, C.c_void_p]),
    "lego_layernorm_bwd_partial_rows": (C.c_int64, [C.c_int64, C.c_int64]),
    "lego_layernorm_bwd_f16": (C.c_int32, [C.c_void_p] * 9 + [C.c_int64, C.c_int64, C.c_void_p]),
    "lego_gemm_f16": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                  C.c_int32, C.c_int32, C.c_int32, LayoutP, C.c_void_p]),
    "lego_gemm_e5m2": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                   C.c_int32, C.c_int32, C.c_int32, LayoutP, C.c_void_p]),
    "lego_gemm_workspace_bytes": (C.c_int64, []),
    "lego_gemm_f16_ws": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                     C.c_int32, C.c_int32, C.c_int32, LayoutP, C.c_void_p, C.c_int64, C.c_void_p]),
    "lego_gemm_e5m2_ws": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                      C.c_int32, C.c_int32, C.c_int32, LayoutP, C.c_void_p, C.c_int64, C.c_void_p]),
    "lego_tune": (C.c_int32, [C.c_int32, C.c_int32]),
    "lego_selftest_bounded_wait": (C.c_int32, [C.c_int64, C.c_void_p]),
    "lego_grouped_gemm_f16": (C.c_int32, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                          C.POINTER(C.c_int64), C.c_int32, C.POINTER(LayoutP), C.c_void_p]),
    "lego_grouped_gemm_f16_static": (C.c_int32, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                                 C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.c_int32,
                                                 C.POINTER(LayoutP), C.c_void_p, C.c_void_p]),
    "lego_copy_2d": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "lego_device_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "lego_status_string": (C.c_char_p, [C.c_int32]),
    "lego_shutdown": (C.c_int32, []),
}

_LIB = None
_LOCK = threading.Lock()


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "liblego_b200.so")


def lib() -> C.CDLL:
    """The loaded shared library with argument types set; raises if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m lego_b200.build` "
                "(needs nvcc with sm_100a support). lego_b200 has no fallback path.")
        handle = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB


class LegoError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().lego_status_string(status).decode()
        super().__init__(f"{where}: {msg} (status {status})")


def check(status: int, where: str) -> None:
    """Map a status of the C ABI onto the exceptions the reference raises:
    argument problems are ValueError (``lego/lego.py:100,170,216,295,395``)."""
    if status == 0:
        return
    if status < 0:
        msg = lib().lego_status_string(status).decode()
        raise ValueError(f"{where}: {msg} (status {status})")
    raise LegoError(status, where)
