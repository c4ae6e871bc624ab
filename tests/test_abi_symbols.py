"""The shared library loads and exports every function include/lego_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

import pytest

from lego_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "lego_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lego_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 17
    handle = ctypes.CDLL(_abi.library_path())
    for name in names:
        assert hasattr(handle, name), f"{name} declared but not exported"
        assert name in _abi.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_abi.SIGNATURES) == names


def test_struct_sizes_match_the_header():
    # lego_block_t: 2 x int32 + 12 x int64 + 12 x int32
    assert ctypes.sizeof(_abi.Block) == 8 + 96 + 48 + 16
    assert ctypes.sizeof(_abi.Stage) == 8 + 4 * ctypes.sizeof(_abi.Block)
    assert ctypes.sizeof(_abi.Layout) == 8 + 96 + 8 * ctypes.sizeof(_abi.Stage)
    assert ctypes.sizeof(_abi.Term) == 32
    assert ctypes.sizeof(_abi.Folded) == 16 + 32 * 32


def test_status_strings_and_host_only_calls():
    lib = _abi.lib()
    assert lib.lego_status_string(0) == b"ok"
    assert b"bijection" in lib.lego_status_string(-5)
    assert lib.lego_layout_check(None) == -1
    assert lib.lego_layernorm_bwd_partial_rows(10, 64) == 10
    assert lib.lego_layernorm_bwd_partial_rows(100000, 64) == 1184


def test_device_timeout_status_maps_to_lego_error():
    """The status a caller sees when a bounded wait inside a kernel ran out (2001), and a CUDA
    runtime error (1000 + cudaError_t), surface as LegoError with the library's text; argument
    errors (negative) as ValueError."""
    lib = _abi.lib()
    assert b"wait" in lib.lego_status_string(2001).lower() or b"timeout" in lib.lego_status_string(2001).lower()
    with pytest.raises(_abi.LegoError) as e:
        _abi.check(2001, "lego_device_status")
    assert e.value.status == 2001 and "lego_device_status" in str(e.value)
    with pytest.raises(_abi.LegoError):
        _abi.check(1000 + 2, "lego_softmax_f16")
    with pytest.raises(ValueError):
        _abi.check(-5, "lego_layout_check")
    _abi.check(0, "anything")
