"""The non-allocating grouped GEMM entry point (lego_grouped_gemm_f16_static).

Some callers cannot let a library call cudaMalloc: a serving process whose device
memory is wholly owned by a caching allocator, for instance.  This entry point
keeps its scratch (problem table + status word) in a __device__ array inside the
library.  The test drives it through the C ABI twice in a row -- the array is
shared between calls and keeps the previous call's contents -- and requires the
very bits the allocating entry point produces, plus a clean status word.  It is
collected last so that a failure here cannot hide any other test, and it must
pass alone in a fresh process as well as after the rest of the suite.
"""
import ctypes as C

import pytest
import torch

from lego_b200 import _abi, ops

pytestmark = pytest.mark.gpu


def _call_static(A, B, status=None):
    g = len(A)
    outs = [torch.empty((a.shape[0], b.shape[1]), dtype=torch.float16, device="cuda") for a, b in zip(A, B)]
    Ptr = C.c_void_p * g
    mnk = (C.c_int64 * (3 * g))(*[v for a, b in zip(A, B) for v in (a.shape[0], b.shape[1], a.shape[1])])
    st = _abi.lib().lego_grouped_gemm_f16_static(
        Ptr(*[t.data_ptr() for t in A]), Ptr(*[t.data_ptr() for t in B]), Ptr(*[t.data_ptr() for t in outs]),
        mnk, g, None, None if status is None else status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return st, outs


def test_static_scratch_matches_allocating_entry_point_twice():
    gen = torch.Generator().manual_seed(21)
    shapes1 = [(256, 512, 192), (130, 264, 72), (1024, 256, 512)]
    shapes2 = [(128, 256, 64), (512, 1024, 256), (384, 768, 320), (1, 8, 8), (640, 512, 1024)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for shapes in (shapes1, shapes2):          # second call reuses the array with a longer table
        A = [(torch.randn(m, k, generator=gen) / 16).half().cuda() for m, n, k in shapes]
        B = [(torch.randn(k, n, generator=gen) / 16).half().cuda() for m, n, k in shapes]
        want = ops.lego_group_gemm_fn(A, B)
        ops.device_status()
        st, got = _call_static(A, B, status)
        assert st == 0, _abi.lib().lego_status_string(st)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for w, g in zip(want, got):
            assert torch.equal(w, g)            # same kernel, same tile order: identical bits
        st, got2 = _call_static(A, B)           # status word inside the array, cleared by the call
        assert st == 0
        torch.cuda.synchronize()
        for w, g in zip(want, got2):
            assert torch.equal(w, g)


def test_static_entry_point_allocates_no_device_memory():
    """Free device memory as the driver reports it is the same before and after a run of
    calls (the first call, made above or here, has already loaded the kernels)."""
    gen = torch.Generator().manual_seed(22)
    A = [(torch.randn(256, 128, generator=gen) / 16).half().cuda() for _ in range(3)]
    B = [(torch.randn(128, 512, generator=gen) / 16).half().cuda() for _ in range(3)]
    outs = [torch.empty((256, 512), dtype=torch.float16, device="cuda") for _ in range(3)]
    Ptr = C.c_void_p * 3
    args = (Ptr(*[t.data_ptr() for t in A]), Ptr(*[t.data_ptr() for t in B]), Ptr(*[t.data_ptr() for t in outs]),
            (C.c_int64 * 9)(*([256, 512, 128] * 3)), 3, None, None, torch.cuda.current_stream().cuda_stream)
    lib = _abi.lib()
    assert lib.lego_grouped_gemm_f16_static(*args) == 0      # loads the module if nothing has yet
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(20):
        assert lib.lego_grouped_gemm_f16_static(*args) == 0
    torch.cuda.synchronize()
    assert lib.lego_device_status(torch.cuda.current_stream().cuda_stream, None) == 0   # reads the in-array word
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for o, a, b in zip(outs, A, B):
        ref = a.float() @ b.float()
        assert ((o.float() - ref).norm() / ref.norm()).item() <= 1e-3


def test_static_scratch_rejects_more_groups_than_it_holds():
    a = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(64, 256, dtype=torch.float16, device="cuda")
    st, _ = _call_static([a] * 65, [b] * 65)
    assert st == -6 and b"sizes" in _abi.lib().lego_status_string(st)
    st, outs = _call_static([a] * 64, [b] * 64)
    assert st == 0
    torch.cuda.synchronize()
    assert all(not o.any() for o in outs)
