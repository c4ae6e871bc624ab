"""Device housekeeping through the C ABI: the bounded waits' give-up path, and one process
driving two GPUs."""
import ctypes as C

import pytest
import torch

from lego_b200 import _abi, ops
from inputs import softmax_input
from oracle import lego_oracle as O

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_the_device_stays_usable():
    """A wait whose barrier nothing completes runs out after its cycle limit, the kernel
    records its code and returns; the host sees LEGO_ERR_DEVICE_TIMEOUT once, and the next
    kernel on the same context runs and is correct.  Nothing faults and nothing hangs."""
    ops.device_status()
    ops.selftest_bounded_wait(1_000_000)         # about half a millisecond of SM clock
    detail = C.c_uint32(0)
    st = _abi.lib().lego_device_status(torch.cuda.current_stream().cuda_stream, C.byref(detail))
    assert st == _abi.ERR_DEVICE_TIMEOUT
    assert detail.value == 0x7E570000
    assert b"bounded wait" in _abi.lib().lego_status_string(st)
    ops.selftest_bounded_wait(200_000)
    with pytest.raises(_abi.LegoError):
        ops.device_status()                      # the Python wrapper raises
    assert ops.device_status() == 0              # the word was cleared by the read
    x = softmax_input(64, 2048)
    y = ops.softmax(x.cuda())
    assert ops.device_status() == 0
    assert (y.cpu().float() - O.softmax(x).float()).abs().max().item() <= 1e-3
    with pytest.raises(ValueError):
        ops.selftest_bounded_wait(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_one_process_two_devices():
    """Kernel set-up (the opt-in to large dynamic shared memory, cluster occupancy) is kept
    per device: every op runs on cuda:0 and then on cuda:1 from the same process."""
    import math
    import lego_b200 as L
    g = torch.Generator().manual_seed(3)
    x = softmax_input(512, 8192)
    a = (torch.randn(512, 256, generator=g) / 16).half()
    b = (torch.randn(256, 512, generator=g) / 16).half()
    t = torch.rand(256, 256, generator=g)
    w, bias = torch.ones(8192).half(), torch.zeros(8192).half()
    for dev in (0, 1):
        with torch.cuda.device(dev):
            d = torch.device("cuda", dev)
            y = ops.softmax(x.to(d))
            assert (y.cpu().float() - O.softmax(x).float()).abs().max().item() <= 1e-3
            yn, mean, rstd = ops.layer_norm_fwd(x.to(d), w.to(d), bias.to(d), 1e-5)
            dx, dw, db = ops.layer_norm_bwd(yn, x.to(d), w.to(d), mean, rstd)
            c = ops.matmul(a.to(d), b.to(d))
            assert ((c.cpu().float() - O.matmul(a, b)).norm() / O.matmul(a, b).norm()).item() <= 1e-3
            cg = ops.lego_group_gemm_fn([a.to(d)], [b.to(d)])[0]
            assert torch.equal(cg, c)
            tt = ops.transpose(t.to(d))
            assert torch.equal(tt.cpu(), t.t().contiguous())
            assert ops.device_status() == 0
