"""Host-resident operands: the calls a user makes with CPU tensors stage the data
through the device in blocks (copy-in / compute / copy-out on three streams).  The
results must be bit-identical to the same call on device-resident tensors, pinned or
pageable input alike, and must come back on the host."""
import pytest
import torch

import lego_b200 as L
from lego_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def small_blocks(monkeypatch):
    """8 MiB blocks so that inputs of some 20 MiB already take the staged route"""
    monkeypatch.setattr(ops, "_HOST_BLOCK_BYTES", 8 << 20)


def _both(x):
    """the tensor as pageable and as pinned host memory"""
    return (("pageable", x), ("pinned", x.pin_memory()))


def test_softmax_host_rows_match_device_rows():
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(2600, 4096, generator=g) * 2).half()   # 20 MiB: three blocks, the last one ragged
    want = ops.softmax(x.cuda()).cpu()
    for name, xh in _both(x):
        got = ops.softmax(xh, ops.row_tiling_layout(2600, 4))
        assert not got.is_cuda, name
        assert torch.equal(got, want), name
    # small inputs take the one-shot route and agree as well
    small = x[:64].contiguous()
    assert torch.equal(ops.softmax(small), ops.softmax(small.cuda()).cpu())


def test_layernorm_host_rows_match_device_rows():
    g = torch.Generator().manual_seed(12)
    x = torch.randn(3, 900, 4096, generator=g).half()       # leading axes are flattened into rows
    w = (1 + 0.1 * torch.randn(4096, generator=g)).half()
    b = (0.1 * torch.randn(4096, generator=g)).half()
    y_d, mean_d, rstd_d = ops.layer_norm_fwd(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    for name, xh in _both(x):
        y, mean, rstd = ops.layer_norm_fwd(xh, w, b, 1e-5)
        assert y.shape == x.shape and not y.is_cuda, name
        assert torch.equal(y, y_d.cpu()), name
        assert torch.equal(mean, mean_d.cpu()) and torch.equal(rstd, rstd_d.cpu()), name


def test_matmul_host_operands_match_device_operands():
    g = torch.Generator().manual_seed(13)
    m, n, k = 2304, 1024, 4096                               # A is 18 MiB: blocks of 1024, 1024 and 256 rows
    a = (torch.randn(m, k, generator=g) / 64).half()
    b = (torch.randn(k, n, generator=g) / 64).half()
    # Whole tiles only: the bits of a tile do not depend on how the rows are blocked.  (With the
    # stream-K tail the k-range of a tile is cut where the SM count says, so the fp32 partial
    # sums of host blocks and of one device call are added in different orders.)
    ops.tune(gemm_streamk=0)
    try:
        want = ops.matmul(a.cuda(), b.cuda()).cpu()
        for name, ah in _both(a):
            got = ops.matmul(ah, b)
            assert not got.is_cuda and torch.equal(got, want), name
        # B given as the .T view of an [n, k] matrix, and the fused activation
        bt = b.t().contiguous()
        got = ops.matmul(a.pin_memory(), bt.t(), activation="leaky_relu")
        assert torch.equal(got, ops.matmul(a.cuda(), b.cuda(), activation="leaky_relu").cpu())
    finally:
        ops.tune(gemm_streamk=0)
    ref = a.float() @ b.float()
    for name, ah in _both(a):
        got = ops.matmul(ah, b)
        assert ((got.float() - ref).norm() / ref.norm()).item() <= 1e-3, name


def test_grouped_gemm_host_groups_match_device_groups():
    g = torch.Generator().manual_seed(14)
    sizes = [(256, 512, 1024), (1024, 256, 512), (384, 768, 256)]
    A = [(torch.randn(m, k, generator=g) / 16).half() for m, n, k in sizes]
    B = [(torch.randn(k, n, generator=g) / 16).half() for m, n, k in sizes]
    want = [c.cpu() for c in ops.lego_group_gemm_fn([t.cuda() for t in A], [t.cuda() for t in B])]
    got = ops.lego_group_gemm_fn([t.pin_memory() for t in A], B)
    assert all(not c.is_cuda for c in got)
    assert all(torch.equal(c, w) for c, w in zip(got, want))
    orders = [L.OrderBy(L.Row(-(-m // 128), -(-n // 256))).TileBy([-(-m // 128), -(-n // 256)]) for m, n, _ in sizes]
    got = ops.lego_group_gemm_fn(A, B, orders)
    assert all(torch.equal(c, w) for c, w in zip(got, want))


def test_eval_range_into_host_memory():
    lay = L.OrderBy(L.Col(2048, 2048)).TileBy([64, 64], [32, 32])   # 2^22 ids = 32 MiB of int64
    want = ops.eval_range(lay).cpu()
    got = ops.eval_range(lay, host=True)
    assert not got.is_cuda and torch.equal(got, want)
    part = ops.eval_range(lay, begin=12345, count=3 * (1 << 20) + 17, host=True)
    assert torch.equal(part, want[12345:12345 + 3 * (1 << 20) + 17])
    assert torch.equal(ops.eval_range(lay, count=1000, host=True), want[:1000])


def test_layernorm_backward_host_rows():
    g = torch.Generator().manual_seed(15)
    rows, cols = 2500, 4096                                  # 20 MiB each of x and dy: three blocks
    x = torch.randn(rows, cols, generator=g).half()
    dy = (0.1 * torch.randn(rows, cols, generator=g)).half()
    w = (1 + 0.1 * torch.randn(cols, generator=g)).half()
    b = (0.1 * torch.randn(cols, generator=g)).half()
    _, mean, rstd = ops.layer_norm_fwd(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    dx_d, dw_d, db_d = ops.layer_norm_bwd(dy.cuda(), x.cuda(), w.cuda(), mean, rstd)
    dx, dw, db = ops.layer_norm_bwd(dy.pin_memory(), x.pin_memory(), w, mean.cpu(), rstd.cpu())
    assert not dx.is_cuda and not dw.is_cuda and not db.is_cuda
    assert torch.equal(dx, dx_d.cpu())                       # rows are independent: same bits
    # the column sums are rounded to fp16 per block (at the magnitude of the block's sum) and once more
    # at the end: a few fp16 ulps of the largest entry, far inside the 1e-2 of the largest entry that
    # the oracle comparison allows
    for got, want in ((dw, dw_d.cpu()), (db, db_d.cpu())):
        assert (got.float() - want.float()).abs().max().item() <= 2e-3 * want.float().abs().max().item()


def test_brick_relayout_host_volume_is_staged_by_slabs():
    """A volume on the host whose re-layout splits along the outermost brick coordinate goes
    through the device slab group by slab group (lego_permute_slabs); bit-identical to the
    one-call re-layout of the device-resident volume, both directions."""
    b, dims = 8, (160, 192, 256)                             # 30 MiB fp32, 20 slabs of 1.5 MiB
    tiles = [d // b for d in dims]
    normal = L.OrderBy(L.Row(*dims)).TileBy(tiles, [b] * 3)
    bricks = L.OrderBy(L.Row(*tiles), L.Row(b, b, b)).TileBy(tiles, [b] * 3)
    assert ops.permute_slab_info(4, normal, bricks) == (20, 8 * 192 * 256)
    x = torch.rand(*dims, generator=torch.Generator().manual_seed(14))
    want = ops.permute(x.cuda(), normal, bricks).cpu()
    assert torch.equal(want.reshape(-1), x.reshape(tiles[0], b, tiles[1], b, tiles[2], b).permute(0, 2, 4, 1, 3, 5)
                       .contiguous().reshape(-1))
    for name, xh in _both(x):
        got = ops.permute(xh, normal, bricks)
        assert not got.is_cuda and got.shape == x.shape, name
        assert torch.equal(got, want), name
        assert torch.equal(ops.permute(got, bricks, normal), x), name
    # a range of slabs on device buffers: what one GPU of several would move
    xd = x.cuda()
    part = ops.permute_slabs(xd[3 * b:10 * b], normal, bricks, 7)
    assert torch.equal(part.cpu().reshape(-1), want.reshape(-1)[3 * 8 * 192 * 256:10 * 8 * 192 * 256])
    with pytest.raises(ValueError):
        ops.permute_slabs(xd[:3 * b], normal, bricks, 4)     # tensor and count disagree
    ops.device_status()
