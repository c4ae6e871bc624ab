"""Row-wise softmax and LayerNorm on the GPU, through the C ABI, against the
oracle (torch CPU fp32, what the reference's own checks compare with).
Tolerances: softmax / LayerNorm output max-abs 1e-3 in fp16, statistics
relative 1e-5; fp32 softmax 1e-6."""
import pytest
import torch

import lego_b200 as L
from lego_b200 import ops
from inputs import layernorm_input, softmax_input
from oracle import lego_oracle as O

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3


def ln_error_ok(y16, ref32):
    """LayerNorm output check against the un-rounded fp32 oracle: max-abs 1e-3
    wherever fp16 can represent it (|y| < 2, half an ulp is below 1e-3); beyond
    that the output grid itself is coarser, so the bound is half an fp16 ulp of
    the value (2^-11 |y|) plus 1e-4 of arithmetic slack."""
    err = (y16.float() - ref32).abs()
    small = ref32.abs() < 2
    ok_small = (err[small] <= TOL_F16).all().item() if small.any() else True
    ok_large = (err[~small] <= ref32[~small].abs() * 2.0 ** -11 + 1e-4).all().item() if (~small).any() else True
    return ok_small and ok_large


def ln_ref32(x, w, b, eps):
    return O.layernorm_fwd(x, w, b, eps, round_output=False)[0]


def test_softmax_config2_rows_subset_and_full_properties():
    x = softmax_input(16384, 8192)
    y = ops.softmax(x.cuda(), ops.row_tiling_layout(16384, 4))
    # oracle on a bounded sample of rows (CPU softmax of the whole matrix takes a while)
    sel = torch.arange(0, 16384, 37)
    assert (y[sel.cuda()].cpu().float() - O.softmax(x[sel]).float()).abs().max().item() <= TOL_F16
    # full size: rows sum to one, order of every row is preserved, nothing negative / NaN
    s = y.float().sum(dim=1)
    assert (s - 1).abs().max().item() < 2e-2
    assert torch.isfinite(y).all() and (y >= 0).all()
    assert torch.equal(y.argmax(dim=1).cpu(), x.float().argmax(dim=1))


@pytest.mark.parametrize("rows,cols", [(1823, 781), (4, 8), (1, 1), (33, 256), (7, 1024), (5, 1032),
                                       (3, 4096), (2, 8192), (2, 8200), (1, 32768), (9, 2047)])
def test_softmax_shapes_f16_f32(rows, cols):
    g = torch.Generator().manual_seed(rows * 131 + cols)
    x32 = torch.randn(rows, cols, generator=g)                     # the reference's own case is 1823 x 781 fp32
    y32 = ops.softmax(x32.cuda()).cpu()
    assert (y32 - torch.softmax(x32, dim=-1)).abs().max().item() <= 1e-6
    x16 = (x32 * 2).half()
    y16 = ops.softmax(x16.cuda()).cpu()
    assert (y16.float() - O.softmax(x16).float()).abs().max().item() <= TOL_F16


@pytest.mark.parametrize("cols", [1024, 1536, 2048, 4096, 5120, 8192, 12288, 16384])
def test_ring_kernel_group_sizes(cols):
    """Enough rows (>= 2 per SM) of 2 KiB or more for the bulk-copy ring kernel, at widths that
    give every consumer-group size from one warp (1024 fp16 values) to sixteen (16384), a width
    that leaves part of a group idle (1536, 5120, 12288), fp16 and fp32, with and without a row
    map; softmax and LayerNorm against the oracle on every row."""
    rows = 332
    g = torch.Generator().manual_seed(cols)
    x32 = torch.randn(rows, cols, generator=g) * 3
    x16 = x32.half()
    rm = L.OrderBy(L.Col(83, 4)).TileBy([83, 4])
    y16 = ops.softmax(x16.cuda()).cpu()
    assert (y16.float() - O.softmax(x16).float()).abs().max().item() <= TOL_F16
    assert torch.equal(ops.softmax(x16.cuda(), rm).cpu(), y16)
    if cols * 4 <= 65536:
        y32 = ops.softmax(x32.cuda()).cpu()
        # the reference's own criterion for its fp32 softmax (torch.allclose defaults) plus 1e-6
        assert torch.allclose(y32, torch.softmax(x32, dim=-1), rtol=1e-5, atol=1e-6)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).half()
    b = (0.1 * torch.randn(cols, generator=g)).half()
    y, mean, rstd = ops.layer_norm_fwd(x16.cuda(), w.cuda(), b.cuda(), 1e-5, rm)
    ry, rmean, rrstd = O.layernorm_fwd(x16, w, b, 1e-5)
    assert ln_error_ok(y.cpu(), ln_ref32(x16, w, b, 1e-5))
    assert ((mean.cpu() - rmean).abs() <= 1e-5 * rmean.abs() + 1e-6).all()
    assert ((rstd.cpu() - rrstd).abs() <= 2e-5 * rrstd.abs()).all()
    ops.device_status()


def test_softmax_row_maps_and_extremes():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(60, 512, generator=g).half()
    ref = O.softmax(x)
    for rm in (L.OrderBy(L.Col(12, 5)).TileBy([12, 5]), L.OrderBy(L.Row(60)).TileBy([15], [4]), None):
        assert torch.equal(ops.softmax(x.cuda(), rm).cpu(), ops.softmax(x.cuda()).cpu())
        assert (ops.softmax(x.cuda(), rm).cpu().float() - ref.float()).abs().max().item() <= TOL_F16
    big = torch.full((2, 64), 60000.0).half()
    big[0, 3] = -60000.0
    out = ops.softmax(big.cuda()).cpu()
    assert torch.isfinite(out).all() and abs(out[1].float().sum().item() - 1) < 1e-2
    ninf = torch.full((1, 16), float("-inf")).half()
    ninf[0, 5] = 1.0
    assert ops.softmax(ninf.cuda()).cpu()[0, 5].item() == 1.0
    with pytest.raises(ValueError):
        ops.softmax(x.cuda(), L.OrderBy(L.Row(59)).TileBy([59]))       # map over the wrong number of rows
    assert ops.softmax(torch.zeros(0, 8, dtype=torch.float16).cuda()).shape == (0, 8)


def test_softmax_host_buffers_end_to_end():
    x = softmax_input(64, 8192)
    y = ops.softmax(x.pin_memory())
    assert not y.is_cuda
    assert (y.float() - O.softmax(x).float()).abs().max().item() <= TOL_F16


def test_layernorm_config3_sample_and_full_properties():
    x, gamma, beta = layernorm_input(16384, 8192)
    y, mean, rstd = ops.layer_norm_fwd(x.cuda(), gamma.cuda(), beta.cuda(), 1e-5, ops.row_tiling_layout(16384, 4))
    sel = torch.arange(0, 16384, 41)
    ry, rm, rr = O.layernorm_fwd(x[sel], gamma, beta, 1e-5)
    assert ln_error_ok(y[sel.cuda()].cpu(), ln_ref32(x[sel], gamma, beta, 1e-5))
    assert (y[sel.cuda()].cpu().float() - ry.float()).abs().max().item() <= 2.0 ** -8   # one fp16 ulp at |y| < 8
    assert ((mean[sel.cuda()].cpu() - rm).abs() <= 1e-5 * rm.abs() + 1e-6).all()
    assert ((rstd[sel.cuda()].cpu() - rr).abs() <= 1e-5 * rr.abs()).all()
    # full size: undoing the affine part gives rows of zero mean and unit variance
    z = (y.float() - beta.cuda().float()) / gamma.cuda().float()
    assert z.mean(dim=1).abs().max().item() < 5e-3
    assert (z.var(dim=1, unbiased=False) - 1).abs().max().item() < 2e-2


@pytest.mark.parametrize("rows,cols", [(1151, 8192), (5, 8), (3, 100), (17, 1000), (4, 4096), (2, 16384),
                                       (1, 32768), (6, 777)])
def test_layernorm_shapes(rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    x = (-2.3 + 0.5 * torch.randn(rows, cols, generator=g)).half()      # the reference test's distribution
    w = torch.rand(cols, generator=g).half()
    b = torch.rand(cols, generator=g).half()
    y, mean, rstd = ops.layer_norm_fwd(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    ry, rm, rr = O.layernorm_fwd(x, w, b, 1e-5)
    assert ln_error_ok(y.cpu(), ln_ref32(x, w, b, 1e-5))
    assert ((mean.cpu() - rm).abs() <= 1e-5 * rm.abs() + 1e-6).all()
    assert ((rstd.cpu() - rr).abs() <= 2e-5 * rr.abs()).all()


def test_layernorm_backward_matches_reference_test():
    # test_lego_layer_norm(1151, 8192, fp16) of the reference: atol 1e-2 on y, dx, dw, db
    rows, cols = 1151, 8192
    g = torch.Generator().manual_seed(0)
    w = torch.rand(cols, generator=g).half()
    b = torch.rand(cols, generator=g).half()
    x = (-2.3 + 0.5 * torch.randn(rows, cols, generator=g)).half()
    dy = (0.1 * torch.randn(rows, cols, generator=g)).half()
    xd = x.cuda().requires_grad_(True)
    wd = w.cuda().requires_grad_(True)
    bd = b.cuda().requires_grad_(True)
    y = ops.lego_layer_norm(xd, (cols,), wd, bd, 1e-5)
    y.backward(dy.cuda())
    ry, rm, rr = O.layernorm_fwd(x, w, b, 1e-5)
    rdx, rdw, rdb = O.layernorm_bwd(dy, x, w, rm, rr)
    assert torch.allclose(y.detach().cpu().float(), ry.float(), atol=1e-2, rtol=0)
    assert torch.allclose(xd.grad.cpu().float(), rdx.float(), atol=1e-2, rtol=0)
    # dw / db sum 1151 rows: compare relative to their magnitude
    assert (wd.grad.cpu().float() - rdw.float()).abs().max().item() <= 1e-2 * rdw.float().abs().max().item()
    assert (bd.grad.cpu().float() - rdb.float()).abs().max().item() <= 1e-2 * rdb.float().abs().max().item()
    # deterministic: a second run gives the same bits
    xd.grad = wd.grad = bd.grad = None
    ops.lego_layer_norm(xd, (cols,), wd, bd, 1e-5).backward(dy.cuda())
    y2 = ops.lego_layer_norm(xd, (cols,), wd, bd, 1e-5)
    assert torch.equal(y2, y)


def _check_layernorm_backward(shapes):
    for rows, cols in shapes:
        g = torch.Generator().manual_seed(rows + cols)
        w = torch.rand(cols, generator=g).half()
        b = torch.rand(cols, generator=g).half()
        x = (-2.3 + 0.5 * torch.randn(rows, cols, generator=g)).half()
        dy = (0.1 * torch.randn(rows, cols, generator=g)).half()
        _, mean, rstd = O.layernorm_fwd(x, w, b, 1e-5)
        rdx, rdw, rdb = O.layernorm_bwd(dy, x, w, mean, rstd)
        dx, dw, db = ops.layer_norm_bwd(dy.cuda(), x.cuda(), w.cuda(), mean.cuda(), rstd.cuda())
        assert torch.allclose(dx.cpu().float(), rdx.float(), atol=1e-2, rtol=0), (rows, cols)
        assert (dx.cpu().float() - rdx.float()).abs().max().item() <= 2e-3, (rows, cols)
        assert (dw.cpu().float() - rdw.float()).abs().max().item() <= 1e-2 * rdw.float().abs().max().item(), (rows, cols)
        assert (db.cpu().float() - rdb.float()).abs().max().item() <= 1e-2 * rdb.float().abs().max().item(), (rows, cols)
        again = ops.layer_norm_bwd(dy.cuda(), x.cuda(), w.cuda(), mean.cuda(), rstd.cuda())
        assert all(torch.equal(a, b) for a, b in zip(again, (dx, dw, db))), (rows, cols)
    ops.device_status()


def test_layernorm_backward_shapes_of_both_kernels():
    """dx / dweight / dbias against the oracle for row counts and widths that take the
    ring-fed kernels (16-byte rows of 1 Ki columns or more) and for neighbours that take the
    register kernel (narrower rows, widths that are no multiple of 8); tolerances of the
    reference's own test (atol 1e-2) for dx, 1e-2 of the largest entry for the column sums."""
    # (4 Ki < cols <= 8 Ki: one group of 512 threads with a folding warp; 8 Ki < cols <= 16 Ki the
    # same kernel with 24 or 32 columns per thread and gamma in shared memory, without bounds
    # predicates at exactly 8192, 12288 and 16384 columns; 16 Ki < cols <= 32 Ki a CTA pair per row)
    _check_layernorm_backward(((1152, 8192), (600, 4096), (2048, 2056), (1152, 1032), (1150, 8192), (512, 8200),
                               (300, 1024), (1200, 1024), (600, 16384), (596, 12296), (300, 9000), (128, 16384),
                               (320, 20480), (600, 32768), (296, 16400), (444, 30008), (37, 1000), (300, 777),
                               (64, 4100), (700, 5120), (333, 6152), (400, 12288), (500, 7168)))


def test_layernorm_backward_row_counts_that_are_no_multiple_of_four():
    """The ring-fed kernels fetch the rows' statistics in 16-byte chunks; the rows of a last,
    incomplete chunk get theirs by plain loads.  Every kernel of the family (groups of rows per
    CTA with one row or a block of rows per slot, one group with 8 .. 32 columns per thread, a
    CTA pair per row), with one to three rows left over, few rows and a single row; then the
    same shapes through the register kernel."""
    shapes = ((4095, 4096), (9479, 1024), (9474, 2048), (1201, 1536), (601, 20480), (131, 32768), (203, 3072),
              (31, 8192), (7, 2048), (3, 4096), (1, 1024), (2, 16384), (149, 12288))
    _check_layernorm_backward(shapes)
    ops.tune(lnbwd_min_rows=1 << 30)
    try:
        _check_layernorm_backward(shapes[3:])
    finally:
        ops.tune(lnbwd_min_rows=1)


def test_layernorm_backward_grouped_kernel_with_and_without_folding_warps():
    """Rows of up to 4 Ki columns: one, two and three consumer groups with a folding warp per
    group, and the same shapes with every consumer folding its group's sums itself."""
    shapes = ((600, 4096), (599, 3072), (333, 2560), (1200, 3584), (7, 4096), (150, 2304))
    _check_layernorm_backward(shapes)
    ops.tune(lnbwd_fold_warp=0)
    try:
        _check_layernorm_backward(shapes)
    finally:
        ops.tune(lnbwd_fold_warp=3)


def test_layernorm_errors():
    x = torch.zeros(2, 40000, dtype=torch.float16, device="cuda")
    w = torch.zeros(40000, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="64KB"):
        ops.layer_norm_fwd(x, w, w, 1e-5)
    with pytest.raises(ValueError):
        ops.layer_norm_fwd(x[:, :64].contiguous(), w[:32], w[:32], 1e-5)
