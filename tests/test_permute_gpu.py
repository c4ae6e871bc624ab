"""Layout reorganisation on the GPU, through the C ABI, bit-exact against the oracle."""
import numpy as np
import pytest
import torch

import lego_b200 as L
from lego_b200 import ops
from helpers import spec_of
from inputs import transpose_input
from oracle import lego_oracle as O

pytestmark = pytest.mark.gpu


def _bits(x):
    """Flat numpy view of a tensor's elements as unsigned integers of their size."""
    kind = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[x.element_size()]
    return x.contiguous().reshape(-1).view(torch.uint8).numpy().view(kind)


def _check(x, src, dst, order=None, kind=None):
    if kind is not None:
        assert ops.permute_plan(x.element_size(), src, dst, order)[0] == kind
    got = ops.permute(x.cuda(), src, dst, order).cpu()
    exp = O.permute(_bits(x), spec_of(src), spec_of(dst))
    assert np.array_equal(_bits(got), exp)
    return got


def test_config1_transpose_4096_bit_exact():
    n = 4096
    a = transpose_input(n)
    src = L.OrderBy(L.Row(n, n)).TileBy([128, 128], [32, 32])
    dst = L.OrderBy(L.Col(n, n)).TileBy([128, 128], [32, 32])
    order = L.OrderBy(L.Col(128, 128)).TileBy([128, 128])
    for o in (order, None, L.OrderBy(L.Row(128, 128)).TileBy([128, 128])):
        out = ops.permute(a.cuda(), src, dst, o).cpu()
        assert torch.equal(out.reshape(n, n), a.t().contiguous())
    assert torch.equal(ops.transpose(a.cuda()).cpu(), a.t().contiguous())
    # second reading of the configuration: re-layout into tile-major order
    tm = L.OrderBy(L.Col(128, 128), L.Row(32, 32)).TileBy([128, 128], [32, 32])
    got = ops.permute(a.cuda(), src, tm).cpu().reshape(128, 128, 32, 32)
    exp = a.reshape(128, 32, 128, 32).permute(2, 0, 1, 3).contiguous()
    assert torch.equal(got, exp)
    # and back: round trip is the identity
    assert torch.equal(ops.permute(got.cuda(), tm, src).cpu().reshape(n, n), a)


@pytest.mark.parametrize("dtype", [torch.uint8, torch.float16, torch.float32, torch.float64])
def test_tiled_transposes_against_oracle(dtype):
    g = torch.Generator().manual_seed(11)
    for r, c, t in [(96, 160, 32), (256, 128, 64), (64, 64, 16), (128, 384, 32)]:
        x = torch.randint(0, 255, (r * c * torch.empty(0, dtype=dtype).element_size(),), generator=g,
                          dtype=torch.uint8).view(dtype).reshape(r, c)
        src = L.OrderBy(L.Row(r, c)).TileBy([r // t, c // t], [t, t])
        dst = L.OrderBy(L.Col(r, c)).TileBy([r // t, c // t], [t, t])
        order = L.OrderBy(L.Col(r // t, c // t)).TileBy([r // t, c // t])
        got = _check(x, src, dst, order)
        assert torch.equal(got.reshape(c, r).view(torch.uint8), x.t().contiguous().view(torch.uint8))
        _check(x, src, dst, None)


def test_three_level_layouts_of_the_mlir_programs():
    n = 256
    x = torch.arange(n * n, dtype=torch.float32).reshape(n, n)       # the reference fills with float(i)
    a = L.OrderBy(L.Row(n, n)).TileBy([8, 8], [4, 1], [8, 32])
    b = L.OrderBy(L.Col(n, n)).TileBy([8, 8], [4, 1], [8, 32])
    got = _check(x, a, b)
    assert torch.equal(got.reshape(n, n), x.t().contiguous())


def test_batched_and_brick_permutations():
    g = torch.Generator().manual_seed(12)
    x = torch.randn(6 * 64 * 128, generator=g)
    # 3-D brick re-layout (row-major volume -> 2x2x4 bricks), a pure gather
    vol = L.OrderBy(L.Row(8, 12, 128)).TileBy([4, 6, 2], [2, 2, 64])
    brick = L.OrderBy(L.Row(4, 6, 2), L.Row(2, 2, 64)).TileBy([4, 6, 2], [2, 2, 64])
    _check(x[:8 * 12 * 128], vol, brick, kind=1)
    # batched transpose: (b, i, j) -> (b, j, i)
    src = L.OrderBy(L.Row(6, 64, 128)).GroupBy([(6, 64, 128)])
    dst = L.OrderBy(L.RegP([6, 64, 128], [0, 2, 1])).GroupBy([(6, 64, 128)])
    got = _check(x, src, dst, kind=3)
    assert torch.equal(got.reshape(6, 128, 64), x.reshape(6, 64, 128).transpose(1, 2).contiguous())


def test_staged_and_ragged_layouts():
    g = torch.Generator().manual_seed(13)
    x = torch.randn(6, generator=g)
    a = L.OrderBy(L.Col(3, 2)).GroupBy([(2, 3)])
    b = L.OrderBy(L.Row(2, 3)).GroupBy([(2, 3)])
    _check(x, a, b, kind=0)
    y = torch.randn(120, generator=g).half()
    c = L.OrderBy(L.Col(6, 4), L.Row(5)).GroupBy([(4, 5, 6)])
    d = L.OrderBy(L.Row(4, 5, 6)).GroupBy([(4, 5, 6)])
    _check(y, c, d, kind=0)
    # odd sizes: no 16-byte structure anywhere -> scalar gather
    z = torch.randn(7 * 9, generator=g)
    e = L.OrderBy(L.Row(7, 9)).TileBy([7, 9])
    f = L.OrderBy(L.Col(7, 9)).TileBy([7, 9])
    got = _check(z, e, f, kind=1)
    assert torch.equal(got.reshape(9, 7), z.reshape(7, 9).t().contiguous())
    one = torch.randn(1)
    s = L.OrderBy(L.Row(1)).TileBy([1])
    assert torch.equal(ops.permute(one.cuda(), s, s).cpu(), one)


def test_argument_errors():
    x = torch.zeros(64, device="cuda")
    a = L.OrderBy(L.Row(8, 8)).TileBy([8, 8])
    with pytest.raises(ValueError):
        ops.permute(x, a, L.OrderBy(L.Row(4, 16)).TileBy([4, 16]))
    with pytest.raises(ValueError):
        ops.permute(x[:32], a, a)
    with pytest.raises(ValueError):
        ops.permute(x, a, a, out=x)        # in place is refused


@pytest.mark.parametrize("dtype,n,t", [(torch.float32, 1024, 32), (torch.float16, 512, 64), (torch.float64, 256, 16)])
def test_tile_ranges_assemble_the_whole_reorganisation(dtype, n, t):
    """One GPU of several moves a contiguous range of tile_order ids.  With the column-major
    tile order a range is a slab of output rows: four ragged ranges written into one buffer
    give the whole transpose, and a single range touches nothing outside its slab."""
    from lego_b200 import shard
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, n, generator=g).to(dtype)
    nt = n // t
    src = L.OrderBy(L.Row(n, n)).TileBy([nt, nt], [t, t])
    dst = L.OrderBy(L.Col(n, n)).TileBy([nt, nt], [t, t])
    order = L.OrderBy(L.Col(nt, nt)).TileBy([nt, nt])
    xd = x.cuda()
    out = torch.full_like(xd, 7.0)
    for rank in range(3):
        r0, r1 = shard.shard_transpose(n, n, rank, 3, t)          # output rows of this rank
        ops.permute(xd, src, dst, order, out=out, tiles=(r0 // t * nt, (r1 - r0) // t * nt))
        done = out.reshape(n, n)[:r1].cpu()
        assert torch.equal(done, x.t().contiguous()[:r1])
        assert bool((out.reshape(n, n)[r1:] == 7.0).all())
    ops.device_status()
    empty = torch.full_like(xd, 7.0)
    ops.permute(xd, src, dst, order, out=empty, tiles=(5, 0))
    assert bool((empty == 7.0).all())
    with pytest.raises(ValueError):
        ops.permute(xd, src, dst, order, out=out, tiles=(nt * nt - 1, 2))     # past the last tile
    with pytest.raises(ValueError):
        ops.permute(xd, src, dst, None, out=out, tiles=(0, 1))                # a range needs a tile order


@pytest.mark.parametrize("kernel", [5, 4])
def test_brick_relayout_384_cubed(golden, kernel):
    """The reference's brick layouts (benchmarks/cuda/bricks_f3d.py:10-13): a 384^3 fp32
    volume from row-major order into 8^3 bricks and back, each as ONE permute call, on the
    DMA kernel (two tensor maps, no thread touches the data) and on the chunk-tiled kernel.
    Checked three ways: against the reference's own index vectors for both layouts (golden
    file), against the oracle on a 96^3 volume, and at full size against the same re-layout
    written as reshape + transpose."""
    n, b = 384, 8
    normal = L.OrderBy(L.Row(n, n, n)).TileBy([n // b] * 3, [b] * 3)
    bricks = L.OrderBy(L.Row(n // b, n // b, n // b), L.Row(b, b, b)).TileBy([n // b] * 3, [b] * 3)
    ops.tune(permute_dma_tile=16384 if kernel == 5 else 0)
    try:
        assert ops.permute_plan(4, normal, bricks)[0] == kernel and ops.permute_plan(4, bricks, normal)[0] == kernel
        x = torch.rand(n, n, n, generator=torch.Generator().manual_seed(8))
        xd = x.cuda()
        out = ops.permute(xd, normal, bricks)
        ops.device_status()
        want = x.reshape(n // b, b, n // b, b, n // b, b).permute(0, 2, 4, 1, 3, 5).contiguous()
        assert torch.equal(out.cpu().reshape(-1), want.reshape(-1))
        assert torch.equal(ops.permute(out, bricks, normal).cpu(), x)          # and back
        ops.device_status()
        # the reference's vectors: the element with logical index (bx, by, bz, i, j, k), i.e. voxel
        # (8 bx + i, 8 by + j, 8 bz + k), sits at normal(idx) before the call and at bricks(idx) after
        for name, buf in (("bricks_normal_384", x), ("bricks_384", out.cpu())):
            gl = golden["layouts"][name]
            bx, by, bz, i, j, k = (torch.from_numpy(v) for v in np.unravel_index(np.asarray(gl["ids"]), gl["dims"]))
            voxel = x[bx * b + i, by * b + j, bz * b + k]
            assert torch.equal(buf.reshape(-1)[torch.tensor(gl["apply"])], voxel), name
        # oracle on a volume it handles in seconds, several element sizes
        m = 96
        sn = L.OrderBy(L.Row(m, m, m)).TileBy([m // b] * 3, [b] * 3)
        sb = L.OrderBy(L.Row(m // b, m // b, m // b), L.Row(b, b, b)).TileBy([m // b] * 3, [b] * 3)
        for dtype in (torch.float16, torch.float32, torch.float64):
            y = torch.rand(m, m, m, generator=torch.Generator().manual_seed(9)).to(dtype)
            _check(y, sn, sb, kind=kernel)
            _check(y, sb, sn, kind=kernel)
        ops.device_status()
    finally:
        ops.tune(permute_dma_tile=16384)


def test_dma_permute_other_shapes_and_sizes():
    """Pairs with a short common run on the DMA kernel: blocks of a matrix, a swap of the
    two middle axes of a 4-D array, a ragged volume; 2-, 8- and 16-byte elements; a grid
    smaller than the machine and one many tiles deep; repeated back-to-back launches."""
    g = torch.Generator().manual_seed(21)
    r, c = 256, 1024
    a = L.OrderBy(L.Row(r, c)).TileBy([r // 8, c // 8], [8, 8])
    blk = L.OrderBy(L.Row(r // 8, c // 8), L.Row(8, 8)).TileBy([r // 8, c // 8], [8, 8])
    x = torch.randn(r, c, generator=g).half()
    _check(x, a, blk, kind=5)
    _check(x, blk, a, kind=5)
    p = L.OrderBy(L.Row(12, 40, 24, 4)).GroupBy([(12, 40, 24, 4)])
    q = L.OrderBy(L.RegP([12, 40, 24, 4], [0, 2, 1, 3])).GroupBy([(12, 40, 24, 4)])
    y = torch.randn(12, 40, 24, 4, generator=g, dtype=torch.float64)
    got = _check(y, p, q, kind=5)
    assert torch.equal(got.reshape(12, 24, 40, 4), y.transpose(1, 2).contiguous())
    _check(y, q, p, kind=5)
    # 16-byte elements (complex128): runs of two elements, written into the maps as four 8-byte ones
    z = torch.randn(16, 24, 32, 2, generator=g, dtype=torch.float64).to(torch.complex128)
    pz = L.OrderBy(L.Row(16, 24, 32, 2)).GroupBy([(16, 24, 32, 2)])
    qz = L.OrderBy(L.RegP([16, 24, 32, 2], [0, 2, 1, 3])).GroupBy([(16, 24, 32, 2)])
    assert ops.permute_plan(16, pz, qz)[0] == 5
    gz = ops.permute(z.cuda(), pz, qz).cpu()
    assert torch.equal(torch.view_as_real(gz.reshape(16, 32, 24, 2)),
                       torch.view_as_real(z.transpose(1, 2).contiguous()))
    # ragged volume, many launches in a row (ring slots and barriers start afresh each time)
    dims, b = (64, 96, 160), 8
    tiles = [d // b for d in dims]
    sn = L.OrderBy(L.Row(*dims)).TileBy(tiles, [b] * 3)
    sb = L.OrderBy(L.Row(*tiles), L.Row(b, b, b)).TileBy(tiles, [b] * 3)
    v = torch.randn(*dims, generator=g)
    vd = v.cuda()
    want = v.reshape(tiles[0], b, tiles[1], b, tiles[2], b).permute(0, 2, 4, 1, 3, 5).contiguous().reshape(-1)
    for _ in range(5):
        out = ops.permute(vd, sn, sb)
        back = ops.permute(out, sb, sn)
    assert torch.equal(out.cpu().reshape(-1), want) and torch.equal(back.cpu(), v)
    ops.device_status()


def test_dma_permute_long_runs():
    """Large problems whose common run is a whole line or more (batched permutations, axis swaps
    with long innermost axes) also move by DMA; same results as the vector copy they replace."""
    g = torch.Generator().manual_seed(31)
    for dims, perm, dtype in (((16, 64, 2048), [1, 0, 2], torch.float32), ((256, 128, 64), [1, 0, 2], torch.float32),
                              ((40, 48, 1000), [1, 0, 2], torch.float32), ((32, 16, 64, 128), [0, 2, 1, 3], torch.float16)):
        src = L.OrderBy(L.Row(*dims)).GroupBy([tuple(dims)])
        dst = L.OrderBy(L.RegP(list(dims), perm)).GroupBy([tuple(dims)])
        x = torch.randn(*dims, generator=g).to(dtype)
        assert ops.permute_plan(x.element_size(), src, dst)[0] == 5
        got = ops.permute(x.cuda(), src, dst).cpu()
        assert torch.equal(got.reshape(-1), x.permute(*perm).contiguous().reshape(-1)), dims
        ops.tune(permute_dma_long=0)
        try:
            assert ops.permute_plan(x.element_size(), src, dst)[0] == 1
            assert torch.equal(ops.permute(x.cuda(), src, dst).cpu(), got), dims
        finally:
            ops.tune(permute_dma_long=1)
        assert torch.equal(ops.permute(got.cuda(), dst, src).cpu().reshape(-1), x.reshape(-1)), dims     # and back
    ops.device_status()
