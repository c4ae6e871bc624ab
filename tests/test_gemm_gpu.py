"""fp16 GEMM and grouped GEMM on tcgen05, through the C ABI, against the oracle
(fp32 CPU product of the fp16 inputs).  Tolerance: relative Frobenius error
<= 1e-3; the reference's own allclose(atol=1e-2) checks are repeated too."""
import math

import numpy as np
import pytest
import torch

import lego_b200 as L
from lego_b200 import ops
from inputs import gemm_input, grouped_input, grouped_sizes
from oracle import lego_oracle as O

pytestmark = pytest.mark.gpu

REL_FRO = 1e-3


def rel_fro(got, ref):
    return ((got.float() - ref).norm() / ref.norm()).item()


def test_matmul_512_like_the_reference_check():
    torch.manual_seed(0)
    a = torch.randn(512, 512).half()
    b = torch.randn(512, 512).half()
    c = ops.matmul(a.cuda(), b.cuda()).cpu()
    ops.device_status()
    ref = O.matmul(a, b)
    assert rel_fro(c, ref) <= REL_FRO
    assert torch.allclose(c.float(), ref.half().float(), atol=1e-2 * 8, rtol=1e-2)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_operand_layout_variants(ta, tb):
    g = torch.Generator().manual_seed(7 + 2 * ta + tb)
    m, n, k = 384, 768, 320
    a = (torch.randn(m, k, generator=g) / math.sqrt(k)).half()
    b = (torch.randn(k, n, generator=g) / math.sqrt(k)).half()
    ad = a.t().contiguous().cuda().t() if ta else a.cuda()       # .T view of a [K, M] buffer
    bd = b.t().contiguous().cuda().t() if tb else b.cuda()
    c = ops.matmul(ad, bd).cpu()
    ops.device_status()
    assert rel_fro(c, O.matmul(a, b)) <= REL_FRO


def test_edges_activation_and_tile_orders():
    g = torch.Generator().manual_seed(9)
    for m, n, k in [(128, 256, 64), (1, 8, 8), (130, 264, 72), (1000, 520, 136), (256, 512, 4096)]:
        a = (torch.randn(m, k, generator=g) / math.sqrt(k)).half()
        b = (torch.randn(k, n, generator=g) / math.sqrt(k)).half()
        ref = O.matmul(a, b)
        c = ops.matmul(a.cuda(), b.cuda()).cpu()
        ops.device_status()
        assert rel_fro(c, ref) <= REL_FRO, (m, n, k)
    a, b = gemm_input(1024, 1024, 512)
    ref = O.matmul(a, b, "leaky_relu")
    assert rel_fro(ops.matmul(a.cuda(), b.cuda(), activation="leaky_relu").cpu(), ref) <= REL_FRO
    base = ops.matmul(a.cuda(), b.cuda())
    for order in (L.OrderBy(L.Row(8, 4)).TileBy([8, 4]), L.OrderBy(L.Col(8, 4)).TileBy([8, 4]),
                  ops.grouped_swizzle_layout(8, 4, 2)):
        assert torch.equal(ops.matmul(a.cuda(), b.cuda(), tile_order=order), base)   # order never changes bits
    with pytest.raises(ValueError):
        ops.matmul(a.cuda(), b.cuda(), tile_order=L.OrderBy(L.Row(4, 4)).TileBy([4, 4]))
    with pytest.raises(ValueError):
        ops.matmul(a.cuda()[:, :100].contiguous(), b.cuda()[:100].contiguous())     # K % 8 != 0
    ops.device_status()


def test_config4_8192_cubed():
    a, b = gemm_input()
    ad, bd = a.cuda(), b.cuda()
    c = ops.matmul(ad, bd)
    ops.device_status()
    # oracle on sampled rows: C[r, :] = A[r, :] @ B in fp32 on the CPU
    rows = torch.tensor([0, 1, 127, 128, 4095, 5000, 8191])
    ref = a[rows].float() @ b.float()
    assert rel_fro(c[rows.cuda()].cpu(), ref) <= REL_FRO
    # full size, size-independent property: (A B) v == A (B v) for a random v, in fp64 on the device
    v = torch.randn(8192, 1, dtype=torch.float64, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    lhs = c.double() @ v
    rhs = ad.double() @ (bd.double() @ v)
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= REL_FRO


def test_grouped_reference_sizes_and_config5():
    torch.manual_seed(0)
    sizes = [1024, 512, 256, 128]
    A = [torch.rand(s, s).half() for s in sizes]
    B = [torch.rand(s, s).half() for s in sizes]
    out = ops.lego_group_gemm_fn([t.cuda() for t in A], [t.cuda() for t in B])
    ops.device_status()
    for c, r in zip(out, O.grouped_matmul(A, B)):
        assert rel_fro(c.cpu(), r) <= REL_FRO
    # config 5 shapes with M shrunk 8x for the CPU oracle; then full size with the product property
    A, B = grouped_input(scale_rows=8)
    out = ops.lego_group_gemm_fn([t.cuda() for t in A], [t.cuda() for t in B])
    ops.device_status()
    for c, r in zip(out, O.grouped_matmul(A, B)):
        assert rel_fro(c.cpu(), r) <= REL_FRO
    sizes5, _ = grouped_sizes()
    assert sizes5[0] == (2048, 1024, 4096) and sizes5[13] == (4096, 4096, 4096)
    A, B = grouped_input()
    Ad, Bd = [t.cuda() for t in A], [t.cuda() for t in B]
    orders = [L.OrderBy(L.Row(-(-a.shape[0] // 128), -(-b.shape[1] // 256))).TileBy(
        [-(-a.shape[0] // 128), -(-b.shape[1] // 256)]) for a, b in zip(A, B)]
    out = ops.lego_group_gemm_fn(Ad, Bd, orders)
    ops.device_status()
    gen = torch.Generator("cuda").manual_seed(2)
    for c, a, b in zip(out, Ad, Bd):
        v = torch.randn(b.shape[1], 1, dtype=torch.float64, device="cuda", generator=gen)
        rhs = a.double() @ (b.double() @ v)
        assert (((c.double() @ v) - rhs).norm() / rhs.norm()).item() <= REL_FRO
    assert ops.lego_group_gemm_fn([], []) == []


def test_narrow_outputs_next_to_wide_ones():
    """Problems narrower than one 256-column tile stage fewer epilogue chunks than they
    skip; mixed with wide problems in one launch they once had their staging buffers
    overwritten before the pending TMA store had read them."""
    g = torch.Generator().manual_seed(31)
    for shapes in ([(128, 256, 64), (128, 64, 64)], [(1, 8, 8)] * 3, [(128, 128, 64)] * 2,
                   [(640, 512, 1024), (1, 8, 8)], [(128, 256, 64), (1, 8, 8), (128, 256, 64)],
                   [(384, 512, 64), (128, 8, 8), (256, 192, 128)]):
        A = [(torch.randn(m, k, generator=g) / 16).half() for m, n, k in shapes]
        B = [(torch.randn(k, n, generator=g) / 16).half() for m, n, k in shapes]
        for _ in range(3):
            out = ops.lego_group_gemm_fn([t.cuda() for t in A], [t.cuda() for t in B])
            ops.device_status()
            for c, r in zip(out, O.grouped_matmul(A, B)):
                assert rel_fro(c.cpu(), r) <= REL_FRO, shapes
    for m, n, k in [(256, 128, 64), (512, 64, 128), (128, 192, 320), (1024, 8, 8)]:
        a = (torch.randn(m, k, generator=g) / 16).half()
        b = (torch.randn(k, n, generator=g) / 16).half()
        for _ in range(3):
            assert rel_fro(ops.matmul(a.cuda(), b.cuda()).cpu(), O.matmul(a, b)) <= REL_FRO, (m, n, k)
    ops.device_status()


def _e5m2_pair(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).half().to(torch.float8_e5m2)
    b = torch.randn(k, n, generator=g).half().to(torch.float8_e5m2)
    return a, b


def test_e5m2_512_like_the_reference_check():
    # the TORCH_HAS_FP8 branch of the reference's check: randn -> e5m2, allclose(atol=0.125)
    # against the fp16 product of the same 8-bit values
    a, b = _e5m2_pair(512, 512, 512, 0)
    c = ops.matmul(a.cuda(), b.cuda()).cpu()
    ops.device_status()
    assert c.dtype == torch.float16
    ref = O.matmul(a.float(), b.float())
    assert rel_fro(c, ref) <= REL_FRO
    assert torch.allclose(c.float(), ref.half().float(), atol=0.125, rtol=0)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_e5m2_operand_layouts_edges_and_both_kernels(ta, tb):
    # (384, 768, 320): even tile rows -> CTA pairs, K not a multiple of the 128-wide stage;
    # (400, 528, 144): ragged M and N, odd tile count -> one CTA per tile
    for m, n, k in ((384, 768, 320), (400, 528, 144), (128, 256, 4096)):
        a, b = _e5m2_pair(m, n, k, 31 + 2 * ta + tb + m)
        ad = a.cuda().t().contiguous().t() if ta else a.cuda()
        bd = b.cuda().t().contiguous().t() if tb else b.cuda()
        c = ops.matmul(ad, bd).cpu()
        ops.device_status()
        ref = O.matmul(a.float(), b.float())
        assert rel_fro(c, ref) <= REL_FRO, (ta, tb, m, n, k)
    a, b = _e5m2_pair(256, 256, 256, 77)
    got = ops.matmul(a.cuda(), b.cuda(), activation="leaky_relu").cpu()
    assert rel_fro(got, O.matmul(a.float(), b.float(), "leaky_relu")) <= REL_FRO
    with pytest.raises(ValueError):
        ops.matmul(a.cuda(), b.cuda().half())                      # mixed operand types
    with pytest.raises(ValueError):
        ops.matmul(a.cuda()[:, :200].contiguous(), b.cuda()[:200])  # K = 200 is not a multiple of 16


def test_stream_k_tail_matches_the_oracle_and_is_deterministic():
    """Shapes whose tile count is not a multiple of the SM pairs: the partial last wave is
    cut along K, partial accumulators go through the workspace and the owner adds them.
    256 x 1536 x 4096 is six pair tiles on 74 pairs, so every tile is shared by about a
    dozen workers (an owner adds up to eleven peers); 1024 x 8192 x 2048 is the M/8 slab of
    the benchmark GEMM's shape with a shorter K (128 pair tiles = 1.73 waves)."""
    g = torch.Generator().manual_seed(41)
    ops.tune(gemm_streamk=2)                      # split whenever a partial wave exists
    for m, n, k in [(256, 1536, 4096), (1024, 8192, 2048), (2304, 2304, 1024), (200, 520, 1096)]:
        a = (torch.randn(m, k, generator=g) / math.sqrt(k)).half()
        b = (torch.randn(k, n, generator=g) / math.sqrt(k)).half()
        ref = O.matmul(a, b)
        ad, bd = a.cuda(), b.cuda()
        first = ops.matmul(ad, bd)
        ops.device_status()
        assert rel_fro(first.cpu(), ref) <= REL_FRO, (m, n, k)
        for _ in range(3):                       # flags are left clean, results repeat bit for bit
            assert torch.equal(ops.matmul(ad, bd), first), (m, n, k)
        ops.device_status()
        ops.tune(gemm_streamk=0)
        try:
            whole = ops.matmul(ad, bd)
        finally:
            ops.tune(gemm_streamk=2)
        ops.device_status()
        assert rel_fro(whole.cpu(), ref) <= REL_FRO
        # fp32 partial sums added in another order: equal up to the last fp16 bit
        assert (first.float() - whole.float()).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())
    ops.tune(gemm_streamk=0)


@pytest.mark.parametrize("streamk,lag", [(0, 0), (0, 3), (2, 4), (2, 1)])
def test_tall_pair_tiles_512x256(streamk, lag):
    """The 512 x 256 pair tile (two 256-row accumulator blocks sharing one B tile), with and
    without the stream-K tail and with several leads of block 0 over block 1 (including k
    loops shorter than twice the lead), fp16 and e5m2, all operand layouts of one shape."""
    ops.tune(gemm_blocks=2, gemm_streamk=streamk, gemm_lag=lag)
    try:
        g = torch.Generator().manual_seed(43)
        for m, n, k in [(512, 256, 64), (1024, 768, 320), (1536, 2304, 1024), (1000, 520, 136)]:
            a = (torch.randn(m, k, generator=g) / math.sqrt(k)).half()
            b = (torch.randn(k, n, generator=g) / math.sqrt(k)).half()
            order = L.OrderBy(L.Col(-(-m // 128), -(-n // 256))).TileBy([-(-m // 128), -(-n // 256)])
            c = ops.matmul(a.cuda(), b.cuda(), tile_order=order)
            ops.device_status()
            assert rel_fro(c.cpu(), O.matmul(a, b)) <= REL_FRO, (m, n, k)
        for ta, tb in [(0, 1), (1, 0), (1, 1)]:
            a = (torch.randn(1024, 320, generator=g) / 16).half()
            b = (torch.randn(320, 768, generator=g) / 16).half()
            ad = a.t().contiguous().cuda().t() if ta else a.cuda()
            bd = b.t().contiguous().cuda().t() if tb else b.cuda()
            assert rel_fro(ops.matmul(ad, bd).cpu(), O.matmul(a, b)) <= REL_FRO, (ta, tb)
        a8, b8 = _e5m2_pair(1024, 512, 384, 5)
        assert rel_fro(ops.matmul(a8.cuda(), b8.cuda()).cpu(), O.matmul(a8.float(), b8.float())) <= REL_FRO
        a, b = gemm_input(4096, 4096, 4096)
        c = ops.matmul(a.cuda(), b.cuda())
        ops.device_status()
        rows = torch.tensor([0, 127, 128, 383, 511, 512, 2049, 4095])
        assert rel_fro(c[rows.cuda()].cpu(), a[rows].float() @ b.float()) <= REL_FRO
    finally:
        ops.tune(gemm_blocks=0, gemm_streamk=0, gemm_lag=4)


def test_grouped_gemm_refuses_stream_capture():
    """The grouped entry points upload their problem table from host memory that dies with
    the call: inside a stream capture they return LEGO_ERR_UNSUPPORTED and enqueue nothing."""
    a = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(64, 256, dtype=torch.float16, device="cuda")
    ops.lego_group_gemm_fn([a], [b])            # set-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        with pytest.raises(ValueError, match="no kernel"):
            ops.lego_group_gemm_fn([a], [b])
        c = ops.matmul(a, b)                     # a plain GEMM is capturable
    graph.replay()
    torch.cuda.synchronize()
    assert c.abs().max().item() == 0
    ops.device_status()


def test_grouped_column_major_orders_take_pair_and_tall_tiles():
    """Per-group column-major tile orders: with a multiple of four tile rows in every group
    the persistent CTA pairs work on 512 x 256 tiles, with a multiple of two on 256 x 256,
    and one group with an odd tile count sends the whole call to one CTA per tile.  Same
    bits in all three (every output element is one k-ordered accumulation)."""
    g = torch.Generator().manual_seed(47)
    for shapes in ([(512, 512, 320), (1024, 256, 192), (512, 768, 64)],       # 4 | tile rows everywhere
                   [(512, 512, 320), (256, 256, 192), (768, 512, 64)],       # 2 | tile rows
                   [(512, 512, 320), (384, 256, 192)]):                      # three tile rows in a group
        A = [(torch.randn(m, k, generator=g) / 16).half() for m, n, k in shapes]
        B = [(torch.randn(k, n, generator=g) / 16).half() for m, n, k in shapes]
        orders = [L.OrderBy(L.Col(m // 128, -(-n // 256))).TileBy([m // 128, -(-n // 256)]) for m, n, k in shapes]
        Ad, Bd = [t.cuda() for t in A], [t.cuda() for t in B]
        out = ops.lego_group_gemm_fn(Ad, Bd, orders)
        ops.device_status()
        plain = ops.lego_group_gemm_fn(Ad, Bd)
        for c, p, r in zip(out, plain, O.grouped_matmul(A, B)):
            assert rel_fro(c.cpu(), r) <= REL_FRO, shapes
            assert torch.equal(c, p), shapes
    # the blocks one rank of eight gets from the 16-group configuration (512-row blocks of several groups)
    from lego_b200 import shard
    sizes, _ = grouped_sizes()
    A, B = grouped_input()
    mine = shard.pack_grouped_gemm_blocks(sizes, 8, 512)[3]
    Ad = [A[gi][b:e].cuda() for gi, b, e in mine]
    Bd = [B[gi].cuda() for gi, b, e in mine]
    orders = [L.OrderBy(L.Col((e - b) // 128, sizes[gi][1] // 256)).TileBy([(e - b) // 128, sizes[gi][1] // 256])
              for gi, b, e in mine]
    out = ops.lego_group_gemm_fn(Ad, Bd, orders)
    ops.device_status()
    for c, (gi, b, e) in zip(out, mine):
        ref = A[gi][b:b + 64].float() @ B[gi].float()
        assert rel_fro(c[:64].cpu(), ref) <= REL_FRO
