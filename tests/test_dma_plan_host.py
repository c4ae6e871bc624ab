"""The DMA permute's planner, checked on the host: the two tensor maps and the tile-id digits
it produces are executed here with numpy the way the copy engine executes them (a box of a
strided tensor, dimension 0 innermost, dense in shared memory), and the result must equal the
oracle's permute bit for bit.  No GPU needed: this is the index arithmetic of every launch."""
import numpy as np
import pytest

import lego_b200 as L
from lego_b200 import ops
from helpers import spec_of
from oracle import lego_oracle as O


def _run_plan(plan, x_words):
    """Execute a plan on a flat array of elements of plan['elem_bytes'] bytes."""
    out = np.zeros_like(x_words)
    written = np.zeros(x_words.shape, dtype=np.int32)
    ld, st = plan["load"], plan["store"]

    def offsets(side, coord):
        # position in shared memory = sum_d i_d * prod_{e<d} box_e (dimension 0 fastest)
        grids = np.meshgrid(*[np.arange(b, dtype=np.int64) for b in reversed(side["box"])], indexing="ij")
        off = np.zeros(grids[0].shape, dtype=np.int64)
        for k, d in enumerate(reversed(range(len(side["box"])))):
            assert 0 <= coord[d] and coord[d] + side["box"][d] <= side["size"][d], "box leaves the tensor"
            off += (coord[d] + grids[k]) * side["stride"][d]
        return off.reshape(-1)

    box_elems = int(np.prod(ld["box"]))
    assert box_elems == int(np.prod(st["box"])) and box_elems * plan["elem_bytes"] == plan["tile_bytes"]
    n_tiles = 1
    for o in plan["outer"]:
        n_tiles *= o["radix"]
    assert n_tiles == plan["n_tiles"]
    for t in range(n_tiles):
        cl, cs = [0] * len(ld["size"]), [0] * len(st["size"])
        rest = t
        for o in plan["outer"]:
            v = rest % o["radix"]
            rest //= o["radix"]
            cl[o["ld"][0]] += v * o["ld"][1]
            cs[o["st"][0]] += v * o["st"][1]
        smem = x_words[offsets(ld, cl)]
        dst = offsets(st, cs)
        out[dst] = smem
        written[dst] += 1
    assert written.min() == 1 and written.max() == 1, "every output element is written exactly once"
    return out


def _check_pair(src, dst, dtype):
    eb = np.dtype(dtype).itemsize
    n = src.size()
    x = (np.arange(n, dtype=np.int64) * 2654435761 % (1 << (8 * min(eb, 4)))).astype(dtype)
    assert ops.permute_plan(eb, src, dst)[0] == 5
    plan = ops.permute_dma_plan(eb, src, dst)
    assert plan["elem_bytes"] == eb
    assert plan["tile_bytes"] <= 16384 and plan["tile_bytes"] % 16 == 0
    for side in (plan["load"], plan["store"]):
        assert 2 <= len(side["size"]) <= 5 and side["stride"][0] == 1
        assert (side["box"][0] * eb) % 16 == 0 and max(side["box"]) <= 256
        assert all((s * eb) % 16 == 0 for s in side["stride"][1:])
    got = _run_plan(plan, x)
    want = O.permute(x, spec_of(src), spec_of(dst))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [np.uint16, np.uint32, np.uint64])
def test_brick_relayouts_as_tensor_map_pairs(dtype):
    """The reference's brick layouts (benchmarks/cuda/bricks_f3d.py:10-13) on a 48^3 and a
    ragged 32 x 48 x 64 volume, both directions."""
    b = 8
    for dims in [(48, 48, 48), (32, 48, 64)]:
        tiles = [d // b for d in dims]
        normal = L.OrderBy(L.Row(*dims)).TileBy(tiles, [b] * 3)
        bricks = L.OrderBy(L.Row(*tiles), L.Row(b, b, b)).TileBy(tiles, [b] * 3)
        _check_pair(normal, bricks, dtype)
        _check_pair(bricks, normal, dtype)


def test_slabs_are_the_same_permutation_with_a_smaller_top_digit():
    """A volume splits along the outermost brick coordinate; a batched axis swap along the batch.
    The plan of k slabs, run on the first k slabs' elements, gives the first k slabs of the result."""
    b, dims = 8, (48, 32, 64)
    tiles = [d // b for d in dims]
    normal = L.OrderBy(L.Row(*dims)).TileBy(tiles, [b] * 3)
    bricks = L.OrderBy(L.Row(*tiles), L.Row(b, b, b)).TileBy(tiles, [b] * 3)
    assert ops.permute_slab_info(4, normal, bricks) == (6, 8 * 32 * 64)
    p = L.OrderBy(L.Row(6, 40, 24, 4)).GroupBy([(6, 40, 24, 4)])
    q = L.OrderBy(L.RegP([6, 40, 24, 4], [0, 2, 1, 3])).GroupBy([(6, 40, 24, 4)])
    assert ops.permute_slab_info(8, p, q) == (6, 40 * 24 * 4)
    t_src = L.OrderBy(L.Row(256, 256)).TileBy([8, 8], [32, 32])
    t_dst = L.OrderBy(L.Col(256, 256)).TileBy([8, 8], [32, 32])
    assert ops.permute_slab_info(4, t_src, t_dst) is None        # a transpose has no common slow digit
    for src, dst, dtype in ((normal, bricks, np.uint32), (bricks, normal, np.uint32), (p, q, np.uint64)):
        eb = np.dtype(dtype).itemsize
        n_slabs, slab = ops.permute_slab_info(eb, src, dst)
        x = (np.arange(src.size(), dtype=np.int64) * 2654435761 % (1 << 32)).astype(dtype)
        want = O.permute(x, spec_of(src), spec_of(dst))
        for k in (1, 2, n_slabs):
            plan = ops.permute_dma_plan(eb, src, dst, slabs=k)
            assert plan["n_tiles"] * plan["tile_bytes"] == k * slab * eb
            got = _run_plan(plan, x[:k * slab])
            assert np.array_equal(got, want[:k * slab]), (k, dtype)


def test_full_size_brick_plan_shape():
    """384^3 fp32: 16 KiB boxes, loads in rows of 256 bytes, a rank-3 map on either side."""
    n, b = 384, 8
    normal = L.OrderBy(L.Row(n, n, n)).TileBy([n // b] * 3, [b] * 3)
    bricks = L.OrderBy(L.Row(n // b, n // b, n // b), L.Row(b, b, b)).TileBy([n // b] * 3, [b] * 3)
    plan = ops.permute_dma_plan(4, normal, bricks)
    assert plan["tile_bytes"] == 16384 and plan["n_tiles"] * plan["tile_bytes"] == n ** 3 * 4
    assert plan["load"] == {"size": [384, 384, 384], "stride": [1, 384, 384 * 384], "box": [64, 8, 8]}
    assert plan["store"]["box"][0] == 8 and len(plan["store"]["size"]) == 3


def test_other_pairs_with_a_short_common_run():
    # 2-D blocks of 8 x 8 inside a matrix <-> block-major, 16-bit elements (16-byte runs)
    r, c = 128, 512
    a = L.OrderBy(L.Row(r, c)).TileBy([r // 8, c // 8], [8, 8])
    blk = L.OrderBy(L.Row(r // 8, c // 8), L.Row(8, 8)).TileBy([r // 8, c // 8], [8, 8])
    _check_pair(a, blk, np.uint16)
    _check_pair(blk, a, np.uint16)
    # 4-D: swap the two middle axes, innermost run of 4 doubles (32 bytes)
    p = L.OrderBy(L.Row(6, 10, 12, 4)).GroupBy([(6, 10, 12, 4)])
    q = L.OrderBy(L.RegP([6, 10, 12, 4], [0, 2, 1, 3])).GroupBy([(6, 10, 12, 4)])
    _check_pair(p, q, np.uint64)
    _check_pair(q, p, np.uint64)


def test_long_common_runs_on_large_problems():
    """Problems of 4 MiB and more whose common run is a whole 128-byte line or longer also move by
    DMA: a run of more than 256 elements is cut into box rows and a part that continues them."""
    for dims, perm, dtype in (((16, 64, 2048), [1, 0, 2], np.uint32),       # runs of 8 KiB, cut into rows of 1 KiB
                              ((64, 64, 256), [1, 0, 2], np.uint32),        # runs of 1 KiB
                              ((256, 128, 64), [1, 0, 2], np.uint32),       # runs of 256 bytes
                              ((40, 48, 1000), [1, 0, 2], np.uint32),       # 1000 = 5 x 200: rows of 800 bytes
                              ((32, 16, 64, 128), [0, 2, 1, 3], np.uint16)):  # batched, 16-bit, runs of 256 bytes
        src = L.OrderBy(L.Row(*dims)).GroupBy([tuple(dims)])
        dst = L.OrderBy(L.RegP(list(dims), perm)).GroupBy([tuple(dims)])
        eb = np.dtype(dtype).itemsize
        if src.size() * eb < (4 << 20):
            assert ops.permute_plan(eb, src, dst)[0] == 1
            continue
        _check_pair(src, dst, dtype)
        _check_pair(dst, src, dtype)
    ops.tune(permute_dma_long=0)
    try:
        big = (64, 64, 256)
        a = L.OrderBy(L.Row(*big)).GroupBy([big])
        b = L.OrderBy(L.RegP(list(big), [1, 0, 2])).GroupBy([big])
        assert ops.permute_plan(4, a, b)[0] == 1
    finally:
        ops.tune(permute_dma_long=1)


def test_pairs_the_dma_kernel_leaves_to_others():
    n = 256
    src = L.OrderBy(L.Row(n, n)).TileBy([8, 8], [32, 32])
    dst = L.OrderBy(L.Col(n, n)).TileBy([8, 8], [32, 32])
    assert ops.permute_plan(4, src, dst)[0] in (2, 3)          # a transpose: no common run
    with pytest.raises(ValueError):
        ops.permute_dma_plan(4, src, dst)
    # runs of a whole line or more stay with the vector copy
    vol = L.OrderBy(L.Row(8, 12, 128)).TileBy([4, 6, 2], [2, 2, 64])
    brick = L.OrderBy(L.Row(4, 6, 2), L.Row(2, 2, 64)).TileBy([4, 6, 2], [2, 2, 64])
    assert ops.permute_plan(4, vol, brick)[0] == 1
    # switched off: the chunk-tiled kernel takes the bricks
    b, m = 8, 48
    sn = L.OrderBy(L.Row(m, m, m)).TileBy([m // b] * 3, [b] * 3)
    sb = L.OrderBy(L.Row(m // b, m // b, m // b), L.Row(b, b, b)).TileBy([m // b] * 3, [b] * 3)
    ops.tune(permute_dma_tile=0)
    try:
        assert ops.permute_plan(4, sn, sb)[0] == 4
    finally:
        ops.tune(permute_dma_tile=16384)
    assert ops.permute_plan(4, sn, sb)[0] == 5
