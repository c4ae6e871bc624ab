"""Host-side logic of the product (no GPU): the numeric layout algebra, the
lowering, and the native constant folding, against the reference's golden
vectors and printed strings."""
import numpy as np
import pytest

import lego_b200 as L
from lego_b200 import ops
from lego_b200.lowering import fold, lower
from helpers import (build_layout, eval_c_string, eval_reference_string, genp_kind_of, golden_spec, same_structure,
                     spec_of, unravel)
from oracle import lego_oracle as O


def test_apply_and_inv_match_reference(golden):
    for name, g in golden["layouts"].items():
        lay = build_layout(g["src"])
        assert list(lay.dims()) == g["dims"], name
        assert same_structure(spec_of(lay), g["spec"]), name
        got = lay.apply(*unravel(g["ids"], g["dims"]))
        assert np.array_equal(np.broadcast_to(got, (len(g["ids"]),)), np.asarray(g["apply"])), name
        inv = lay.inv(np.asarray(g["inv_flat"], dtype=np.int64))
        exp = np.asarray(g["inv"], dtype=np.int64).reshape(len(g["inv_flat"]), len(g["dims"]))
        for k in range(len(g["dims"])):
            assert np.array_equal(np.broadcast_to(inv[k], exp[:, k].shape), exp[:, k]), (name, k)
        # scalar calls give plain ints, like the reference's numeric path
        assert lay.apply(*[int(v[0]) for v in unravel(g["ids"][:1], g["dims"])]) == g["apply"][0]


def test_fold_matches_reference(golden):
    staged = set()
    for name, g in golden["layouts"].items():
        lay = build_layout(g["src"])
        f = fold(lay)
        assert f.size == int(np.prod(g["dims"]))
        if not f.foldable:
            staged.add(name)
            continue
        idx = unravel(g["ids"], g["dims"])
        acc = np.zeros(len(g["ids"]), dtype=np.int64)
        for t in f.terms:
            acc += ((idx[t.src] // t.div) % t.mod) * t.stride
        assert np.array_equal(acc, np.asarray(g["apply"])), name
        # the same terms invert the map
        flat = np.asarray(g["apply"], dtype=np.int64)
        for k in range(len(g["dims"])):
            back = sum(((flat // t.stride) % t.mod) * t.div for t in f.terms if t.src == k)
            assert np.array_equal(np.broadcast_to(back, idx[k].shape), idx[k]), (name, k)
    # cuts that no digit split can realise, and GenP blocks, stay on the staged interpreter
    assert staged == {"misaligned_col", "misaligned_row", "misaligned_two"} | {n for n in golden["layouts"]
                                                                             if n.startswith("genp_")}


def test_fold_examples():
    f = fold(L.OrderBy(L.Col(128, 128), L.Row(32, 32)).TileBy([128, 128], [32, 32]))
    assert [(t.src, t.stride) for t in f.terms] == [(1, 131072), (0, 1024), (2, 32), (3, 1)]
    f = fold(ops.grouped_swizzle_layout(64, 32, 8))
    assert [(t.src, t.div, t.mod, t.stride) for t in f.terms] == [(0, 8, 8, 256), (1, 1, 32, 8), (0, 1, 8, 1)]


def test_getitem_matches_printed_strings(golden):
    sizes = dict(M=256, N=512, K=192, BM=64, BN=128, BK=32, pid_m=3, pid_n=2, k=5,
                 n_rows=37, n_cols=64, BLOCK_SIZE=64, row_idx=11, pid=7, BLOCK_SIZE_N=128,
                 gm=256, gn=512, gk=192, BLOCK_SIZE_M=64, BLOCK_SIZE_K=32, tile_m_idx=3,
                 tile_n_idx=2, kk=5, i=1, j=0, w=1, q=1)
    sizes_ln = dict(sizes, N=512, M=24, k=2)
    checked = 0
    for name, s in golden["strings"].items():
        if "layout" not in s:
            continue
        env = sizes_ln if name.startswith("layernorm") else sizes
        if name == "graphene":
            env = dict(i=1, j=0, k=1, w=1, q=1)
        lay = build_layout(s["layout"], env)
        key = []
        for item in s["key"]:
            if item == ":":
                key.append(slice(None))
            elif item.startswith("arange("):
                key.append(np.arange(env[item[7:-1]], dtype=np.int64))   # an expression, not a slice
            elif item.isdigit():
                key.append(int(item))
            else:
                key.append(env[item])
        got = np.asarray(lay[tuple(key)])
        exp = np.asarray(eval_reference_string(s["text"], env))
        if s.get("flat"):
            got, exp = got.ravel(), exp.ravel()
        assert got.shape == exp.shape and np.array_equal(got, exp), name
        checked += 1
    assert checked >= 15


def test_swizzle_inverse_matches_printed_strings(golden):
    s = golden["strings"]
    for npm, npn, gm in [(64, 32, 8), (16, 4, 8), (4, 8, 8)]:
        pid = np.arange(npm * npn, dtype=np.int64)
        env = {"pid": pid, "num_pid_m": npm, "num_pid_n": npn, "GM": gm}
        lay = ops.grouped_swizzle_layout(npm, npn, gm)
        pm, pn = lay.inv(pid)
        assert np.array_equal(pm, eval_reference_string(s["matmul_pid_m"]["text"], env))
        assert np.array_equal(pn, eval_reference_string(s["matmul_pid_n"]["text"], env))


def test_errors_follow_the_reference():
    lay = L.OrderBy(L.Row(4, 4)).TileBy([2, 2], [2, 2])
    with pytest.raises(ValueError):
        lay.apply(1, 2, 3)                      # lego/lego.py:394-396
    with pytest.raises(ValueError):
        L.flatten_index((1, 2), (3,))           # lego/lego.py:99-100
    with pytest.raises(ValueError):
        L.Row(4, 4).apply((1,))                 # lego/lego.py:216-217
    with pytest.raises(ValueError):
        L.OrderBy(L.Row(2), L.Row(3)).apply((1,))   # lego/lego.py:294-296
    with pytest.raises(ValueError):
        L.RegP([2, 2], [0, 0])
    # the grouped swizzle for 10 tile rows in groups of 8 is not a bijection: rejected at lowering
    with pytest.raises(ValueError, match="bijection"):
        lower(ops.grouped_swizzle_layout(10, 4, 8))


def test_genp_tables_constraints_and_symbolic_offsets(golden):
    from lego_b200.lowering import genp_tables
    # an arbitrary callable is tabulated over its domain; the table must be a permutation
    xor = L.GenP((4, 8), lambda x: (x[0] * 8 + x[1]) ^ 5, lambda f: ((f ^ 5) // 8, (f ^ 5) % 8))
    fwd, back = genp_tables(xor)
    assert np.array_equal(fwd, np.arange(32) ^ 5) and np.array_equal(fwd[back], np.arange(32))
    g = golden["layouts"]["genp_xor_4x8"]
    assert np.array_equal(fwd[np.asarray(g["ids"])], np.asarray(g["apply"]))     # the reference ran the same callable
    scalar_only = L.GenP((3, 3), lambda x: int(x[0]) * 3 + (int(x[1]) + 1) % 3, None)   # int() refuses arrays
    assert sorted(genp_tables(scalar_only)[0].tolist()) == list(range(9))
    with pytest.raises(ValueError, match="bijection"):
        genp_tables(L.GenP((4, 4), lambda x: x[0] * 4, None))
    with pytest.raises(ValueError, match="index range"):
        genp_tables(L.GenP((4, 4), lambda x: x[0] * 4 + x[1] + 1, None))
    with pytest.raises(ValueError, match="disagrees"):
        genp_tables(L.GenP((4, 4), lambda x: x[0] * 4 + x[1], lambda f: (f % 4, f // 4)))
    with pytest.raises(ValueError, match="table limit"):
        genp_tables(L.GenP((1 << 13, 1 << 12), lambda x: x[0], None))
    # user constraints on concrete sizes are facts to check (lego/lego.py:76-85)
    lay = L.OrderBy(L.Row(24, 512)).TileBy([24, 4], [1, 128], user_constraints=[L.divisibility_constraint(512, 128),
                                                                              L.le_constraint(1, 24),
                                                                              L.equal_constraint(4 * 128, 512)])
    assert len(lay.user_constraints) == 3
    for bad in (L.divisibility_constraint(500, 128), L.le_constraint(24, 24), L.equal_constraint(3, 4)):
        with pytest.raises(ValueError, match="constraint"):
            L.OrderBy(L.Row(24, 512)).TileBy([24, 4], [1, 128], user_constraints=[bad])
    # get_arange is a slice with explicit bounds
    assert np.array_equal(lay[3, 1, 0, L.get_arange(0, 128)], lay[3, 1, 0, :])
    # string coordinates give the closed-form expression the reference prints
    sp = pytest.importorskip("sympy")
    t = L.OrderBy(L.Row(4096, 4096)).TileBy([128, 128], [32, 32])
    e = t["bi", "bj", :, :]
    assert str(e) == "131072*bi + 32*bj + 4096*((tl.arange(0, 32))[:, None]) + ((tl.arange(0, 32))[None, :])"
    sw = ops.grouped_swizzle_layout(64, 32, 8)
    pm, pn = sp.symbols("pm pn", integer=True, nonnegative=True)
    f = sp.lambdify((pm, pn), sw["pm", "pn"], "numpy")
    a, b = np.indices((64, 32))
    assert np.array_equal(f(a, b), sw.apply(a, b))
    br = golden["c_strings"]["bricks_out"]
    bl = build_layout(golden["layouts"]["bricks_384"]["src"])
    assert str(bl["bx", "by", "bz", "i", "j", "k"]).replace(" ", "") == br["text"].replace(" ", "")
    with pytest.raises(ValueError, match="closed-form"):
        L.OrderBy(L.Col(3, 2)).GroupBy([(2, 3)])["a", "b"]


def test_c_printer_strings_match_the_layouts(golden):
    cs = golden["c_strings"]
    rng = np.random.default_rng(4)
    bx, by, bz = (rng.integers(0, 48, 512) for _ in range(3))
    i, j, k = (rng.integers(0, 8, 512) for _ in range(3))
    env = dict(bx=bx, by=by, bz=bz, i=i, j=j, k=k)
    for name in ("bricks_normal_out", "bricks_out"):
        lay = build_layout(golden["layouts"][cs[name]["layout"]]["src"])
        assert np.array_equal(eval_c_string(cs[name]["text"], env), lay.apply(bx, by, bz, i, j, k)), name
    n = 11
    ii, jj = np.indices((n, n))
    got = eval_c_string(cs["nw_antidiag"]["text"], dict(n=n, i=ii.ravel(), j=jj.ravel()))
    assert np.array_equal(got, L.antidiag(n, (ii.ravel(), jj.ravel())))


def test_genp_bodies_round_trip():
    n = 7
    lay = L.OrderBy(L.GenP((n, n), lambda i: L.antidiag(n, i), lambda f: L.antidiag_inv(n, f),
                           kind="antidiag")).GroupBy([(n, n)])
    ii, jj = np.indices((n, n))
    flat = lay.apply(ii.ravel(), jj.ravel())
    assert np.array_equal(np.sort(flat), np.arange(n * n))
    assert np.array_equal(flat, O.groupby_apply(spec_of(lay), [ii.ravel(), jj.ravel()]))
    bi, bj = lay.inv(flat)
    assert np.array_equal(bi, ii.ravel()) and np.array_equal(bj, jj.ravel())
    assert lower(lay).stages[0].blocks[0].kind == 1
    assert not fold(lay).foldable


def test_permute_plans():
    n = 4096
    src = L.OrderBy(L.Row(n, n)).TileBy([128, 128], [32, 32])
    dst = L.OrderBy(L.Col(n, n)).TileBy([128, 128], [32, 32])
    order = L.OrderBy(L.Col(128, 128)).TileBy([128, 128])
    assert ops.permute_plan(4, src, dst, order) == (3, 32, 32)       # tiles named by the layout, TMA-fed
    assert ops.permute_plan(4, src, dst) == (3, 32, 32)              # free choice: 128 B x 8 vectors
    assert ops.permute_plan(2, src, dst) == (3, 64, 64)
    assert ops.permute_plan(8, src, dst) == (3, 16, 16)
    kind, ti, to = ops.permute_plan(1, src, dst)
    assert kind == 2 and ti * to <= 16384                              # bytes: shared-memory tiled kernel
    small = L.OrderBy(L.Row(48, 80)).TileBy([3, 5], [16, 16])
    small_t = L.OrderBy(L.Col(48, 80)).TileBy([3, 5], [16, 16])
    assert ops.permute_plan(4, small, small_t, L.OrderBy(L.Row(3, 5)).TileBy([3, 5])) == (2, 16, 16)
    tm = L.OrderBy(L.Col(128, 128), L.Row(32, 32)).TileBy([128, 128], [32, 32])
    rm = L.OrderBy(L.Row(n, n)).TileBy([128, 128], [32, 32])
    assert ops.permute_plan(4, rm, tm)[0] == 5                         # common 32-element runs, 64 MiB: DMA permute
    ops.tune(permute_dma_long=0)
    try:
        assert ops.permute_plan(4, rm, tm) == (1, 32, 32)              # without it: output-order vector copy
    finally:
        ops.tune(permute_dma_long=1)
    a = L.OrderBy(L.Col(3, 2)).GroupBy([(2, 3)])
    b = L.OrderBy(L.Row(2, 3)).GroupBy([(2, 3)])
    assert ops.permute_plan(4, a, b)[0] == 0                           # staged interpreter
    with pytest.raises(ValueError):
        ops.permute_plan(4, src, L.OrderBy(L.Row(8, 8)).TileBy([8, 8]))
    with pytest.raises(ValueError):
        ops.permute_plan(3, src, dst)


def test_ops_fail_loudly_without_a_gpu():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.softmax(torch.zeros(4, 8, dtype=torch.float16))


def test_host_row_blocks_cover_the_rows_once():
    """Row blocks of the host-staging path: contiguous, in order, cover every row exactly once,
    honour the row multiple, and never come out empty."""
    from lego_b200 import ops
    for rows, row_bytes, mult in ((16384, 16384, 1), (2600, 8192, 1), (2304, 8192, 256), (7, 1 << 30, 1),
                                  (1000, 3, 1), (512, 16384, 256), (1, 1, 1), (16387, 16384, 4), (9001, 4096, 4)):
        blocks = ops._row_blocks(rows, row_bytes, mult)
        assert blocks[0][0] == 0 and blocks[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert all(r1 > r0 for r0, r1 in blocks)
        assert all((r1 - r0) % mult == 0 for r0, r1 in blocks[:-1])
        assert all((r1 - r0) * row_bytes <= max(ops._HOST_BLOCK_BYTES, mult * row_bytes) for r0, r1 in blocks)
