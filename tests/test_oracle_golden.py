"""Pin the oracle: every function of oracle/lego_oracle.py against outputs of the
reference itself (tests/golden/layouts.json, made by tests/golden/make_golden.py)."""
import numpy as np
import pytest

from helpers import eval_c_string, eval_reference_string, golden_spec, unravel
from oracle import lego_oracle as O


def test_golden_file_is_complete(golden):
    assert golden["reference"] == "tavakkoliamirmohammad/LEGO"
    assert len(golden["layouts"]) >= 30
    assert len(golden["strings"]) >= 15


def test_apply_matches_reference(golden):
    for name, g in golden["layouts"].items():
        idx = unravel(g["ids"], g["dims"])
        got = O.groupby_apply(golden_spec(g), idx)
        assert np.array_equal(got, np.asarray(g["apply"], dtype=np.int64)), name


def test_inv_matches_reference(golden):
    for name, g in golden["layouts"].items():
        got = O.groupby_inv(golden_spec(g), np.asarray(g["inv_flat"], dtype=np.int64))
        exp = np.asarray(g["inv"], dtype=np.int64).reshape(len(g["inv_flat"]), len(g["dims"]))
        for k in range(len(g["dims"])):
            assert np.array_equal(np.broadcast_to(got[k], exp[:, k].shape), exp[:, k]), (name, k)


def test_apply_is_a_bijection_where_the_reference_is(golden):
    for name, g in golden["layouts"].items():
        size = int(np.prod(g["dims"]))
        if size > 1 << 16:
            continue
        full = O.groupby_apply_all(golden_spec(g))
        assert np.array_equal(np.sort(full), np.arange(size)), name
        back = O.groupby_inv(golden_spec(g), full)
        idx = unravel(np.arange(size), g["dims"])
        for k in range(len(g["dims"])):
            assert np.array_equal(back[k], idx[k]), (name, k)


def test_genp_and_brick_layouts_are_pinned(golden):
    names = set(golden["layouts"])
    assert {"genp_antidiag_8", "genp_antidiag_33", "genp_reverse_6x10", "genp_mixed_3x5x5", "genp_tiled_antidiag",
            "genp_xor_4x8", "bricks_normal_384", "bricks_384"} <= names
    # the whole domain of the small GenP layouts was recorded, so the oracle's bodies are pinned everywhere
    for name in ("genp_antidiag_8", "genp_antidiag_33", "genp_reverse_6x10", "genp_xor_4x8"):
        g = golden["layouts"][name]
        assert g["ids"] == list(range(int(np.prod(g["dims"])))), name


def test_c_printer_strings(golden):
    """The expressions LEGOCCodePrinter prints into the CUDA programs, evaluated as C would,
    against the oracle: brick offsets (with and without the stencil displacement) and the
    anti-diagonal GenP with a symbolic n."""
    cs = golden["c_strings"]
    rng = np.random.default_rng(3)
    m = 4096
    bx, by, bz = (rng.integers(0, 48, m) for _ in range(3))
    i, j, k = (rng.integers(2, 6, m) for _ in range(3))
    di, dj, dk = (rng.integers(-2, 3, m) for _ in range(3))
    env = dict(bx=bx, by=by, bz=bz, i=i, j=j, k=k, i_diff=di, j_diff=dj, k_diff=dk)
    for name, shifted in (("bricks_normal_out", False), ("bricks_out", False), ("bricks_normal_in", True),
                          ("bricks_in", True)):
        spec = golden_spec(golden["layouts"][cs[name]["layout"]])
        idx = [bx, by, bz, i + di, j + dj, k + dk] if shifted else [bx, by, bz, i, j, k]
        assert np.array_equal(eval_c_string(cs[name]["text"], env), O.groupby_apply(spec, idx)), name
    for n in (1, 2, 7, 64):
        ii, jj = np.indices((n, n))
        got = eval_c_string(cs["nw_antidiag"]["text"], dict(n=n, i=ii.ravel(), j=jj.ravel()))
        spec = {"dims": [n, n], "objects": [[{"kind": "antidiag", "dims": [n, n]}],
                                            [{"kind": "regp", "dims": [n, n], "perm": [0, 1]}],
                                            [{"kind": "regp", "dims": [n, n], "perm": [0, 1]}]]}
        assert np.array_equal(got, O.groupby_apply(spec, [ii.ravel(), jj.ravel()])), n


def test_swizzle_string(golden):
    s = golden["strings"]
    for npm, npn, gm in [(64, 32, 8), (16, 4, 8), (4, 8, 8), (8, 8, 8), (1, 5, 8)]:
        pid = np.arange(npm * npn, dtype=np.int64)
        env = {"pid": pid, "num_pid_m": npm, "num_pid_n": npn, "GM": gm}
        pm = eval_reference_string(s["matmul_pid_m"]["text"], env)
        pn = eval_reference_string(s["matmul_pid_n"]["text"], env)
        om, on = O.grouped_swizzle(pid, npm, npn, gm)
        assert np.array_equal(pm, om) and np.array_equal(pn, on)
        spec = {"dims": [npm, npn],
                "objects": [[{"kind": "regp", "dims": [max(npm // gm, 1), 1], "perm": [1, 0]},
                             {"kind": "regp", "dims": [min(npm, gm), npn], "perm": [1, 0]}],
                            [{"kind": "regp", "dims": [max(npm // gm, 1), min(npm, gm), 1, npn],
                              "perm": [0, 2, 1, 3]}],
                            [{"kind": "regp", "dims": [npm, npn], "perm": [0, 1]}]]}
        im, inn = O.groupby_inv(spec, pid)
        assert np.array_equal(im, pm) and np.array_equal(inn, pn)


def test_swizzle_is_not_bijective_when_group_does_not_divide():
    pm, pn = O.grouped_swizzle(np.arange(40), 10, 4, 8)
    assert len({(int(a), int(b)) for a, b in zip(pm, pn)}) < 40


def test_grouped_tiles_order():
    tiles = O.grouped_tiles([(256, 512, 64), (128, 256, 64)], 128, 256)
    assert tiles == [(0, 0, 0), (0, 0, 1), (0, 1, 0), (0, 1, 1), (1, 0, 0)]


def test_permute_is_transpose():
    g_src = {"dims": [2, 3, 4, 4], "objects": [
        [{"kind": "regp", "dims": [8, 12], "perm": [0, 1]}],
        [{"kind": "regp", "dims": [8, 12], "perm": [0, 1]}],
        [{"kind": "regp", "dims": [2, 3, 4, 4], "perm": [0, 2, 1, 3]}]]}
    g_dst = {"dims": [2, 3, 4, 4], "objects": [
        [{"kind": "regp", "dims": [8, 12], "perm": [1, 0]}],
        [{"kind": "regp", "dims": [8, 12], "perm": [0, 1]}],
        [{"kind": "regp", "dims": [2, 3, 4, 4], "perm": [0, 2, 1, 3]}]]}
    x = np.arange(96, dtype=np.float32)
    out = O.permute(x, g_src, g_dst)
    assert np.array_equal(out.reshape(12, 8), x.reshape(8, 12).T)


def test_float_paths_match_torch():
    torch = pytest.importorskip("torch")
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 33, generator=g).half()
    w = torch.randn(33, generator=g).half()
    b = torch.randn(33, generator=g).half()
    y, mean, rstd = O.layernorm_fwd(x, w, b, 1e-5)
    ref = torch.nn.functional.layer_norm(x.float(), (33,), w.float(), b.float(), 1e-5)
    assert torch.allclose(y.float(), ref, atol=2e-3)
    assert torch.allclose(O.softmax(x).float().sum(-1), torch.ones(7), atol=2e-3)
    xa = x.float().requires_grad_(True)
    wa = w.float().requires_grad_(True)
    ba = b.float().requires_grad_(True)
    dy = torch.randn(7, 33, generator=g).half()
    torch.nn.functional.layer_norm(xa, (33,), wa, ba, 1e-5).backward(dy.float())
    dx, dw, db = O.layernorm_bwd(dy, x, w, mean, rstd)
    assert torch.allclose(dx.float(), xa.grad, atol=5e-3)
    assert torch.allclose(dw.float(), wa.grad, atol=2e-2)
    assert torch.allclose(db.float(), ba.grad, atol=2e-2)
