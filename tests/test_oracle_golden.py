"""Pin the oracle: every function of oracle/lego_oracle.py against outputs of the
reference itself (tests/golden/layouts.json, made by tests/golden/make_golden.py)."""
import numpy as np
import pytest

from helpers import eval_reference_string, unravel
from oracle import lego_oracle as O


def test_golden_file_is_complete(golden):
    assert golden["reference"] == "tavakkoliamirmohammad/LEGO"
    assert len(golden["layouts"]) >= 30
    assert len(golden["strings"]) >= 15


def test_apply_matches_reference(golden):
    for name, g in golden["layouts"].items():
        idx = unravel(g["ids"], g["dims"])
        got = O.groupby_apply(g["spec"], idx)
        assert np.array_equal(got, np.asarray(g["apply"], dtype=np.int64)), name


def test_inv_matches_reference(golden):
    for name, g in golden["layouts"].items():
        got = O.groupby_inv(g["spec"], np.asarray(g["inv_flat"], dtype=np.int64))
        exp = np.asarray(g["inv"], dtype=np.int64).reshape(len(g["inv_flat"]), len(g["dims"]))
        for k in range(len(g["dims"])):
            assert np.array_equal(np.broadcast_to(got[k], exp[:, k].shape), exp[:, k]), (name, k)


def test_apply_is_a_bijection_where_the_reference_is(golden):
    for name, g in golden["layouts"].items():
        size = int(np.prod(g["dims"]))
        if size > 1 << 16:
            continue
        full = O.groupby_apply_all(g["spec"])
        assert np.array_equal(np.sort(full), np.arange(size)), name
        back = O.groupby_inv(g["spec"], full)
        idx = unravel(np.arange(size), g["dims"])
        for k in range(len(g["dims"])):
            assert np.array_equal(back[k], idx[k]), (name, k)


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
