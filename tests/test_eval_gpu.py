"""Index-map evaluator on the GPU, through the C ABI, bit-exact against the oracle."""
import numpy as np
import pytest
import torch

import lego_b200 as L
from lego_b200 import ops
from helpers import build_layout, genp_kind_of, golden_spec, spec_of, unravel
from oracle import lego_oracle as O

pytestmark = pytest.mark.gpu


def test_range_apply_inv_for_every_golden_layout(golden):
    cases = []
    for name, g in golden["layouts"].items():
        cases.append((name, g, build_layout(g["src"])))                 # GenP blocks as look-up tables
        if genp_kind_of(g):
            cases.append((name + " (closed form)", g, build_layout(g["src"], genp_kind=genp_kind_of(g))))
    for name, g, lay in cases:
        size = lay.size()
        spec = golden_spec(g)
        # golden vectors of the reference itself
        ids = torch.tensor(g["ids"], dtype=torch.int64)
        idx = torch.stack([torch.from_numpy(v) for v in unravel(g["ids"], g["dims"])], dim=1).contiguous()
        got = ops.eval_apply(lay, idx.cuda()).cpu().numpy()
        assert np.array_equal(got, np.asarray(g["apply"])), name
        inv = ops.eval_inv(lay, torch.tensor(g["inv_flat"], dtype=torch.int64).cuda()).cpu().numpy()
        assert np.array_equal(inv, np.asarray(g["inv"]).reshape(inv.shape)), name
        # whole domain against the oracle (bounded so the CPU side stays quick)
        if size <= 1 << 22:
            full = ops.eval_range(lay).cpu().numpy()
            assert np.array_equal(full, O.groupby_apply_all(spec)), name
            assert np.array_equal(np.sort(full), np.arange(size)), name
            back = ops.eval_inv(lay, torch.from_numpy(full).cuda()).cpu().numpy()
            exp = np.stack(unravel(np.arange(size), g["dims"]), axis=1)
            assert np.array_equal(back, exp), name
        del ids


def test_full_size_domains_are_bijections():
    # 4096^2 tiled (config 1), 2^27 rows x cols (configs 2/3), swizzle 64 x 32 (config 4)
    for lay in (L.OrderBy(L.Col(128, 128), L.Row(32, 32)).TileBy([128, 128], [32, 32]),
                L.OrderBy(L.Col(4096, 4096)).TileBy([128, 128], [32, 32]),
                L.OrderBy(L.Row(16384, 8192)).TileBy([16384, 64], [1, 128])):
        size = lay.size()
        flat = ops.eval_range(lay)
        seen = torch.zeros(size, dtype=torch.int8, device="cuda")
        seen[flat] = 1
        assert int(seen.sum()) == size                       # onto => bijection
        back = ops.eval_inv(lay, flat[:1 << 20])
        ids = np.arange(1 << 20)
        exp = np.stack(unravel(ids, lay.dims()), axis=1)
        assert np.array_equal(back.cpu().numpy(), exp)
        # sampled against the oracle
        sel = torch.randint(0, size, (4096,), generator=torch.Generator().manual_seed(5)).numpy()
        ref = O.groupby_apply(spec_of(lay), unravel(sel, lay.dims()))
        assert np.array_equal(flat.cpu().numpy()[sel], ref)


def test_inv_ragged_counts_ranks_and_unaligned_output():
    """inv on position counts that are no multiple of a warp, for ranks 2, 3 and 4, into an output
    that starts 16-byte aligned (thread-per-position kernel) and 8 bytes off (per-word kernel)."""
    import ctypes
    from lego_b200 import _abi
    from lego_b200.lowering import lower
    lays = (L.OrderBy(L.Col(96, 80)).TileBy([96, 80]), L.OrderBy(L.Row(24, 20, 18)).TileBy([24, 20, 18]),
            L.OrderBy(L.Col(64, 96)).TileBy([8, 6], [8, 16]))
    for lay in lays:
        size, rank = lay.size(), len(lay.dims())
        for n in (4096, 4097, 4127, 7001):
            sel = torch.randint(0, size, (n,), generator=torch.Generator().manual_seed(n)).numpy()
            flat = O.groupby_apply(spec_of(lay), unravel(sel, lay.dims()))
            exp = np.stack(unravel(sel, lay.dims()), axis=1)
            dev = torch.from_numpy(flat).cuda()
            assert np.array_equal(ops.eval_inv(lay, dev).cpu().numpy(), exp), (rank, n)
            room = torch.zeros(n * rank + 1, dtype=torch.int64, device="cuda")
            off = room[1:].view(n, rank)                       # 8 bytes past a 16-byte boundary
            desc = lower(lay)
            _abi.check(_abi.lib().lego_eval_inv(ctypes.byref(desc), dev.data_ptr(), off.data_ptr(), n, None),
                       "lego_eval_inv")
            assert np.array_equal(off.cpu().numpy(), exp), (rank, n)


def test_wide_index_space_uses_64_bit_arithmetic():
    lay = L.OrderBy(L.Col(1 << 17, 1 << 16)).TileBy([1 << 10, 1 << 9], [128, 128])   # 2^33 elements
    begin = (1 << 32) + 12345
    got = ops.eval_range(lay, begin, 1 << 16).cpu().numpy()
    ids = np.arange(begin, begin + (1 << 16))
    assert np.array_equal(got, O.groupby_apply(spec_of(lay), unravel(ids, lay.dims())))
    back = ops.eval_inv(lay, torch.from_numpy(got).cuda()).cpu().numpy()
    assert np.array_equal(back, np.stack(unravel(ids, lay.dims()), axis=1))


def test_genp_blocks_on_the_device():
    n = 33
    lay = L.OrderBy(L.GenP((n, n), lambda i: L.antidiag(n, i), lambda f: L.antidiag_inv(n, f),
                           kind="antidiag")).GroupBy([(n, n)])
    full = ops.eval_range(lay).cpu().numpy()
    assert np.array_equal(full, O.groupby_apply_all(spec_of(lay)))
    back = ops.eval_inv(lay, torch.arange(n * n).cuda()).cpu().numpy()
    oi, oj = O.groupby_inv(spec_of(lay), np.arange(n * n))
    assert np.array_equal(back[:, 0], oi) and np.array_equal(back[:, 1], oj)
    rev = L.OrderBy(L.GenP((5, 7), lambda i: (5 - 1 - i[0]) * 7 + 7 - 1 - i[1],
                           lambda f: ((34 - f) // 7, (34 - f) % 7), kind="reverse")).GroupBy([(5, 7)])
    assert np.array_equal(ops.eval_range(rev).cpu().numpy(), np.arange(35)[::-1])
    assert np.array_equal(ops.eval_inv(rev, torch.arange(35).cuda()).cpu().numpy(),
                          np.stack(unravel(np.arange(35)[::-1], (5, 7)), axis=1))


def test_empty_and_bad_arguments():
    lay = L.OrderBy(L.Row(8, 8)).TileBy([2, 2], [4, 4])
    assert ops.eval_range(lay, 0, 0).numel() == 0
    assert ops.eval_apply(lay, torch.zeros((0, 4), dtype=torch.int64).cuda()).numel() == 0
    with pytest.raises(ValueError):
        ops.eval_range(lay, 60, 10)
    with pytest.raises(ValueError):
        ops.eval_apply(lay, torch.zeros((4, 3), dtype=torch.int64).cuda())


def test_range_windows_odd_offsets_and_term_mixes():
    """Windows that start and end anywhere (odd offsets, a few ids past a 1024-id block,
    unaligned output pointers) over layouts with one, two and many digits that change
    inside a run of 32 ids."""
    cases = (L.OrderBy(L.Col(512, 512)).TileBy([16, 16], [32, 32]),          # one fast digit (32 wide)
             L.OrderBy(L.Col(960, 400)).TileBy([80, 50], [12, 8]),           # innermost digits 8 and 12 wide: two fast
             L.OrderBy(L.Col(6, 10, 14, 18)).TileBy([3, 5, 7, 9], [2, 2, 2, 2]),  # many narrow digits
             L.OrderBy(L.Row(70000)).TileBy([17500], [4]))                   # identity map, one term
    for lay in cases:
        size = lay.size()
        want = O.groupby_apply_all(spec_of(lay))
        assert np.array_equal(ops.eval_range(lay).cpu().numpy(), want)
        for begin, count in ((1, size - 1), (1023, 4097), (size - 5001, 5001), (2048, 4096), (31, 8191)):
            got = ops.eval_range(lay, begin, count).cpu().numpy()
            assert np.array_equal(got, want[begin:begin + count]), (lay.dims(), begin, count)
