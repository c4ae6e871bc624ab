"""Generate ``tests/golden/layouts.json`` by running the reference itself.

    python tests/golden/make_golden.py /path/to/reference

The reference (tavakkoliamirmohammad/LEGO) is pure Python + SymPy + Z3 and
imports on a CPU-only machine.  It cannot travel to the machine the GPU tests
run on, so its outputs are frozen here:

* ``layouts``: for each named layout (every layout the five benchmark kernels
  use, the appendix examples and edge cases) the logical dims, the structure of
  ``GroupBy.objects`` as a plain spec, ``GroupBy.apply`` at sampled logical ids
  and the scalar ``GroupBy.inv`` at sampled flat positions.
* ``strings``: the index expressions the reference prints into its Triton
  kernels (the same text as ``triton_generated/**``), generated symbolically,
  with concrete values at which the tests evaluate them.

* ``c_strings``: the expressions ``LEGOCCodePrinter`` prints into the CUDA benchmark
  programs (brick offsets, the anti-diagonal GenP with symbolic n).

The layout source strings use only names that exist both in the reference's
``lego.lego`` and in ``lego_b200`` (Row, Col, RegP, GenP, OrderBy, antidiag,
antidiag_inv, new_antidiag), so the tests rebuild the same layout with the
product's classes.
"""
from __future__ import annotations

import json
import os
import random
import sys

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/reference (a checkout of tavakkoliamirmohammad/LEGO)")
REF = sys.argv[1]
sys.path.insert(0, REF)

import sympy as sp  # noqa: E402
from lego.lego_python import LEGOPythonCodePrinter  # noqa: E402
import lego.lego as R  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

LAYOUTS = {
    # --- transpose (benchmarks/mlir/transpose_{naive,smem}.py, BASELINE config 1)
    "t_src_4096": "OrderBy(Row(4096,4096)).TileBy([128,128],[32,32])",
    "t_dst_4096": "OrderBy(Col(4096,4096)).TileBy([128,128],[32,32])",
    "t_tilemajor_4096": "OrderBy(Col(128,128),Row(32,32)).TileBy([128,128],[32,32])",
    "t_order_col128": "OrderBy(Col(128,128)).TileBy([128,128])",
    "t_order_row128": "OrderBy(Row(128,128)).TileBy([128,128])",
    "t_read3_256": "OrderBy(Row(256,256)).TileBy([8,8],[4,1],[8,32])",
    "t_write3_256": "OrderBy(Row(256,256)).TileBy([8,8],[1,4],[32,8])",
    "t_thread_r": "OrderBy(Row(8,32)).TileBy([8,32])",
    "t_thread_w": "OrderBy(Col(32,8)).TileBy([32,8])",
    "t_src_96x160": "OrderBy(Row(96,160)).TileBy([3,5],[32,32])",
    "t_dst_96x160": "OrderBy(Col(96,160)).TileBy([3,5],[32,32])",
    # --- row maps (softmax / LayerNorm, configs 2 and 3)
    "rows_16384_by4": "OrderBy(Row(16384)).TileBy([4096],[4])",
    "rows_1823": "OrderBy(Row(1823)).TileBy([1823])",
    "rows_col_12x5": "OrderBy(Col(12,5)).TileBy([12,5])",
    "softmax_in": "OrderBy(Row(37,64)).TileBy([37,64])",
    "ln_x": "OrderBy(Row(24,512)).TileBy([24,4],[1,128])",
    # --- GEMM operands and tile orders (config 4)
    "mm_a_nt": "OrderBy(Row(512,256)).TileBy([4,4],[128,64])",
    "mm_a_t": "OrderBy(Col(512,256)).TileBy([4,4],[128,64])",
    "mm_b_nt": "OrderBy(Row(256,512)).TileBy([4,2],[64,256])",
    "mm_b_t": "OrderBy(Col(256,512)).TileBy([4,2],[64,256])",
    "mm_c": "OrderBy(Row(512,512)).TileBy([4,2],[128,256])",
    "swizzle_64x32_g8": "OrderBy(Col(8,1),Col(8,32)).TileBy([64,32])",
    "swizzle_16x4_g8": "OrderBy(Col(2,1),Col(8,4)).TileBy([16,4])",
    "swizzle_4x8_g8": "OrderBy(Col(1,1),Col(4,8)).TileBy([4,8])",
    # --- grouped GEMM per-group tile order (config 5)
    "gg_tiles_8x16": "OrderBy(Row(8,16)).TileBy([8,16])",
    # --- appendix / edge cases
    "graphene": "OrderBy(RegP([2,2,2,2,2],[4,1,3,2,0])).GroupBy([(2,2,2,2,2)])",
    "chain_4x4": "OrderBy(Row(4,4)).OrderBy(Col(4,4)).TileBy([2,2],[2,2])",
    "misaligned_col": "OrderBy(Col(3,2)).GroupBy([(2,3)])",
    "misaligned_row": "OrderBy(Row(6,4)).GroupBy([(4,6)])",
    "misaligned_two": "OrderBy(Col(6,4),Row(5)).GroupBy([(4,5,6)])",
    "brick_3d": "OrderBy(Row(4,6,2),Col(2,2,4)).TileBy([4,6,2],[2,2,4])",
    "ones": "OrderBy(Row(1,7,1)).TileBy([1,7,1])",
    "regp_3": "OrderBy(RegP([3,4,5],[1,2,0])).GroupBy([(3,4,5)])",
    "two_blocks_regp": "OrderBy(RegP([3,4],[1,0]),RegP([5,2],[0,1])).GroupBy([(12,10)])",
    "single": "OrderBy(Row(1)).TileBy([1])",
    # --- 3-D bricks (benchmarks/cuda/bricks_f3d.py:10-13; bricks_laplasian.py uses the same two)
    "bricks_normal_384": "OrderBy(Row(384,384,384)).TileBy([48,48,48],[8,8,8])",
    "bricks_384": "OrderBy(Row(48,48,48),Row(8,8,8)).TileBy([48,48,48],[8,8,8])",
    # --- GenP blocks (lego/lego.py:150-178 with the bodies of :490-535; benchmarks/cuda/nw_sympy.py:9-11)
    "genp_antidiag_8": "OrderBy(GenP([8,8], lambda x: antidiag(8,x), lambda f: antidiag_inv(8,f))).TileBy((8,8))",
    "genp_antidiag_33": "OrderBy(GenP([33,33], lambda x: antidiag(33,x), lambda f: antidiag_inv(33,f))).TileBy((33,33))",
    "genp_reverse_6x10": ("OrderBy(GenP([6,10], lambda x: new_antidiag(6,10,x), "
                          "lambda f: ((59-f)//10, (59-f)%10))).TileBy((6,10))"),
    "genp_mixed_3x5x5": ("OrderBy(Row(3), GenP([5,5], lambda x: antidiag(5,x), lambda f: antidiag_inv(5,f)))"
                         ".GroupBy([(3,5,5)])"),
    "genp_tiled_antidiag": ("OrderBy(Row(2,3), GenP([4,4], lambda x: antidiag(4,x), lambda f: antidiag_inv(4,f)))"
                            ".TileBy([2,3],[4,4])"),
    "genp_xor_4x8": ("OrderBy(GenP([4,8], lambda x: (x[0]*8 + x[1]) ^ 5, lambda f: ((f ^ 5)//8, (f ^ 5)%8)))"
                     ".TileBy((4,8))"),
}

# which closed form a GenP layout's block is (for the spec the oracle reads); anything else
# is recorded by the source of its f_apply
GENP_KIND = {"genp_antidiag_8": "antidiag", "genp_antidiag_33": "antidiag", "genp_reverse_6x10": "reverse",
             "genp_mixed_3x5x5": "antidiag", "genp_tiled_antidiag": "antidiag"}
GENP_SRC = {"genp_xor_4x8": "lambda x: (x[0]*8 + x[1]) ^ 5"}

MAX_FULL = 4096
N_APPLY = 1536
N_INV = 192


def block_spec(p, name):
    dims = [int(d) for d in p.dims()]
    if isinstance(p, R.GenP):
        if name in GENP_KIND:
            return {"kind": GENP_KIND[name], "dims": dims}
        return {"kind": "callable", "dims": dims, "f_apply_src": GENP_SRC[name]}
    if not isinstance(p, R.RegP):
        raise TypeError("unknown permutation block")
    perm = [int(v) for v in p.perm(list(range(len(dims))))]  # the permutation lives in a closure
    return {"kind": "regp", "dims": dims, "perm": perm}


def layout_spec(layout, name):
    return {"dims": [int(d) for d in layout.dims()],
            "objects": [[block_spec(p, name) for p in o.perms] for o in layout.objects]}


def unravel(flat, dims):
    out = []
    for n in reversed(dims):
        out.append(flat % n)
        flat //= n
    return out[::-1]


def sample_layout(name, src, rng):
    layout = eval(src, {k: getattr(R, k) for k in ("Row", "Col", "RegP", "GenP", "OrderBy", "antidiag",
                                                   "antidiag_inv", "new_antidiag")})
    dims = [int(d) for d in layout.dims()]
    size = 1
    for d in dims:
        size *= d
    if size <= MAX_FULL:
        ids = list(range(size))
    else:
        ids = sorted(set([0, 1, size - 1, size - 2] + [rng.randrange(size) for _ in range(N_APPLY)]))
    applied = [int(layout.apply(*unravel(i, dims))) for i in ids]
    inv_flat = ids if size <= N_INV else sorted(set([0, size - 1] + [rng.randrange(size) for _ in range(N_INV)]))
    inv = [[int(v) for v in layout.inv(f)] for f in inv_flat]
    print(f"  {name}: dims={dims} apply@{len(ids)} inv@{len(inv_flat)}", flush=True)
    return {"src": src, "dims": dims, "spec": layout_spec(layout, name), "ids": ids, "apply": applied,
            "inv_flat": inv_flat, "inv": inv}


def golden_strings():
    """Index expressions exactly as the generators print them
    (benchmarks/triton/*.py), symbolic in the sizes."""
    out = {}
    M, N, K, BM, BN, BK, npm, npn, GM, pid, k = sp.symbols(
        "M N K BM BN BK num_pid_m num_pid_n GM pid k", integer=True, positive=True)
    pr = LEGOPythonCodePrinter(allow_unknown_functions=True)

    def show(e):
        return pr.doprint(sp.simplify(e))

    # benchmarks/triton/matmul_sympy.py:37-65
    for ta in (False, True):
        for tb in (False, True):
            tag = ("TA" if ta else "NTA") + "_" + ("TB" if tb else "NTB")
            a = R.OrderBy(R.Col(M, K) if ta else R.Row(M, K)).TileBy([M / BM, K / BK], [BM, BK])
            b = R.OrderBy(R.Col(K, N) if tb else R.Row(K, N)).TileBy([K / BK, N / BN], [BK, BN])
            out[f"matmul_{tag}_a"] = {
                "text": show(a["pid_m", k, :, :]),
                "layout": ("OrderBy(Col(M,K)).TileBy([M//BM,K//BK],[BM,BK])" if ta
                           else "OrderBy(Row(M,K)).TileBy([M//BM,K//BK],[BM,BK])"),
                "key": ["pid_m", "k", ":", ":"]}
            out[f"matmul_{tag}_b"] = {
                "text": show(b[k, "pid_n", :, :]),
                "layout": ("OrderBy(Col(K,N)).TileBy([K//BK,N//BN],[BK,BN])" if tb
                           else "OrderBy(Row(K,N)).TileBy([K//BK,N//BN],[BK,BN])"),
                "key": ["k", "pid_n", ":", ":"]}
    c = R.OrderBy(R.Row(M, N)).TileBy([M / BM, N / BN], [BM, BN])
    out["matmul_c"] = {"text": show(c["pid_m", "pid_n", :, :]),
                       "layout": "OrderBy(Row(M,N)).TileBy([M//BM,N//BN],[BM,BN])",
                       "key": ["pid_m", "pid_n", ":", ":"]}
    sw = R.OrderBy(R.Col(sp.Max(npm // GM, 1), 1), R.Col(sp.Min(npm, GM), npn)).TileBy([npm, npn]).inv(pid)
    out["matmul_pid_m"] = {"text": show(sw[0]), "inv_of": "swizzle", "component": 0}
    out["matmul_pid_n"] = {"text": show(sw[1]), "inv_of": "swizzle", "component": 1}

    # benchmarks/triton/softmax_sympy.py:6-9
    n_rows, n_cols, BS = sp.symbols("n_rows n_cols BLOCK_SIZE", integer=True, positive=True)
    sm = R.OrderBy(R.Row(n_rows, n_cols)).TileBy([n_rows, n_cols])
    out["softmax_in"] = {"text": show(sm["row_idx", R.get_arange(0, BS)]),
                         "layout": "OrderBy(Row(n_rows,n_cols)).TileBy([n_rows,n_cols])",
                         "key": ["row_idx", "arange(BLOCK_SIZE)"]}

    # benchmarks/triton/layernorm_triton.py:10-26
    Ms, Ns, BSN = sp.symbols("M N BLOCK_SIZE_N", integer=True, positive=True)
    xl = R.OrderBy(R.Row(Ms, Ns)).TileBy([Ms, Ns / BSN], [1, BSN],
                                          user_constraints=[R.divisibility_constraint(Ns, BSN)])
    pr2 = LEGOPythonCodePrinter(allow_unknown_functions=True, do_broadcast=False)
    out["layernorm_xy"] = {"text": pr2.doprint(sp.simplify(xl["pid", "k", 0, :])),
                           "layout": "OrderBy(Row(M,N)).TileBy([M,N//BLOCK_SIZE_N],[1,BLOCK_SIZE_N])",
                           "key": ["pid", "k", "0", ":"], "flat": True}
    out["layernorm_col"] = {"text": pr2.doprint(sp.simplify(xl[0, "k", 0, :])),
                            "layout": "OrderBy(Row(M,N)).TileBy([M,N//BLOCK_SIZE_N],[1,BLOCK_SIZE_N])",
                            "key": ["0", "k", "0", ":"], "flat": True}

    # benchmarks/triton/grouped_gemm_sympy.py:7-24
    gm, gn, gk, BSM, BSNg, BSK = sp.symbols(
        "gm gn gk BLOCK_SIZE_M BLOCK_SIZE_N BLOCK_SIZE_K", integer=True, positive=True)
    ga = R.OrderBy(R.Row(gm, gk)).TileBy([gm / BSM, gk / BSK], [BSM, BSK])
    gb = R.OrderBy(R.Row(gk, gn)).TileBy([gk / BSK, gn / BSNg], [BSK, BSNg])
    gc = R.OrderBy(R.Row(gm, gn)).TileBy([gm / BSM, gn / BSNg], [BSM, BSNg])
    out["grouped_a"] = {"text": show(ga["tile_m_idx", "kk", :, :]),
                        "layout": "OrderBy(Row(gm,gk)).TileBy([gm//BLOCK_SIZE_M,gk//BLOCK_SIZE_K],[BLOCK_SIZE_M,BLOCK_SIZE_K])",
                        "key": ["tile_m_idx", "kk", ":", ":"]}
    out["grouped_b"] = {"text": show(gb["kk", "tile_n_idx", :, :]),
                        "layout": "OrderBy(Row(gk,gn)).TileBy([gk//BLOCK_SIZE_K,gn//BLOCK_SIZE_N],[BLOCK_SIZE_K,BLOCK_SIZE_N])",
                        "key": ["kk", "tile_n_idx", ":", ":"]}
    out["grouped_c"] = {"text": show(gc["tile_m_idx", "tile_n_idx", :, :]),
                        "layout": "OrderBy(Row(gm,gn)).TileBy([gm//BLOCK_SIZE_M,gn//BLOCK_SIZE_N],[BLOCK_SIZE_M,BLOCK_SIZE_N])",
                        "key": ["tile_m_idx", "tile_n_idx", ":", ":"]}

    # benchmarks/examples/graphene.py
    i, j, kk, w, q = sp.symbols("i j k w q", integer=True)
    gl = R.OrderBy(R.RegP([2, 2, 2, 2, 2], [4, 1, 3, 2, 0])).GroupBy([(2, 2, 2, 2, 2)])
    out["graphene"] = {"text": str(gl[i, j, kk, w, q]),
                       "layout": "OrderBy(RegP([2,2,2,2,2],[4,1,3,2,0])).GroupBy([(2,2,2,2,2)])",
                       "key": ["i", "j", "k", "w", "q"], "flat": True}
    return out


def golden_c_strings():
    """Index expressions as LEGOCCodePrinter (lego/lego_c.py:9-38) prints them into the CUDA
    benchmark programs: the brick offsets of benchmarks/cuda/bricks_f3d.py:10-21 (the text of
    benchmarks/cuda/bricks/main.cu:48,56-57,91,99-100) and the anti-diagonal GenP of
    benchmarks/cuda/nw_sympy.py:9-11 with a symbolic n."""
    from lego.lego_c import LEGOCCodePrinter
    pr = LEGOCCodePrinter()
    out = {}
    i, j, k, i_diff, j_diff, k_diff, bx, by, bz = sp.symbols("i j k i_diff j_diff k_diff bx by bz",
                                                             integer=True, positive=True)
    N, B = 384, 8
    normal = R.OrderBy(R.Row(N, N, N)).TileBy([N // B] * 3, [B] * 3)
    bricks = R.OrderBy(R.Row(N // B, N // B, N // B), R.Row(B, B, B)).TileBy([N // B] * 3, [B] * 3)
    out["bricks_normal_out"] = {"text": pr.doprint(sp.simplify(normal[bx, by, bz, i, j, k])),
                                "layout": "bricks_normal_384", "key": ["bx", "by", "bz", "i", "j", "k"]}
    out["bricks_out"] = {"text": pr.doprint(sp.simplify(bricks[bx, by, bz, i, j, k])),
                         "layout": "bricks_384", "key": ["bx", "by", "bz", "i", "j", "k"]}
    out["bricks_normal_in"] = {
        "text": pr.doprint(sp.simplify(normal[bx, by, bz, i + i_diff, j + j_diff, k + k_diff])),
        "layout": "bricks_normal_384", "key": ["bx", "by", "bz", "i+i_diff", "j+j_diff", "k+k_diff"]}
    out["bricks_in"] = {
        "text": pr.doprint(sp.simplify(bricks[bx, by, bz, i + i_diff, j + j_diff, k + k_diff])),
        "layout": "bricks_384", "key": ["bx", "by", "bz", "i+i_diff", "j+j_diff", "k+k_diff"]}
    n, ii, jj = sp.symbols("n i j", integer=True, postive=True)
    anti = R.OrderBy(R.GenP([n, n], lambda x: R.antidiag(n, x), None)).TileBy((n, n))
    out["nw_antidiag"] = {"text": pr.doprint(sp.simplify(anti[ii, jj])), "genp": "antidiag", "key": ["i", "j"]}
    return out


def main():
    rng = random.Random(20240607)
    print("sampling layouts through the reference ...", flush=True)
    layouts = {name: sample_layout(name, src, rng) for name, src in LAYOUTS.items()}
    print("printing golden strings ...", flush=True)
    strings = golden_strings()
    for k_, v in strings.items():
        print(f"  {k_}: {v['text']}")
    c_strings = golden_c_strings()
    for k_, v in c_strings.items():
        print(f"  {k_}: {v['text']}")
    path = os.path.join(HERE, "layouts.json")
    with open(path, "w") as f:
        json.dump({"reference": "tavakkoliamirmohammad/LEGO", "sympy": sp.__version__,
                   "layouts": layouts, "strings": strings, "c_strings": c_strings}, f, separators=(",", ":"))
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
