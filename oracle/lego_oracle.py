"""CPU restatement of the reference's algorithms.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference legs may
import it.  Nothing under ``lego_b200/`` imports it, and the ops there fail if
the CUDA library is missing instead of routing through here.

Parity is pinned: ``tests/golden/layouts.json`` holds outputs of the reference
itself (tavakkoliamirmohammad/LEGO, imported and run by
``tests/golden/make_golden.py``) for every layout used by the benchmarks plus
edge cases, and the expression strings the reference prints for its kernels;
``tests/test_oracle_golden.py`` checks every function below against them.

Index maps follow the reference line by line in numpy int64 (plain ``+ * // %``;
the reference's SymPy/Z3 layers only simplify the same arithmetic).  A layout is
described by a plain "spec" so the oracle shares no code with the product:

    {"dims": [...logical dims...],
     "objects": [                     # GroupBy.objects, in the reference's order
        [ {"kind": "regp", "dims": [...], "perm": [...]}, ... ],   # one OrderBy
        ... ]}

Floating-point paths restate what the reference's own checks compare against
(``torch.softmax``, ``F.layer_norm``, ``torch.matmul`` in fp32 on the CPU).
"""
from __future__ import annotations

import numpy as np


def spec_of(layout) -> dict:
    """Plain spec of a layout object that exposes the reference's attributes
    (``.objects`` -> OrderBy with ``.perms``; a perm has ``.dims()`` and either
    ``.permutation`` (RegP / Row / Col), ``.kind`` (a named GenP body) or, for a GenP
    given only by callables, the user's ``f_apply`` itself.  Structure only: no arithmetic
    of the layout object is used."""
    objects = []
    for o in layout.objects:
        stage = []
        for p in o.perms:
            if hasattr(p, "permutation"):
                stage.append({"kind": "regp", "dims": list(p.dims()), "perm": list(p.permutation)})
            elif getattr(p, "kind", None) is None and hasattr(p, "f_apply"):
                # a GenP given only by the user's callables: the oracle calls them itself
                stage.append({"kind": "callable", "dims": list(p.dims()), "f_apply": p.f_apply})
            else:
                stage.append({"kind": p.kind, "dims": list(p.dims())})
        objects.append(stage)
    return {"dims": list(layout.dims()), "objects": objects}


# --------------------------------------------------------------------------
# index maps
# --------------------------------------------------------------------------

def flatten_index(indices, dims):
    """lego/lego.py:93-109 -- B_n(i, n) = sum_k i_k * prod(dims[k+1:])."""
    if len(indices) != len(dims):
        raise ValueError("Number of indices must match number of dimensions")
    flat = 0
    rank = len(dims)
    for k in range(rank):
        tail = 1
        for n in dims[k + 1:]:
            tail = tail * int(n)
        flat = flat + np.asarray(indices[k], dtype=np.int64) * tail
    return flat


def unflatten_index(flat, dims):
    """lego/lego.py:112-136 -- successive quotient by the tail product, then
    remainder; the leading index is not wrapped."""
    if not dims:
        return ()
    out = []
    cur = np.asarray(flat, dtype=np.int64)
    rank = len(dims)
    for k in range(rank):
        tail = 1
        for n in dims[k + 1:]:
            tail = tail * int(n)
        out.append(cur // tail)
        cur = cur % tail
    return tuple(out)


def _sigma(values, perm):
    """lego/lego.py:181-186 -- new[i] = values[perm[i]]."""
    return [values[p] for p in perm]


def _inverse_permutation(perm):
    """lego/lego.py:189-194."""
    inv = [0] * len(perm)
    for i, p in enumerate(perm):
        inv[p] = i
    return inv


def _antidiag(n, idx):
    """lego/lego.py:490-506 -- anti-diagonal numbering of an n x n square."""
    i, j = (np.asarray(v, dtype=np.int64) for v in idx)
    a = i + j + 1
    upper = (a * (a - 1) // 2) + i
    lower = (n * n - n) + i - ((2 * n - a) * (2 * n - a - 1) // 2)
    return np.where(a <= n, upper, lower)


def _reverse(n1, n2, idx):
    """lego/lego.py:534-535 -- (n1-1-i)*n2 + n2-1-j."""
    i, j = (np.asarray(v, dtype=np.int64) for v in idx)
    return (n1 - 1 - i) * n2 + n2 - 1 - j


def _callable_table(block):
    """GenP.apply, lego/lego.py:168-171, for an arbitrary user callable: f_apply at every
    index of the block, one scalar call at a time, in row-major order of the block's dims."""
    if "_table" not in block:
        dims = [int(d) for d in block["dims"]]
        size = 1
        for d in dims:
            size *= d
        table = np.empty(size, dtype=np.int64)
        for r in range(size):
            idx, rest = [], r
            for d in reversed(dims):
                idx.append(rest % d)
                rest //= d
            table[r] = int(block["f_apply"](tuple(reversed(idx))))
        block["_table"] = table
    return block["_table"]


def block_apply(block, idx):
    """RegP.apply, lego/lego.py:215-218 (GenP.apply :168-171 for the two bodies
    the reference ships)."""
    dims = block["dims"]
    if len(idx) != len(dims):
        raise ValueError("Input index dimension mismatch")
    kind = block.get("kind", "regp")
    if kind == "regp":
        return flatten_index(_sigma(list(idx), block["perm"]), _sigma(dims, block["perm"]))
    if kind == "antidiag":
        return _antidiag(dims[0], idx)
    if kind == "reverse":
        return _reverse(dims[0], dims[1], idx)
    if kind == "callable":
        return _callable_table(block)[flatten_index(list(idx), dims)]
    raise ValueError(kind)


def block_inv(block, flat):
    """RegP.inv, lego/lego.py:220-224."""
    kind = block.get("kind", "regp")
    dims = block["dims"]
    if kind == "regp":
        moved = unflatten_index(flat, _sigma(dims, block["perm"]))
        return tuple(_sigma(list(moved), _inverse_permutation(block["perm"])))
    if kind == "reverse":
        w = dims[0] * dims[1] - 1 - np.asarray(flat, dtype=np.int64)
        return (w // dims[1], w % dims[1])
    if kind == "antidiag":
        # brute-force table: the oracle only needs to be right, not fast
        n = dims[0]
        ii, jj = np.indices((n, n))
        table = np.empty(n * n, dtype=np.int64)
        table[_antidiag(n, (ii.ravel(), jj.ravel()))] = np.arange(n * n)
        cell = table[np.asarray(flat, dtype=np.int64)]
        return (cell // n, cell % n)
    if kind == "callable":
        # GenP.inv, lego/lego.py:173-174, is the user's f_inv; the oracle inverts f_apply by
        # brute force instead, which also holds a wrong f_inv to account
        fwd = _callable_table(block)
        back = np.empty_like(fwd)
        back[fwd] = np.arange(fwd.size)
        return unflatten_index(back[np.asarray(flat, dtype=np.int64)], dims)
    raise ValueError(kind)


def _size(block):
    out = 1
    for d in block["dims"]:
        out *= int(d)
    return out


def orderby_dims(stage):
    """OrderBy._compute_dims, lego/lego.py:351-358."""
    return [d for b in stage for d in b["dims"]]


def orderby_apply(stage, idx):
    """OrderBy.apply, lego/lego.py:288-316."""
    if len(idx) != len(orderby_dims(stage)):
        raise ValueError("Input index length must match combined dimension length")
    out = 0
    at = 0
    for b in stage:
        r = len(b["dims"])
        out = out * _size(b) + block_apply(b, idx[at:at + r])
        at += r
    return out


def orderby_inv(stage, flat):
    """OrderBy.inv, lego/lego.py:318-349."""
    rem = np.asarray(flat, dtype=np.int64)
    found = []
    for b in reversed(stage):
        n = _size(b)
        cur = rem % n
        rem = rem // n
        found = list(block_inv(b, cur)) + found
    return tuple(found)


def groupby_apply(spec, idx):
    """GroupBy.apply, lego/lego.py:388-404."""
    dims = spec["dims"]
    if len(idx) != len(dims):
        raise ValueError("Input index dimension mismatch")
    flat = flatten_index(idx, dims)
    for stage in reversed(spec["objects"]):
        flat = orderby_apply(stage, unflatten_index(flat, orderby_dims(stage)))
    return np.asarray(flat, dtype=np.int64)


def groupby_inv(spec, flat):
    """GroupBy.inv, lego/lego.py:406-421 (the numeric content; :422-433 only
    simplifies the resulting expressions)."""
    cur = np.asarray(flat, dtype=np.int64)
    for stage in spec["objects"]:
        sd = orderby_dims(stage)
        if not sd:
            continue
        cur = flatten_index(orderby_inv(stage, cur), sd)
    return unflatten_index(cur, spec["dims"])


def groupby_apply_all(spec):
    """apply over the whole logical domain, row-major (what the loop of
    lego/lego_mlir.py:85-108 enumerates)."""
    n = 1
    for d in spec["dims"]:
        n *= int(d)
    ids = np.arange(n, dtype=np.int64)
    return groupby_apply(spec, unflatten_index(ids, spec["dims"]))


# --------------------------------------------------------------------------
# layout-driven data movement
# --------------------------------------------------------------------------

def permute(x_flat: np.ndarray, src_spec, dst_spec) -> np.ndarray:
    """out[dst(idx)] = in[src(idx)] over the common logical domain: the
    TB[...] = TA[...] assignment of benchmarks/mlir/transpose_naive.py:55-58,
    with MLIRTensor.__getitem__/__setitem__ (lego/lego_mlir.py:363-390)
    addressing through the layouts."""
    if list(src_spec["dims"]) != list(dst_spec["dims"]):
        raise ValueError("src and dst layouts must share the logical domain")
    s = groupby_apply_all(src_spec)
    d = groupby_apply_all(dst_spec)
    out = np.empty_like(x_flat)
    out[d] = x_flat[s]
    return out


# --------------------------------------------------------------------------
# tile orders
# --------------------------------------------------------------------------

def grouped_swizzle(pid, num_pid_m, num_pid_n, gm):
    """The expression the reference prints for (pid_m, pid_n),
    triton_generated/matmul/matmul_NTA_NTB.py:108-109."""
    pid = np.asarray(pid, dtype=np.int64)
    g = min(gm, num_pid_m)
    pid_m = pid % g + ((pid // (num_pid_n * g)) % max(1, num_pid_m // gm)) * g
    pid_n = (pid % (num_pid_n * g)) // g
    return pid_m, pid_n


def grouped_tiles(mnk, bm, bn):
    """Flat tile id -> (group, tile_m, tile_n) in the order the persistent loop of
    triton_generated/grouped_gemm/grouped_gemm.py:60-82 visits tiles."""
    out = []
    for g, (m, n, _k) in enumerate(mnk):
        num_m = -(-m // bm)
        num_n = -(-n // bn)
        for t in range(num_m * num_n):
            out.append((g, t // num_n, t % num_n))
    return out


# --------------------------------------------------------------------------
# floating-point paths (torch CPU, fp32): what the reference asserts against
# --------------------------------------------------------------------------

def softmax(x):
    """triton_generated/softmax/softmax.py:240 checks against torch.softmax;
    fp16 inputs are evaluated in fp32 and rounded once."""
    import torch
    return torch.softmax(x.float(), dim=-1).to(x.dtype)


def layernorm_fwd(x, gamma, beta, eps, round_output=True):
    """triton_generated/layernorm/layernorm.py:421 checks against F.layer_norm;
    mean / rstd as the kernel of :71-87 defines them (biased variance).  With
    round_output=False y stays fp32, for error bounds below one output ulp."""
    import torch
    xf = x.float()
    mean = xf.mean(dim=-1)
    var = ((xf - mean[:, None]) ** 2).mean(dim=-1)
    rstd = 1.0 / torch.sqrt(var + eps)
    y = (xf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()
    return (y.to(x.dtype) if round_output else y), mean, rstd


def layernorm_bwd(dy, x, gamma, mean, rstd):
    """Gradients as _lego_layer_norm_bwd_dx_fused / _bwd_dwdb define them,
    triton_generated/layernorm/layernorm.py:163-267."""
    xf, dyf, w = x.float(), dy.float(), gamma.float()
    n = x.shape[-1]
    xhat = (xf - mean[:, None]) * rstd[:, None]
    wdy = w * dyf
    c1 = (xhat * wdy).sum(dim=-1, keepdim=True) / n
    c2 = wdy.sum(dim=-1, keepdim=True) / n
    dx = (wdy - (xhat * c1 + c2)) * rstd[:, None]
    dw = (dyf * xhat).sum(dim=0)
    db = dyf.sum(dim=0)
    return dx.to(x.dtype), dw.to(gamma.dtype), db.to(gamma.dtype)


def matmul(a, b, activation=""):
    """triton_generated/matmul/matmul_NTA_NTB.py:252 checks against torch.matmul;
    fp32 accumulation of the fp16 inputs, optional leaky_relu (:125-127)."""
    import torch
    c = a.float() @ b.float()
    if activation == "leaky_relu":
        c = torch.where(c >= 0, c, 0.01 * c)
    return c


def grouped_matmul(group_a, group_b):
    """triton_generated/grouped_gemm/grouped_gemm.py:346."""
    return [a.float() @ b.float() for a, b in zip(group_a, group_b)]
