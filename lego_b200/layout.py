"""Numeric LEGO layout algebra: the Python API surface of the library.

The objects mirror the reference's layout vocabulary (``lego/lego.py:150-487``):
``Row``/``Col``/``RegP``/``GenP`` permutation blocks, ``OrderBy(...)`` with the
``.OrderBy`` chain, ``.TileBy(*levels)`` and ``.GroupBy(group_dims)``, and the
resulting ``GroupBy`` layout with ``apply``/``inv``/``dims``/``__getitem__``.

Where the reference builds SymPy expressions and prints them into kernel text,
these objects are concrete (integer dims) and evaluate on Python ints or on
numpy int64 arrays with ordinary broadcasting; ``lego_b200.lowering`` turns the
same objects into the descriptor the CUDA kernels consume.  Nothing here runs
on the data path of an op: it is host-side set-up arithmetic.
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Sequence, Tuple

import numpy as np

__all__ = [
    "Row", "Col", "RegP", "GenP", "OrderBy", "GroupBy",
    "flatten_index", "unflatten_index", "get_sigma_perm", "inverse_permutation",
    "antidiag", "antidiag_inv", "new_antidiag", "new_antidiag_inv",
    "get_arange", "divisibility_constraint", "le_constraint", "equal_constraint",
]


# -- constraint helpers (``lego/lego.py:67-85``) -------------------------------
#
# The reference hands these to its simplifier as facts about symbolic sizes.  Sizes here
# are concrete, so a constraint is a fact that can be checked on the spot: the helpers
# return a small record, and ``TileBy`` / ``GroupBy`` raise ``ValueError`` when a
# ``user_constraints`` entry does not hold.

class Constraint:
    def __init__(self, kind: str, lhs, rhs):
        self.kind, self.lhs, self.rhs = kind, lhs, rhs

    def holds(self) -> bool:
        lhs, rhs = int(self.lhs), int(self.rhs)
        if self.kind == "divisible":
            return rhs != 0 and lhs % rhs == 0
        if self.kind == "less":
            return lhs < rhs
        return lhs == rhs

    def __repr__(self):
        op = {"divisible": "%% %s == 0", "less": "< %s", "equal": "== %s"}[self.kind] % (self.rhs,)
        return f"Constraint({self.lhs} {op})"


def divisibility_constraint(lhs, rhs) -> Constraint:
    """``lhs % rhs == 0`` (``lego/lego.py:76-77``)."""
    return Constraint("divisible", lhs, rhs)


def le_constraint(lhs, rhs) -> Constraint:
    """``lhs < rhs`` -- strict, like the reference's helper of this name (``lego/lego.py:80-81``)."""
    return Constraint("less", lhs, rhs)


def equal_constraint(lhs, rhs) -> Constraint:
    """``lhs == rhs`` (``lego/lego.py:84-85``)."""
    return Constraint("equal", lhs, rhs)


def _check_constraints(constraints) -> list:
    out = list(constraints or ())
    for c in out:
        if isinstance(c, Constraint) and not c.holds():
            raise ValueError(f"user constraint does not hold: {c!r}")
    return out


class Arange:
    """Placeholder for ``tl.arange(start, stop)`` as a key item of ``layout[...]``
    (``get_arange``, ``lego/lego.py:67-69``): numerically it is that range of integers,
    broadcast like a slice at the same key position."""

    def __init__(self, start: int, stop: int):
        self.start, self.stop = int(start), int(stop)

    def __repr__(self):
        return f"tl.arange({self.start}, {self.stop})"


def get_arange(start, stop) -> Arange:
    return Arange(start, stop)


def _prod(xs: Iterable[int]) -> int:
    out = 1
    for x in xs:
        out *= int(x)
    return out


def _as_index(x):
    """Ints stay Python ints (exact, unbounded); anything else becomes int64."""
    if isinstance(x, (int, np.integer)):
        return int(x)
    return np.asarray(x, dtype=np.int64)


def get_sigma_perm(d: int, q: int) -> List[int]:
    """Level-major -> dimension-major interleave of ``q`` levels of rank ``d``
    (``lego/lego.py:88-90``): position ``k*q+h`` takes element ``k + d*h``."""
    return [k + d * h for k in range(d) for h in range(q)]


def inverse_permutation(p: Sequence[int]) -> List[int]:
    inv = [0] * len(p)
    for pos, src in enumerate(p):
        inv[src] = pos
    return inv


def _gather(values: Sequence, perm: Sequence[int]) -> list:
    return [values[p] for p in perm]


def flatten_index(indices: Sequence, dims: Sequence[int]):
    """Row-major mixed-radix encode, ``sum_k i_k * prod(dims[k+1:])``
    (``lego/lego.py:93-109``).  Horner form; never mutates its inputs."""
    if len(indices) != len(dims):
        raise ValueError("Number of indices must match number of dimensions")
    flat = 0
    for i, n in zip(indices, dims):
        flat = flat * int(n) + _as_index(i)
    return flat


def unflatten_index(flat, dims: Sequence[int]) -> tuple:
    """Inverse of :func:`flatten_index` (``lego/lego.py:112-136``): the leading
    index is the plain quotient (no wrap), the others are ``// then %``."""
    if not dims:
        return ()
    flat = _as_index(flat)
    out = []
    rest = _prod(dims)
    for n in dims:
        rest //= int(n)
        out.append(flat // rest)
        flat = flat % rest
    return tuple(out)


class _Block:
    """A permutation block: maps a multi-index over ``dims()`` to a flat id."""

    def apply(self, idx):  # pragma: no cover - interface
        raise NotImplementedError

    def inv(self, flat):  # pragma: no cover - interface
        raise NotImplementedError

    def dims(self) -> tuple:  # pragma: no cover - interface
        raise NotImplementedError

    def size(self) -> int:
        return _prod(self.dims())


class RegP(_Block):
    """Regular permutation block (``lego/lego.py:197-228``):
    ``apply(idx) = flatten(sigma(idx), sigma(dims))`` with
    ``sigma(v)[i] = v[perm[i]]``."""

    def __init__(self, dims: Sequence[int], perm: Sequence[int]):
        self._dims = tuple(int(d) for d in dims)
        self.permutation = tuple(int(p) for p in perm)
        if sorted(self.permutation) != list(range(len(self._dims))):
            raise ValueError(f"perm {list(perm)} is not a permutation of rank {len(self._dims)}")
        if any(d <= 0 for d in self._dims):
            raise ValueError("Permutation dimensions cannot be zero")

    def dims(self) -> tuple:
        return self._dims

    def permuted_dims(self) -> tuple:
        return tuple(_gather(self._dims, self.permutation))

    def apply(self, idx):
        if len(idx) != len(self._dims):
            raise ValueError("Input index dimension mismatch")
        return flatten_index(_gather(idx, self.permutation), self.permuted_dims())

    def inv(self, flat):
        moved = unflatten_index(flat, self.permuted_dims())
        return tuple(_gather(moved, inverse_permutation(self.permutation)))

    def __repr__(self):
        return f"RegP({list(self._dims)}, {list(self.permutation)})"


def Row(*dims: int) -> RegP:
    """Identity order: last dim fastest (``lego/lego.py:231-234``)."""
    return RegP(dims, list(range(len(dims))))


def Col(*dims: int) -> RegP:
    """Reversed order: first dim fastest (``lego/lego.py:237-240``)."""
    return RegP(dims, list(range(len(dims)))[::-1])


class GenP(_Block):
    """General permutation block given by a pair of callables
    (``lego/lego.py:150-178``).  ``f_apply`` takes the index tuple and returns
    the flat id; ``f_inv`` takes a flat id and returns the index tuple.  A
    ``kind`` tag names the bodies the device evaluator computes in closed form
    (``"antidiag"``, ``"reverse"``); any other block is tabulated over its domain when
    it is lowered and evaluated on the device by table look-up."""

    def __init__(self, dims: Sequence[int], f_apply: Callable, f_inv: Callable, kind: str | None = None):
        self._dims = tuple(int(d) for d in dims)
        self.f_apply = f_apply
        self.f_inv = f_inv
        self.kind = kind

    def dims(self) -> tuple:
        return self._dims

    def apply(self, idx):
        if len(idx) != len(self._dims):
            raise ValueError("Input index dimension mismatch")
        return self.f_apply(tuple(idx))

    def inv(self, flat):
        return tuple(self.f_inv(flat))

    def __repr__(self):
        return f"GenP({list(self._dims)}, kind={self.kind!r})"


class OrderBy(_Block):
    """Concatenation of permutation blocks (``lego/lego.py:243-362``): the
    blocks' flat ids are the digits of a big-endian mixed-radix number whose
    radices are the blocks' sizes."""

    def __init__(self, *perms: _Block):
        if not perms:
            raise ValueError("OrderBy needs at least one permutation block")
        self.perms = tuple(perms)
        self._dims = tuple(d for p in self.perms for d in p.dims())
        self.q = len(self.perms)
        self.d = len(self.perms[0].dims())
        self.chain: List["OrderBy"] = [self]

    # -- builders -----------------------------------------------------------
    def OrderBy(self, *perms: _Block) -> "OrderBy":
        """Append a further ordering stage; returns the head of the chain, as
        the reference does (``lego/lego.py:261-265``)."""
        self.chain.append(OrderBy(*perms))
        return self

    def GroupBy(self, group_dims: Sequence[Sequence[int]], user_constraints=()) -> "GroupBy":
        return GroupBy(group_dims, list(self.chain), user_constraints)

    def TileBy(self, *levels: Sequence[int], user_constraints=()) -> "GroupBy":
        """View the ordered space as ``q = len(levels)`` nested tilings of a
        rank-``d`` tensor (``lego/lego.py:270-286``).  Logical coordinates are
        level-major ``(tile..., sub-tile..., element...)``.  Stages, first to
        last in ``objects``: each ordering of the chain followed by the block
        that undoes its level/dimension interleave, then the block that turns
        level-major coordinates into the tensor's row-major element id."""
        if not levels:
            raise ValueError("TileBy needs at least one level")
        d = len(levels[0])
        if any(len(lv) != d for lv in levels):
            raise ValueError("all TileBy levels must have the same rank")
        dims = tuple(int(x) for lv in levels for x in lv)
        stages: List[OrderBy] = []
        for o in self.chain:
            interleave = get_sigma_perm(o.d, o.q)
            if len(interleave) != len(o.dims()):
                raise ValueError("all blocks of an OrderBy under TileBy must have the same rank")
            stages.append(o)
            stages.append(OrderBy(RegP(_gather(o.dims(), interleave), inverse_permutation(interleave))))
        stages.append(OrderBy(RegP(dims, get_sigma_perm(d, len(levels)))))
        return GroupBy([dims], stages, user_constraints)

    # -- evaluation ---------------------------------------------------------
    def dims(self) -> tuple:
        return self._dims

    def apply(self, idx):
        if len(idx) != len(self._dims):
            raise ValueError(
                f"Input index length {len(idx)} must match combined dimension length {len(self._dims)}")
        flat = 0
        at = 0
        for p in self.perms:
            r = len(p.dims())
            flat = flat * p.size() + p.apply(tuple(idx[at:at + r]))
            at += r
        return flat

    def inv(self, flat):
        flat = _as_index(flat)
        pieces: list = []
        for p in reversed(self.perms):
            n = p.size()
            pieces = list(p.inv(flat % n)) + pieces
            flat = flat // n
        return tuple(pieces)

    def __repr__(self):
        return "OrderBy(" + ", ".join(map(repr, self.perms)) + ")"


class GroupBy(_Block):
    """A complete layout (``lego/lego.py:365-487``): logical coordinates over
    ``dims()`` are flattened row-major, then pushed through ``objects`` from
    last to first, each stage re-cutting the flat id over its own dims."""

    def __init__(self, group_dims: Sequence[Sequence[int]], objects: Sequence[OrderBy], user_constraints=()):
        self._dims = tuple(int(d) for g in group_dims for d in g)
        self.objects = list(objects)
        self.d = len(group_dims[0])
        self.user_constraints = _check_constraints(user_constraints)

    def dims(self) -> tuple:
        return self._dims

    def size(self) -> int:
        return _prod(self._dims)

    def apply(self, *idx):
        if len(idx) != len(self._dims):
            raise ValueError(
                f"Input index dimension mismatch. Expected {len(self._dims)}, got {len(idx)}")
        flat = flatten_index(idx, self._dims)
        for obj in reversed(self.objects):
            flat = obj.apply(unflatten_index(flat, obj.dims()))
        return flat

    def inv(self, flat) -> tuple:
        """Flat position -> logical coordinates (``lego/lego.py:406-433``)."""
        flat = _as_index(flat)
        for obj in self.objects:
            if not obj.dims():
                continue
            flat = flatten_index(obj.inv(flat), obj.dims())
        return unflatten_index(flat, self._dims)

    def apply_range(self, begin: int = 0, count: int | None = None) -> np.ndarray:
        """``apply`` over logical flat ids ``begin .. begin+count`` (row-major
        over ``dims()``); what ``lego_eval_range`` computes on the device."""
        if count is None:
            count = self.size() - begin
        ids = np.arange(begin, begin + count, dtype=np.int64)
        return np.asarray(self.apply(*unflatten_index(ids, self._dims)), dtype=np.int64)

    def __getitem__(self, key):
        """Numeric form of the reference's offset query (``lego/lego.py:443-487``).
        Each key item is an int, an int array, or a slice.  A slice at key
        position ``p`` becomes an ``arange`` laid on broadcast axis ``p % nd``
        of an ``nd``-dimensional result, ``nd`` being the rank of the first
        stage, exactly where the reference puts its ``tl.arange`` terms."""
        if not isinstance(key, tuple):
            key = (key,)
        if len(key) != len(self._dims):
            raise ValueError(
                f"Input index dimension mismatch. Expected {len(self._dims)}, got {len(key)}")
        nd = len(self.objects[0].dims()) if self.objects else len(self._dims)
        idx = []
        for pos, item in enumerate(key):
            if isinstance(item, (slice, Arange)):
                start = 0 if item.start is None else int(item.start)
                stop = self._dims[pos] if item.stop is None else int(item.stop)
                shape = [1] * nd
                shape[pos % nd] = stop - start
                idx.append(np.arange(start, stop, dtype=np.int64).reshape(shape))
            elif isinstance(item, str) or type(item).__module__.startswith("sympy"):
                return self._symbolic_getitem(key)
            else:
                idx.append(_as_index(item))
        return self.apply(*idx)

    def _symbolic_getitem(self, key):
        """The offset as a SymPy expression in the named coordinates, the form the
        reference returns for printing into kernel text (``lego/lego.py:443-487``).  The
        dims are concrete, so the closed form comes from the library's constant folding
        (one ``stride * ((c // div) % mod)`` term per digit, the div / mod dropped where the
        coordinate's range makes them the identity) instead of a rewrite-rule search.  A
        string names an integer symbol in ``[0, dim)``; a slice or ``get_arange`` becomes a
        ``tl.arange(start, stop)`` function term.  Needs SymPy and a layout that folds."""
        import sympy as sp
        from .lowering import fold
        folded = fold(self)
        if not folded.foldable:
            raise ValueError("this layout does not reduce to digit strides: no closed-form offset expression")
        nd = len(self.objects[0].dims()) if self.objects else len(self._dims)

        class TritonRange(sp.Function):
            """``tl.arange(start, stop)`` laid on broadcast axis ``axis`` of ``nd`` (the
            reference's placeholder of the same name, ``lego/lego.py:10-64``)."""
            is_integer = True

            @classmethod
            def eval(cls, *args):
                return None

            def _sympystr(self, printer):
                a, b, axis, total = (int(v) for v in self.args)
                where = ", ".join(":" if i == axis else "None" for i in range(total))
                return f"((tl.arange({a}, {b}))[{where}])"

        coords = []
        for pos, item in enumerate(key):
            if isinstance(item, str):
                coords.append(sp.Symbol(item, integer=True, nonnegative=True))
            elif isinstance(item, (slice, Arange)):
                start = 0 if item.start is None else int(item.start)
                stop = self._dims[pos] if item.stop is None else int(item.stop)
                coords.append(TritonRange(start, stop, pos % nd, nd))
            else:
                coords.append(sp.sympify(item))
        expr = sp.Integer(0)
        for t in folded.terms:
            c = coords[t.src]
            if t.div != 1:
                c = sp.floor(c / t.div)
            if t.div * t.mod != self._dims[t.src]:
                c = sp.Mod(c, t.mod)
            expr += t.stride * c
        return expr

    def __repr__(self):
        return f"GroupBy(dims={list(self._dims)}, objects={self.objects})"


# -- bodies for GenP ---------------------------------------------------------

def antidiag(n: int, args):
    """Anti-diagonal enumeration of an ``n x n`` square (``lego/lego.py:490-506``):
    cells are numbered along successive anti-diagonals ``i + j = const``."""
    i, j = (_as_index(a) for a in args)
    k = i + j + 1
    upper = (k * (k - 1)) // 2 + i
    m = 2 * n - k
    lower = (n * n - n) + i - (m * (m - 1)) // 2
    if isinstance(k, int):
        return upper if k <= n else lower
    return np.where(k <= n, upper, lower)


def new_antidiag(n1: int, n2: int, args):
    """Point reflection of an ``n1 x n2`` grid, ``(n1-1-i) * n2 + (n2-1-j)``
    (``lego/lego.py:534-535``)."""
    i, j = (_as_index(a) for a in args)
    return (n1 - 1 - i) * n2 + (n2 - 1 - j)


def new_antidiag_inv(n1: int, n2: int, flat):
    """Inverse of :func:`new_antidiag` (the reference gives none; the map is an involution
    on flat ids: ``flat -> n1 * n2 - 1 - flat`` in row-major coordinates)."""
    w = n1 * n2 - 1 - _as_index(flat)
    return w // n2, w % n2


def antidiag_inv(n: int, flat):
    """Inverse of :func:`antidiag` (``lego/lego.py:509-531``).  The lower triangle
    is the point mirror of the upper one, so both halves use one triangular-root
    search; the floating-point root is only a first guess, fixed by exact integer
    comparisons."""
    scalar = isinstance(flat, (int, np.integer))
    f = np.atleast_1d(np.asarray(flat, dtype=np.int64))
    upper = f < n * (n + 1) // 2
    g = np.where(upper, f, n * n - 1 - f)
    k = ((np.sqrt(8.0 * g + 1.0) - 1.0) * 0.5).astype(np.int64) + 1
    for _ in range(2):
        k = np.where(k * (k - 1) // 2 > g, k - 1, k)
        k = np.where((k + 1) * k // 2 <= g, k + 1, k)
    i_m = g - k * (k - 1) // 2
    i = np.where(upper, i_m, n - 1 - i_m)
    diag = np.where(upper, k, 2 * n - k)
    j = diag - 1 - i
    if scalar:
        return int(i[0]), int(j[0])
    return i.reshape(np.shape(flat)), j.reshape(np.shape(flat))
