"""Shared test helpers: bridge product layouts to the oracle's plain specs and
evaluate the reference's printed index strings numerically."""
import types

import numpy as np

import lego_b200 as L


def build_layout(src: str, env=None, genp_kind=None):
    """Build a lego_b200 layout from the source string stored in the golden file.  The same
    string builds the layout with the reference's classes.  ``genp_kind`` tags every GenP
    block with a closed form the device evaluator knows (the strings themselves, shared with
    the reference, give only the callables, which lower to look-up tables)."""
    def genp(dims, f_apply, f_inv):
        return L.GenP(dims, f_apply, f_inv, kind=genp_kind)
    ns = {"Row": L.Row, "Col": L.Col, "RegP": L.RegP, "OrderBy": L.OrderBy, "GenP": genp,
          "antidiag": L.antidiag, "antidiag_inv": L.antidiag_inv, "new_antidiag": L.new_antidiag}
    if env:
        ns.update(env)
    return eval(src, ns)


def golden_spec(g: dict) -> dict:
    """The oracle spec stored with a golden layout; a GenP recorded by the source of its
    ``f_apply`` gets the callable back."""
    spec = {"dims": list(g["spec"]["dims"]), "objects": []}
    for stage in g["spec"]["objects"]:
        out = []
        for b in stage:
            b = dict(b)
            if b.get("kind") == "callable":
                b["f_apply"] = eval(b.pop("f_apply_src"))
            out.append(b)
        spec["objects"].append(out)
    return spec


def genp_kind_of(g: dict):
    """"antidiag" / "reverse" when every GenP block of a golden layout is that closed form."""
    kinds = {b["kind"] for stage in g["spec"]["objects"] for b in stage if b["kind"] != "regp"}
    return kinds.pop() if len(kinds) == 1 and kinds <= {"antidiag", "reverse"} else None


def same_structure(spec_a: dict, spec_b: dict) -> bool:
    """Dims, stages, block dims and RegP permutations agree (GenP bodies are compared by value elsewhere)."""
    if spec_a["dims"] != spec_b["dims"] or len(spec_a["objects"]) != len(spec_b["objects"]):
        return False
    for sa, sb in zip(spec_a["objects"], spec_b["objects"]):
        if len(sa) != len(sb):
            return False
        for a, b in zip(sa, sb):
            if a["dims"] != b["dims"] or (a["kind"] == "regp") != (b["kind"] == "regp"):
                return False
            if a["kind"] == "regp" and a["perm"] != b["perm"]:
                return False
    return True


def eval_c_string(text: str, env: dict):
    """Evaluate an index expression as LEGOCCodePrinter prints it: integer ``/`` and the
    ``cond ? a : b`` of a Piecewise (at most one, at the top level, which is all the
    reference's programs contain)."""
    t = " ".join(text.split())

    def strip(e):
        e = e.strip()
        while e.startswith("(") and _matching(e, 0) == len(e) - 1:
            e = e[1:-1].strip()
        return e

    t = strip(t)
    depth, q, c = 0, -1, -1
    for pos, ch in enumerate(t):
        depth += ch == "("
        depth -= ch == ")"
        if depth == 0 and ch == "?" and q < 0:
            q = pos
        if depth == 0 and ch == ":" and q >= 0:
            c = pos
    py = (lambda e: eval(strip(e).replace("/", "//"), {}, dict(env)))
    if q < 0:
        return py(t)
    cond, a, b = t[:q], t[q + 1:c], t[c + 1:]
    return np.where(py(cond), py(a), py(b))


def _matching(e: str, start: int) -> int:
    depth = 0
    for pos in range(start, len(e)):
        depth += e[pos] == "("
        depth -= e[pos] == ")"
        if depth == 0:
            return pos
    return -1


from oracle.lego_oracle import spec_of  # noqa: E402,F401  (structure-only bridge from a layout object to an oracle spec)


def unravel(ids, dims):
    ids = np.asarray(ids, dtype=np.int64)
    return [np.asarray(v, dtype=np.int64) for v in np.unravel_index(ids, dims)]


def eval_reference_string(text: str, env: dict):
    """Evaluate an index expression as the reference prints it into Triton code."""
    tl = types.SimpleNamespace(arange=lambda a, b: np.arange(a, b, dtype=np.int64))
    ns = {"tl": tl, "min": min, "max": max}
    ns.update(env)
    return eval(text, ns)
