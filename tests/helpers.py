"""Shared test helpers: bridge product layouts to the oracle's plain specs and
evaluate the reference's printed index strings numerically."""
import types

import numpy as np

import lego_b200 as L


def build_layout(src: str, env=None):
    """Build a lego_b200 layout from the source string stored in the golden file."""
    ns = {"Row": L.Row, "Col": L.Col, "RegP": L.RegP, "OrderBy": L.OrderBy}
    if env:
        ns.update(env)
    return eval(src, ns)


def spec_of(layout) -> dict:
    """Oracle spec of a lego_b200 layout (structure only; no product arithmetic)."""
    objects = []
    for o in layout.objects:
        stage = []
        for p in o.perms:
            if isinstance(p, L.RegP):
                stage.append({"kind": "regp", "dims": list(p.dims()), "perm": list(p.permutation)})
            else:
                stage.append({"kind": p.kind, "dims": list(p.dims())})
        objects.append(stage)
    return {"dims": list(layout.dims()), "objects": objects}


def unravel(ids, dims):
    ids = np.asarray(ids, dtype=np.int64)
    return [np.asarray(v, dtype=np.int64) for v in np.unravel_index(ids, dims)]


def eval_reference_string(text: str, env: dict):
    """Evaluate an index expression as the reference prints it into Triton code."""
    tl = types.SimpleNamespace(arange=lambda a, b: np.arange(a, b, dtype=np.int64))
    ns = {"tl": tl, "min": min, "max": max}
    ns.update(env)
    return eval(text, ns)
