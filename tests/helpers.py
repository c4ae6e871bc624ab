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
