"""Shared helpers of the parity tests: seeded inputs, error metrics, the per-case report."""
import json
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tolerances of the parity bar.  3xTF32 (default math): max relative error <= 1e-4; plain TF32 is
# reported separately against 5e-3.  "Relative" is taken two ways, both must hold:
#   normwise      max|a-b| / max|b|
#   componentwise max(|a-b| / sum|x||w|), the denominator of the standard forward-error bound of a
#                 dot product (zero-mean inputs make |b| itself pass through zero)
TOL = {"3xtf32": dict(norm=1e-4, comp=1e-5), "tf32": dict(norm=5e-3, comp=2e-3)}


def out_hw(IH, IW, FH, FW, sh, sw, ph, pw):
    return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1


def gen(shape, dist, rng):
    if dist == "u11":
        return rng.uniform(-1, 1, shape).astype(np.float32)
    if dist == "u01":
        return rng.uniform(0, 1, shape).astype(np.float32)
    if dist == "n01":
        return rng.standard_normal(shape).astype(np.float32)
    if dist == "relu":
        return np.maximum(rng.standard_normal(shape), 0).astype(np.float32)
    raise ValueError(dist)


FLOOR_TAU = 1e-3


def floor_rel(got, ref64):
    """max |a-b| / max(|b|, tau * max|b|), tau = 1e-3: the relative error of every element, with the
    denominators of the elements that pass through zero (zero-mean inputs) floored at a thousandth of
    the largest reference value."""
    ref64 = np.asarray(ref64, np.float64)
    err = np.abs(np.asarray(got, np.float64) - ref64)
    big = max(float(np.abs(ref64).max()), 1e-30)
    return float((err / np.maximum(np.abs(ref64), FLOOR_TAU * big)).max())


def metrics(got, ref64, S):
    got = np.asarray(got, np.float64)
    err = np.abs(got - ref64)
    norm = float(err.max() / max(np.abs(ref64).max(), 1e-30))
    comp = float((err / np.maximum(S, 1e-30)).max())
    return dict(norm=norm, comp=comp, floor_rel=floor_rel(got, ref64), max_abs=float(err.max()),
                finite=bool(np.isfinite(got).all()))


_REPORT = []


def worst_floor_rel():
    """Largest floor-relative error per math mode over every case recorded so far."""
    worst = {}
    for e in _REPORT:
        mode = e.get("mode", "3xtf32")
        for v in e.values():
            if isinstance(v, dict) and "floor_rel" in v:
                worst[mode] = max(worst.get(mode, 0.0), v["floor_rel"])
    return worst


def record(entry):
    """Appends one case to the parity report (diagnostics for a failed run).  The report is written as
    JSON only where ALPHA_PARITY_REPORT names a file."""
    _REPORT.append(entry)
    out = os.environ.get("ALPHA_PARITY_REPORT")
    if not out:
        return
    try:
        os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
        with open(out, "w") as f:
            json.dump(_REPORT, f, indent=1)
    except OSError:
        pass
