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


def metrics(got, ref64, S):
    got = np.asarray(got, np.float64)
    err = np.abs(got - ref64)
    norm = float(err.max() / max(np.abs(ref64).max(), 1e-30))
    comp = float((err / np.maximum(S, 1e-30)).max())
    return dict(norm=norm, comp=comp, max_abs=float(err.max()), finite=bool(np.isfinite(got).all()))


_REPORT = []


def record(entry):
    """Appends one case to the parity report written at the end of the run (diagnostics for a failed run)."""
    _REPORT.append(entry)
    out = os.path.join(ROOT, "gpurun_out")
    try:
        os.makedirs(out, exist_ok=True)
        with open(os.path.join(out, "parity_report.json"), "w") as f:
            json.dump(_REPORT, f, indent=1)
    except OSError:
        pass
