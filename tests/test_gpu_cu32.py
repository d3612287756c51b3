"""GPU parity against the reference's own cu32 kernels rebuilt for sm_100 ("cu32 outputs").

oracle/build_ref_gpu.sh compiles the reference's three CUDA libraries where its checkout exists;
the built libraries travel with the repository snapshot.  Where they are missing the tests skip.
Bar: max|ours - cu32| / max|cu32| <= 1e-4 in 3xTF32 mode, 5e-3 in TF32 mode, on identical seeded
inputs, plus the reference's own samePercentRelative thresholds on positive inputs.
"""
import zlib

import numpy as np
import pytest

from helpers import gen, out_hw, record

pytestmark = pytest.mark.gpu

# shapes obey the natives' contract: N, IC, OC multiples of 4, GK >= 8
CASES = {
    "cfg1": (4, 32, 32, 16, 32, 3, 3, 1, 1, 1, 1),
    "s1_64_64": (8, 14, 14, 64, 64, 3, 3, 1, 1, 1, 1),
    "s1_128_256_V2": (64, 7, 7, 128, 256, 3, 3, 1, 1, 1, 1),
    "s2_3x3": (8, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
    "s2_4x4_deconv": (8, 16, 16, 32, 64, 4, 4, 2, 2, 1, 1),
    "w1": (8, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "5x5": (4, 12, 12, 32, 36, 5, 5, 1, 1, 2, 2),
    "small_ic_crossadd": (4, 16, 16, 4, 32, 3, 3, 1, 1, 1, 1),
    "nopad": (4, 10, 10, 32, 32, 3, 3, 1, 1, 0, 0),
}


@pytest.fixture(scope="module")
def ref():
    import torch
    from oracle import cu32_ref
    if not cu32_ref.available():
        pytest.skip("oracle/_ref/libcu32_*.so not built (needs the reference checkout)")
    torch.cuda.set_device(0)
    return cu32_ref.Cu32Reference()


@pytest.fixture(scope="module")
def eng(pkg):
    return pkg.submodule("engine").Engine()


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(CASES))
def test_against_cu32_outputs(pkg, eng, ref, oracle_mod, name, mode):
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 7)
    dev = torch.device("cuda:0")
    X, W, dY = (torch.from_numpy(a).to(dev) for a in (gen((N, IH, IW, IC), "u11", rng), gen((OC, FH, FW, IC), "u11", rng),
                                                      gen((N, OH, OW, OC), "n01", rng)))
    got = dict(fwd=eng.conv3D(X, W, sh, sw, ph, pw), dx=eng.dconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw),
               dw=eng.dconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw))
    assert lib.device_status() == 0
    want = dict(fwd=ref.conv3D(X, W, sh, sw, ph, pw))
    k_fwd = ref.last
    want["dx"] = ref.dconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
    k_dx = ref.last
    want["dw"] = ref.dconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    tol = 1e-4 if mode == "3xtf32" else 5e-3
    # The Pascal-era kernels are not reliable on sm_100 for every shape (deltaX_s1_texture returns
    # wrong numbers for this file's s1_64_64 inputs): an op counts only where cu32 agrees with the
    # reference's own CPU loop; where it does not, ours must agree with the CPU loop instead.
    Xn, Wn, dYn = X.cpu().numpy(), W.cpu().numpy(), dY.cpu().numpy()
    cpu = dict(fwd=O.conv3D_f64(Xn, Wn, sh, sw, ph, pw, threads=8)[0],
               dx=O.deconv3D_deltaX_f64(dYn, Wn, IH, IW, sh, sw, ph, pw, threads=8)[0],
               dw=O.deconv3D_deltaW_f64(Xn, dYn, FH, FW, sh, sw, ph, pw, threads=8)[0])
    errs, cu32_ok = {}, {}
    for op in ("fwd", "dx", "dw"):
        a, b, c = got[op].double().cpu().numpy(), want[op].double().cpu().numpy(), cpu[op]
        cu32_ok[op] = bool(np.abs(b - c).max() <= 1e-3 * np.abs(c).max())
        errs[op] = float(np.abs(a - b).max() / np.abs(b).max()) if cu32_ok[op] else float(np.abs(a - c).max() / np.abs(c).max())
    record(dict(case=name, mode=mode, vs="cu32", ref_kernels=[k_fwd, k_dx, ref.last], cu32_agrees_with_cpu=cu32_ok, **errs))
    for op in ("fwd", "dx", "dw"):
        assert errs[op] <= tol, (op, errs, cu32_ok)


def test_reference_thresholds_against_cu32(pkg, eng, ref, oracle_mod):
    """Positive inputs, the reference's own acceptance test applied between the two GPU results."""
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    N, IH, IW, IC, OC = 8, 16, 16, 64, 64
    rng = np.random.default_rng(99)
    dev = torch.device("cuda:0")
    X, W, dY = (torch.from_numpy(gen(s, "u01", rng)).to(dev) for s in ((N, IH, IW, IC), (OC, 3, 3, IC), (N, IH, IW, OC)))
    assert O.samePercentRelative(ref.conv3D(X, W, 1, 1, 1, 1).cpu().numpy(), eng.conv3D(X, W, 1, 1, 1, 1).cpu().numpy(), 1e-5) >= 0.999
    assert O.samePercentRelative(ref.dconv3D_deltaX(dY, W, IH, IW, 1, 1, 1, 1).cpu().numpy(),
                                 eng.dconv3D_deltaX(dY, W, IH, IW, 1, 1, 1, 1).cpu().numpy(), 1e-4) >= 0.999
    assert O.samePercentRelative(ref.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1).cpu().numpy(),
                                 eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1).cpu().numpy(), 1e-5) == 1.0
