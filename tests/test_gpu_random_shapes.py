"""Seeded random layer shapes (odd sizes, strides, paddings, channel counts) against the oracle:
exercises the kernel selection - halo, pair, im2col, patch matrix, flat 1x1 views, stride phases,
narrow column tiles, stacked small images, gather kernels - on shapes nobody picked by hand."""
import numpy as np
import pytest

from helpers import TOL, gen, metrics, out_hw, record

pytestmark = pytest.mark.gpu


def _shapes(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < count:
        N = int(rng.integers(1, 10))
        IH, IW = int(rng.integers(1, 21)), int(rng.integers(1, 21))
        IC = int(rng.choice([4, 8, 12, 16, 32, 36, 64, 96, 128]))
        OC = int(rng.choice([4, 8, 20, 32, 64, 72, 128, 256]))
        FH = int(rng.choice([1, 2, 3, 3, 3, 4, 5, 7]))
        FW = FH if rng.random() < 0.7 else int(rng.choice([1, 2, 3, 5]))
        sh = int(rng.choice([1, 1, 1, 2, 2, 3])); sw = sh if rng.random() < 0.8 else int(rng.choice([1, 2]))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
        if OH < 1 or OW < 1:
            continue
        # the engine's deltaX needs (IH + 2 ph - FH) divisible by sh, as the reference does
        if (IH + 2 * ph - FH) % sh or (IW + 2 * pw - FW) % sw:
            continue
        out.append((N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw))
    return out


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_random_shapes(pkg, oracle_mod, mode):
    import torch
    eng = pkg.submodule("engine").Engine()
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    O = oracle_mod
    dev = torch.device("cuda:0")
    tol = TOL[mode]
    bad = []
    for i, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in enumerate(_shapes(2024, 40)):
        OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
        rng = np.random.default_rng(1000 + i)
        X = gen((N, IH, IW, IC), "u11", rng); W = gen((OC, FH, FW, IC), "u11", rng); dY = gen((N, OH, OW, OC), "n01", rng)
        tX, tW, tdY = (torch.from_numpy(a).to(dev) for a in (X, W, dY))
        res = {}
        Y = eng.conv3D(tX, tW, sh, sw, ph, pw).cpu().numpy(); res["fwd_algo"] = lib.last_algo()
        dX = eng.dconv3D_deltaX(tdY, tW, IH, IW, sh, sw, ph, pw).cpu().numpy(); res["dx_algo"] = lib.last_algo()
        dW = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw).cpu().numpy(); res["dw_algo"] = lib.last_algo()
        assert lib.device_status() == 0, (i, res)
        res["fwd"] = metrics(Y, *O.conv3D_f64(X, W, sh, sw, ph, pw, threads=8))
        res["dx"] = metrics(dX, *O.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=8))
        res["dw"] = metrics(dW, *O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8))
        record(dict(case="random_%d" % i, shape=(N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), mode=mode, **res))
        for op in ("fwd", "dx", "dw"):
            m = res[op]
            if not (m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"]):
                bad.append((i, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), op, res[op + "_algo"], m["norm"], m["comp"]))
    assert not bad, bad
