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


def _dw_shapes(seed, count):
    """Shapes that reach the halo-tile deltaW kernel's forms: 32-channel multiples, strides 1 and 2 in either
    direction, filter rows of 1 to 7 taps, odd images whose stride lattices differ in length."""
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < count:
        N = int(rng.integers(1, 7))
        FH, FW = int(rng.choice([1, 2, 3, 3, 4, 5, 7])), int(rng.choice([1, 2, 3, 3, 4, 5, 7]))
        sh, sw = int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 2]))
        ph, pw = int(rng.integers(0, FH)), int(rng.integers(0, FW))
        OH, OW = int(rng.integers(1, 30)), int(rng.integers(1, 30))
        IH = (OH - 1) * sh + FH - 2 * ph + int(rng.integers(0, sh))
        IW = (OW - 1) * sw + FW - 2 * pw + int(rng.integers(0, sw))
        if IH < sh or IW < sw or IH < 1 or IW < 1:
            continue
        IC = 32 * int(rng.choice([1, 1, 2, 4, 8])); OC = 4 * int(rng.integers(1, 72))
        out.append((N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, OH, OW))
    return out


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_random_deltaW_forms(pkg, oracle_mod, mode):
    import torch
    eng = pkg.submodule("engine").Engine()
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    O = oracle_mod
    dev = torch.device("cuda:0")
    tol = TOL[mode]
    bad, seen = [], set()
    try:
        for i, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, OH, OW) in enumerate(_dw_shapes(77, 60)):
            rng = np.random.default_rng(5000 + i)
            X = gen((N, IH, IW, IC), "relu", rng); dY = gen((N, OH, OW, OC), "n01", rng)
            dW = eng.dconv3D_deltaW(torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev), FH, FW, sh, sw, ph, pw).cpu().numpy()
            algo, plan = lib.last_algo(), lib.last_plan()
            assert lib.device_status() == 0, (i, algo, plan)
            if algo.startswith("dw_halo"):
                seen.update(k for k in ("strided", "2 phases", "tap groups", "stacked", "diagonal") if k in plan)
            m = metrics(dW, *O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8))
            record(dict(case="random_dw_%d" % i, shape=(N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), mode=mode, dw_algo=algo, dw=m))
            if not (m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"]):
                bad.append((i, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), algo, plan, m["norm"], m["comp"]))
    finally:
        lib.set_math_mode("3xtf32")
    assert not bad, bad
    assert {"strided", "2 phases", "tap groups"} <= seen, seen     # the sample reaches the forms it is meant for


GUARD_FLOATS = 1024      # 4 KB of poison on either side of every output


def _guarded(shape, dev):
    """An output tensor carved out of the middle of a poisoned buffer: (view, whole buffer)."""
    import torch
    n = int(np.prod(shape))
    whole = torch.full((n + 2 * GUARD_FLOATS,), float("nan"), device=dev)
    whole.view(torch.int32).fill_(0x7FC0DEAD)      # a NaN with a payload no kernel produces
    return whole[GUARD_FLOATS:GUARD_FLOATS + n].view(shape), whole


def _bands_intact(whole):
    bits = whole.view(np.int32) if isinstance(whole, np.ndarray) else whole.view(__import__("torch").int32)
    head, tail = bits[:GUARD_FLOATS], bits[-GUARD_FLOATS:]
    return bool((head == 0x7FC0DEAD).all()) and bool((tail == 0x7FC0DEAD).all())


EXTRA_GUARD_SHAPES = [
    (8, 28, 28, 128, 128, 3, 3, 1, 1, 1, 1),     # CTA-pair kernel
    (4, 7, 7, 512, 512, 3, 3, 1, 1, 1, 1),       # stacked images, 256-column tiles
    (8, 2, 2, 512, 512, 3, 3, 1, 1, 1, 1),       # patch matrix + split-K
    (8, 16, 16, 64, 128, 3, 3, 2, 2, 1, 1),      # stride 2: col2im deltaX, im2col forward and deltaW
    (4, 32, 32, 4, 64, 7, 7, 2, 2, 3, 3),        # IC = 4 stem
    (3, 13, 11, 36, 20, 3, 3, 1, 1, 1, 1),       # odd everything
    (4, 16, 16, 32, 64, 4, 4, 2, 2, 1, 1),       # 4x4 stride 2 (deconvolution)
]


def test_outputs_stay_inside_their_buffers(pkg):
    """Every output (Y, deltaX, deltaW) lies between two poisoned guard bands: no kernel, TMA store or helper
    of any selection path may write a byte outside the tensor it was given, and it must write all of it."""
    import torch
    base = pkg.submodule("engine").CudaFloat32EngineBase()
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(9)
    shapes = [s for s in _shapes(77, 30) if s[3] % 4 == 0 and s[4] % 4 == 0] + EXTRA_GUARD_SHAPES
    for mode in ("3xtf32", "tf32"):
        lib.set_math_mode(mode)
        for (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) in shapes:
            OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
            X = torch.randn((N, IH, IW, IC), device=dev, generator=g)
            W = torch.randn((OC, FH, FW, IC), device=dev, generator=g)
            dY = torch.randn((N, OH, OW, OC), device=dev, generator=g)
            Y, Yw = _guarded((N, OH, OW, OC), dev)
            dX, dXw = _guarded((N, IH, IW, IC), dev)
            dW, dWw = _guarded((OC, FH, FW, IC), dev)
            base.conv3D(Y, OH, OW, X, IH, IW, W, FH, FW, N, IC, OC, sh, sw, ph, pw)
            a1 = lib.last_algo()
            base.dconv3D_deltaX(dX, IH, IW, dY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw)
            a2 = lib.last_algo()
            base.dconv3D_deltaW(dW, FH, FW, X, IH, IW, dY, OH, OW, N, IC, OC, sh, sw, ph, pw)
            a3 = lib.last_algo()
            torch.cuda.synchronize()
            tag = (mode, (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), a1, a2, a3)
            assert _bands_intact(Yw) and _bands_intact(dXw) and _bands_intact(dWw), tag
            assert bool(torch.isfinite(Y).all()) and bool(torch.isfinite(dX).all()) and bool(torch.isfinite(dW).all()), tag
    lib.set_math_mode("3xtf32")
    assert lib.device_status() == 0


def test_output_channel_sweep(pkg, oracle_mod):
    """oc = 4 .. 192 in steps of 4 on one small layer, the sweep of the reference's own native test driver
    (Cuda_conv3D/test.cuh:980, 1008): every residual column-tile width of every kernel, against the oracle."""
    import torch
    eng = pkg.submodule("engine").Engine()
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    O = oracle_mod
    dev = torch.device("cuda:0")
    N, IH, IW, IC, F = 4, 8, 8, 32, 3
    rng = np.random.default_rng(4)
    X = gen((N, IH, IW, IC), "u11", rng)
    tX = torch.from_numpy(X).to(dev)
    bad = []
    for OC in range(4, 193, 4):
        W = gen((OC, F, F, IC), "u11", rng); dY = gen((N, IH, IW, OC), "n01", rng)
        tW, tdY = torch.from_numpy(W).to(dev), torch.from_numpy(dY).to(dev)
        got = (eng.conv3D(tX, tW, 1, 1, 1, 1).cpu().numpy(), eng.dconv3D_deltaX(tdY, tW, IH, IW, 1, 1, 1, 1).cpu().numpy(),
               eng.dconv3D_deltaW(tX, tdY, F, F, 1, 1, 1, 1).cpu().numpy())
        ref = (O.conv3D_f64(X, W, 1, 1, 1, 1, threads=8), O.deconv3D_deltaX_f64(dY, W, IH, IW, 1, 1, 1, 1, threads=8),
               O.deconv3D_deltaW_f64(X, dY, F, F, 1, 1, 1, 1, threads=8))
        for op, a, (b, S) in zip(("fwd", "dx", "dw"), got, ref):
            m = metrics(a, b, S)
            if not (m["finite"] and m["norm"] <= TOL["3xtf32"]["norm"] and m["comp"] <= TOL["3xtf32"]["comp"]):
                bad.append((OC, op, m["norm"], m["comp"]))
    assert lib.device_status() == 0
    assert not bad, bad
