"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle.

Every case runs the three contractions of one conv layer (forward with bias, deltaX, deltaW) on
seeded inputs and compares with the oracle's fp64 loops under the bounds in helpers.TOL, and - on
positive inputs, as the reference's own tests use - with the reference's samePercentRelative
acceptance thresholds (experiments/test_cuda/Cuda_conv3D_test.java:86-97,
Cuda_dconv3D_dX_test.java:93-100, Cuda_dconv3D_dW_test.java:98-105).
"""
import zlib

import numpy as np
import pytest

from helpers import TOL, gen, metrics, out_hw, record

pytestmark = pytest.mark.gpu

# (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw)
CASES = {
    "cfg1_32x32_ic16_oc32": (4, 32, 32, 16, 32, 3, 3, 1, 1, 1, 1),
    "ic32_oc64_16x16": (8, 16, 16, 32, 64, 3, 3, 1, 1, 1, 1),
    "ic64_oc64_14x14": (8, 14, 14, 64, 64, 3, 3, 1, 1, 1, 1),
    "ic64_oc128_7x7": (12, 7, 7, 64, 128, 3, 3, 1, 1, 1, 1),
    "ic64_oc256_14x14": (8, 14, 14, 64, 256, 3, 3, 1, 1, 1, 1),   # plain TF32 takes the CTA-pair kernel here
    "ic8_oc16_9x7": (4, 9, 7, 8, 16, 3, 3, 1, 1, 1, 1),
    "ic32_oc20_ragged": (4, 11, 13, 32, 20, 3, 3, 1, 1, 1, 1),
    "ic96_oc36_5x5": (4, 12, 12, 96, 36, 5, 5, 1, 1, 2, 2),
    "stride2_3x3": (4, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
    "stride2_4x4_dcgan": (4, 16, 16, 32, 64, 4, 4, 2, 2, 1, 1),
    "w1_1x1": (4, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "nopad_3x3": (4, 10, 10, 32, 32, 3, 3, 1, 1, 0, 0),
    "oc264_two_ntiles": (4, 8, 8, 32, 264, 3, 3, 1, 1, 1, 1),
    "ic4_stem_7x7": (4, 32, 32, 4, 64, 7, 7, 2, 2, 3, 3),
    "ic12_oc12": (4, 8, 8, 12, 12, 3, 3, 1, 1, 1, 1),
    "rect_filter_3x5": (4, 12, 10, 32, 32, 3, 5, 1, 1, 1, 2),
    "asym_stride_2x1": (4, 12, 12, 32, 32, 3, 3, 2, 1, 1, 1),
}


@pytest.fixture(scope="module")
def eng(pkg):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return pkg.submodule("engine").Engine()


def _run_case(pkg, eng, O, name, mode, dists=("u11", "u11", "n01"), tile="auto"):
    import torch
    lib = pkg.submodule("lib")
    lib.set_option("CONV_TILE", tile)
    lib.set_math_mode(mode)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    X = gen((N, IH, IW, IC), dists[0], rng)
    W = gen((OC, FH, FW, IC), dists[1], rng)
    B = rng.uniform(-0.1, 0.1, (OC,)).astype(np.float32)
    dY = gen((N, OH, OW, OC), dists[2], rng)
    dev = torch.device("cuda:0")
    tX, tW, tB, tdY = (torch.from_numpy(a).to(dev) for a in (X, W, B, dY))
    res = {}
    Y = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
    res["fwd_algo"] = lib.last_algo()
    dX = eng.dconv3D_deltaX(tdY, tW, IH, IW, sh, sw, ph, pw)
    res["dx_algo"] = lib.last_algo()
    dW = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw)
    res["dw_algo"] = lib.last_algo()
    status = lib.device_status()
    Y, dX, dW = Y.cpu().numpy(), dX.cpu().numpy(), dW.cpu().numpy()
    Y64, SY = O.conv3D_f64(X, W, sh, sw, ph, pw, threads=8)
    Y64 = Y64 + B.astype(np.float64)
    SY = SY + np.abs(B).astype(np.float64)
    dX64, SX = O.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=8)
    dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
    res.update(case=name, mode=mode, tile=tile, status=status, fwd=metrics(Y, Y64, SY), dx=metrics(dX, dX64, SX),
               dw=metrics(dW, dW64, SW))
    record(res)
    return res, (X, W, B, dY, Y, dX, dW)


@pytest.mark.parametrize("tile", ["im2col", "halo"])
@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(CASES))
def test_layer_parity(pkg, eng, oracle_mod, name, mode, tile):
    """tile: 'im2col' = one TMA load per filter tap, 'halo' = input tile fetched once with its halo
    (stride-1 shapes; others fall back to the per-tap kernel)."""
    res, _ = _run_case(pkg, eng, oracle_mod, name, mode, tile=tile)
    assert res["status"] == 0, "kernel status word %d" % res["status"]
    tol = TOL[mode]
    for op in ("fwd", "dx", "dw"):
        m = res[op]
        assert m["finite"], (op, m)
        assert m["norm"] <= tol["norm"], (op, res[op + "_algo"], m)
        assert m["comp"] <= tol["comp"], (op, res[op + "_algo"], m)


@pytest.mark.parametrize("name", ["cfg1_32x32_ic16_oc32", "ic64_oc64_14x14", "stride2_3x3"])
def test_reference_acceptance_thresholds(pkg, eng, oracle_mod, name):
    """The reference's own pass criteria on its own kind of inputs (uniform [0,1))."""
    O = oracle_mod
    res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, O, name, "3xtf32", dists=("u01", "u01", "u01"))
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    Yo = O.add_bias_row(O.conv3D_naive(X, W, sh, sw, ph, pw, threads=8), B)
    dXo = O.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw, threads=8)
    dWo = O.deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
    assert O.samePercentRelative(Yo, Y, 1e-5) >= 0.999
    assert O.samePercentRelative(dXo, dX, 1e-4) >= 0.999
    assert O.samePercentRelative(dWo, dW, 1e-5) == 1.0


def test_algo_selection(pkg, eng, oracle_mod):
    """Shapes with channel counts that are multiples of 32 must run on the tensor path."""
    res, _ = _run_case(pkg, eng, oracle_mod, "ic64_oc64_14x14", "3xtf32", tile="im2col")
    assert res["fwd_algo"] == "igemm" and res["dx_algo"] == "igemm" and res["dw_algo"].startswith("dw")
    res, _ = _run_case(pkg, eng, oracle_mod, "ic64_oc64_14x14", "3xtf32", tile="halo")
    assert res["fwd_algo"].startswith("halo") and res["dx_algo"].startswith("halo")


# The channel configurations of the benchmark's 3x3 sweep at a batch the oracle finishes in seconds.
# They take kernel forms the smaller cases never reach: CTA pairs with side columns (128- and
# 256-channel blocks), and at 7x7x512 two stacked images per accumulator with 256-column tiles.
BENCH_CASES = {
    "bench_56x56x64": (2, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1),
    "bench_28x28x128": (8, 28, 28, 128, 128, 3, 3, 1, 1, 1, 1),
    "bench_14x14x256": (8, 14, 14, 256, 256, 3, 3, 1, 1, 1, 1),
    "bench_7x7x512": (4, 7, 7, 512, 512, 3, 3, 1, 1, 1, 1),
}
CASES.update(BENCH_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(BENCH_CASES))
def test_bench_channel_configurations(pkg, eng, oracle_mod, name, mode):
    import torch
    lib = pkg.submodule("lib")
    res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, mode, dists=("relu", "n01", "n01"))
    assert res["status"] == 0
    tol = TOL[mode]
    for op in ("fwd", "dx", "dw"):
        m = res[op]
        assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, op, res[op + "_algo"], m)
    # the kernel form must be the one the benchmark's batch-256 launch of this layer takes
    N, IH, IW, IC, OC = CASES[name][:5]
    dev = torch.device("cuda:0")
    old = lib.set_option("SKINNY", 0)    # at this reduced batch the layer has few tiles; the benchmark's batch does not
    try:
        _, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, mode, dists=("relu", "n01", "n01"))
        eng.conv3D(torch.from_numpy(X).to(dev), torch.from_numpy(W).to(dev), 1, 1, 1, 1)
        small = lib.last_plan()
    finally:
        lib.set_option("SKINNY", old)
    big_X = torch.zeros((256, IH, IW, IC), device=dev)
    eng.conv3D(big_X, torch.from_numpy(W).to(dev), 1, 1, 1, 1)
    big = lib.last_plan()
    assert lib.device_status() == 0
    assert res["fwd_algo"].startswith("halo") and big.startswith(("halo", "tapstack")), (res["fwd_algo"], big)
    if "halo_pair" in big:
        assert small == big, (small, big)   # the pair kernel's form does not depend on the batch
    if mode == "3xtf32":
        if OC == 512:
            assert "halo_pair" in big and "three+side" in big and "BN=256" in big and "NI=2" in big, big
        elif OC >= 128:
            assert "halo_pair" in big and "three+side" in big, big
    elif OC % 256 == 0:
        assert "halo_pair" in big, big
    elif OC == 64:
        assert big.startswith("tapstack"), big   # one MMA per filter row


# Few output tiles and a long reduction (deep layers at a small batch): the forward / deltaX kernel
# splits the reduction over otherwise idle SMs and a second kernel adds the partial sums.
SKINNY_CASES = {
    "skinny_2x2x512": (8, 2, 2, 512, 512, 3, 3, 1, 1, 1, 1),
    "skinny_4x4x256": (16, 4, 4, 256, 256, 3, 3, 1, 1, 1, 1),
    "skinny_16x16x128": (4, 16, 16, 128, 128, 3, 3, 1, 1, 1, 1),
    "skinny_1x1_1024": (4, 7, 7, 1024, 256, 1, 1, 1, 1, 0, 0),
    "skinny_ragged_oc": (4, 16, 8, 160, 72, 3, 3, 1, 1, 1, 1),
}
CASES.update(SKINNY_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(SKINNY_CASES))
def test_split_reduction_for_skinny_layers(pkg, eng, oracle_mod, name, mode):
    import re
    import torch
    lib = pkg.submodule("lib")
    res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, mode)
    assert res["status"] == 0
    tol = TOL[mode]
    for op in ("fwd", "dx", "dw"):
        m = res[op]
        assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, op, res[op + "_algo"], m)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    dev = torch.device("cuda:0")
    tX, tW, tB = (torch.from_numpy(a).to(dev) for a in (X, W, B))
    y1 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
    plan = lib.last_plan()
    found = re.search(r"ksplit=(\d+)", plan)
    assert found and int(found.group(1)) > 1, plan
    ks = int(found.group(1))
    # bit-identical repeats (the partial sums are added in a fixed order), in either math mode's one-issuer forms
    y2 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
    if mode == "3xtf32":
        assert torch.equal(y1, y2)
    # the same layer with the reduction in one piece: equal to rounding
    old = lib.set_option("SKINNY", 0)
    try:
        y3 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
        assert "ksplit=1" in lib.last_plan() or "halo_pair" in lib.last_plan(), lib.last_plan()
    finally:
        lib.set_option("SKINNY", old)
    assert float((y1 - y3).abs().max()) <= tol["norm"] * float(y3.abs().max())
    # bias and activation are applied once, by the kernel that adds the partial sums
    ya = eng.conv3D_leakyRelu(tX, tW, tB, 0.1, sh, sw, ph, pw)
    assert "ksplit=%d" % ks in lib.last_plan()
    assert torch.equal(ya, torch.where(y1 > 0, y1, y1 * 0.1)) or float((ya - torch.where(y1 > 0, y1, y1 * 0.1)).abs().max()) <= 1e-6 * float(y1.abs().max())
    assert lib.device_status() == 0


def test_lo_plane_of_w_formed_in_the_kernel_equals_the_presplit_plane(pkg, eng):
    """Option HALO_SPLITB: a 1x1 product in 3xTF32 loads only W and lets the split warps form the lo plane of
    every W tile in shared memory; by default the lo plane comes from a separate pass over W.  Same arithmetic,
    same bits."""
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(31)
    for (N, HW, IC, OC, F, p_) in ((8, 14, 256, 192, 1, 0), (64, 2, 128, 256, 3, 1), (4, 32, 4, 64, 7, 3)):
        s_ = 2 if F == 7 else 1
        X = torch.randn((N, HW, HW, IC), device=dev, generator=g)
        W = torch.randn((OC, F, F, IC), device=dev, generator=g) * 0.1
        b = eng.conv3D(X, W, s_, s_, p_, p_)
        n0 = lib.launch_count(); eng.conv3D(X, W, s_, s_, p_, p_); presplit = lib.launch_count() - n0
        old = lib.set_option("HALO_SPLITB", 1)
        try:
            a = eng.conv3D(X, W, s_, s_, p_, p_)
            n0 = lib.launch_count(); eng.conv3D(X, W, s_, s_, p_, p_); fused = lib.launch_count() - n0
        finally:
            lib.set_option("HALO_SPLITB", old)
        assert torch.equal(a, b), (N, HW, IC, OC, F)
        assert fused == presplit - 1          # the pass over W is gone
    assert lib.device_status() == 0


EDGE_CASES = {
    "one_pixel_image": (4, 1, 1, 32, 32, 3, 3, 1, 1, 1, 1),
    "single_image_tiny": (1, 3, 3, 8, 4, 3, 3, 1, 1, 1, 1),
    "wide_pad_5x5_on_2x2": (4, 2, 2, 32, 32, 5, 5, 1, 1, 2, 2),
    "m_is_one_tile_plus_one": (1, 43, 3, 32, 32, 3, 3, 1, 1, 1, 1),
    "oc4_ic64": (4, 6, 6, 64, 4, 3, 3, 1, 1, 1, 1),
    "stride3_7x7": (4, 20, 20, 32, 32, 7, 7, 3, 3, 3, 3),
    "floor_division_output": (4, 10, 10, 32, 32, 3, 3, 2, 2, 0, 0),
}
CASES.update(EDGE_CASES)


@pytest.mark.parametrize("name", list(EDGE_CASES))
@pytest.mark.parametrize("tile", ["im2col", "halo"])
def test_edge_cases(pkg, eng, oracle_mod, name, tile):
    res, _ = _run_case(pkg, eng, oracle_mod, name, "3xtf32", tile=tile)
    assert res["status"] == 0
    for op in ("fwd", "dx", "dw"):
        m = res[op]
        assert m["finite"] and m["norm"] <= TOL["3xtf32"]["norm"] and m["comp"] <= TOL["3xtf32"]["comp"], (op, m)


def test_golden_vectors(pkg, eng):
    """Outputs of the reference's own compiled CPU loops (tests/golden/conv_golden.npz)."""
    import os
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv_golden.npz"))
    dev = torch.device("cuda:0")
    for name in sorted({k.split("/")[0] for k in g.files}):
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = (int(v) for v in g[name + "/shape"])
        X, W, dY = (torch.from_numpy(g[name + "/" + k]).to(dev) for k in ("X", "W", "dY"))
        Y = eng.conv3D(X, W, sh, sw, ph, pw).cpu().numpy()
        dX = eng.dconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw).cpu().numpy()
        dW = eng.dconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw).cpu().numpy()
        assert lib.device_status() == 0
        for got, key in ((Y, "ref_Y"), (dX, "ref_dX"), (dW, "ref_dW")):
            ref = g[name + "/" + key]
            assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), (name, key)


def test_full_size_adjoint_identity(pkg, eng):
    """At the benchmark's full size (X[256,56,56,64]) the oracle is too slow; the three kernels are
    tied together instead by <conv(X,W), dY> = <X, deltaX(dY,W)> = <W, deltaW(X,dY)>."""
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(11)
    N, HW, Cc = 256, 56, 64
    X = torch.randn((N, HW, HW, Cc), device=dev, generator=gen).relu_()
    W = torch.randn((Cc, 3, 3, Cc), device=dev, generator=gen) * (2.0 / (9 * Cc)) ** 0.5
    dY = torch.randn((N, HW, HW, Cc), device=dev, generator=gen)
    Y = eng.conv3D(X, W, 1, 1, 1, 1)
    dX = eng.dconv3D_deltaX(dY, W, HW, HW, 1, 1, 1, 1)
    dW = eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1)
    assert lib.device_status() == 0

    def dot(a, b):
        return float((a.double() * b.double()).sum())
    a, b, c = dot(Y, dY), dot(X, dX), dot(W, dW)
    scale = float(Y.double().norm() * dY.double().norm()) / (Y.numel() ** 0.5)
    assert abs(a - b) <= 1e-4 * scale and abs(a - c) <= 1e-4 * scale, (a, b, c, scale)
    # linearity in the weights: conv(X, 2W) = 2 conv(X, W) exactly (scaling by 2 is exact in fp32)
    Y2 = eng.conv3D(X, W * 2, 1, 1, 1, 1)
    assert torch.equal(Y2, Y * 2)


def test_run_to_run_reproducibility(pkg, eng):
    """3xTF32 results are bit-identical from run to run (one MMA issuer, fixed reduction order). Plain
    TF32 forward / deltaX alternates W-tile stages between two issuing threads, so its accumulation
    order depends on timing: equal to a few ulps there."""
    import torch
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(23)
    for (N, HW, Cc) in ((64, 56, 64), (64, 28, 128), (32, 14, 256)):
        X = torch.randn((N, HW, HW, Cc), device=dev, generator=gen)
        W = torch.randn((Cc, 3, 3, Cc), device=dev, generator=gen) * 0.05
        dY = torch.randn((N, HW, HW, Cc), device=dev, generator=gen)
        for mode in ("3xtf32", "tf32"):
            lib.set_math_mode(mode)
            runs = [(eng.conv3D(X, W, 1, 1, 1, 1), eng.dconv3D_deltaX(dY, W, HW, HW, 1, 1, 1, 1),
                     eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1)) for _ in range(3)]
            assert lib.device_status() == 0
            for r in runs[1:]:
                for a, b in zip(runs[0], r):
                    if mode == "3xtf32":
                        assert torch.equal(a, b), (N, HW, Cc, mode)
                    else:
                        assert float((a - b).abs().max()) <= 2e-6 * float(a.abs().max()), (N, HW, Cc, mode)
    lib.set_math_mode("3xtf32")


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", ["cfg1_32x32_ic16_oc32", "ic64_oc64_14x14", "ic32_oc20_ragged", "ic64_oc128_7x7", "ic8_oc16_9x7"])
def test_winograd_forward(pkg, eng, oracle_mod, name, mode):
    """Winograd F(2,3) forward variant (3x3, stride 1) against the fp64 loop, same bounds as the
    direct kernels; ragged cases cover odd output widths."""
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 1)
    X = gen((N, IH, IW, IC), "u11", rng)
    W = gen((OC, FH, FW, IC), "u11", rng)
    B = rng.uniform(-0.1, 0.1, (OC,)).astype(np.float32)
    dev = torch.device("cuda:0")
    tX, tW, tB = (torch.from_numpy(a).to(dev) for a in (X, W, B))
    lib.set_algo("winograd")
    try:
        Y = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
        algo = lib.last_algo()
        status = lib.device_status()
    finally:
        lib.set_algo("auto")
    assert status == 0 and algo == "winograd"
    Y64, SY = O.conv3D_f64(X, W, sh, sw, ph, pw, threads=8)
    m = metrics(Y.cpu().numpy(), Y64 + B.astype(np.float64), SY + np.abs(B).astype(np.float64))
    record(dict(case=name, mode=mode, tile="winograd", fwd=m))
    # the transforms add and halve in fp32 before the products: allow twice the direct bound
    assert m["finite"] and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= 2 * TOL[mode]["comp"], m


@pytest.mark.parametrize("pair,mode", [("1", "tf32"), ("1", "3xtf32"), ("2", "3xtf32"), ("3", "3xtf32")])
def test_cta_pair_kernel(pkg, eng, oracle_mod, pair, mode):
    """The cta_group::2 form of the halo kernel (two CTAs per MMA) in plain TF32, wide 3xTF32 and
    three-MMA 3xTF32 (one accumulator, and with the correction terms in side columns), forced on shapes it would not be chosen for, against the oracle."""
    L = pkg.submodule("lib")
    old = L.set_option("HALO_PAIR", int(pair))
    try:
        for name in ("ic64_oc64_14x14", "ic64_oc128_7x7", "ic32_oc64_16x16"):
            res, _ = _run_case(pkg, eng, oracle_mod, name, mode)
            assert res["fwd_algo"].startswith("halo_pair"), res["fwd_algo"]
            tol = TOL[mode]
            for op in ("fwd", "dx"):
                m = res[op]
                assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, op, res[op + "_algo"], m)
    finally:
        L.set_option("HALO_PAIR", old)


def test_pair_kernel_is_chosen_for_256_channel_blocks(pkg, eng, oracle_mod):
    res, _ = _run_case(pkg, eng, oracle_mod, "ic64_oc256_14x14", "tf32")
    assert res["fwd_algo"].startswith("halo_pair"), res["fwd_algo"]
    assert res["fwd"]["norm"] <= TOL["tf32"]["norm"] and res["fwd"]["comp"] <= TOL["tf32"]["comp"], res["fwd"]


# Plain TF32 with few output channels: the taps of a filter row share one MMA (conv_tapstack_kernel).
# (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw)
TAPSTACK_CASES = {
    "ts_56x56x64": (2, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1),        # the benchmark's first layer
    "ts_ragged_oc48": (3, 13, 57, 32, 48, 3, 3, 1, 1, 1, 1),     # OH % 4 != 0, two column blocks of 29, BN % 32 != 0
    "ts_fw2": (2, 7, 29, 96, 64, 3, 2, 1, 1, 1, 0),              # two taps per row, three channel chunks
    "ts_5x5_oc16": (2, 9, 30, 32, 16, 5, 5, 1, 1, 2, 2),         # generic filter width, 16-column tap blocks
    "ts_nopad": (2, 20, 31, 64, 32, 3, 3, 1, 1, 0, 0),
    "ts_oc20": (2, 8, 28, 32, 20, 3, 3, 1, 1, 1, 1),             # output channels not a multiple of 16
    "ts_wide_image": (1, 9, 112, 32, 64, 3, 3, 1, 1, 1, 1),      # four column blocks
    "ts_small": (1, 5, 6, 32, 8, 3, 3, 1, 1, 1, 1),              # two partly filled tiles
}
CASES.update(TAPSTACK_CASES)


@pytest.mark.parametrize("name", list(TAPSTACK_CASES))
def test_tap_stacked_kernel(pkg, eng, oracle_mod, name):
    """Forced on every case (option HALO_TAPSTACK = 2), against the oracle under the TF32 bounds, and against
    the tap-by-tap kernels: both truncate the same operands, so they differ only by summation order."""
    import torch
    L = pkg.submodule("lib")
    old = L.set_option("HALO_TAPSTACK", 2)
    try:
        res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, "tf32")
        assert res["status"] == 0
        assert res["fwd_algo"] == "halo_tapstack", res["fwd_algo"]
        for op in ("fwd", "dx"):
            m = res[op]
            assert m["finite"] and m["norm"] <= TOL["tf32"]["norm"] and m["comp"] <= TOL["tf32"]["comp"], (op, res[op + "_algo"], m)
        # bias + LeakyReLU in the epilogue
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
        dev = torch.device("cuda:0")
        tX, tW, tB = (torch.from_numpy(a).to(dev) for a in (X, W, B))
        Ya = eng.conv3D_leakyRelu(tX, tW, tB, 0.1, sh, sw, ph, pw)
        assert L.last_algo() == "halo_tapstack"
        want = np.where(Y > 0, Y, np.float32(0.1) * Y)
        np.testing.assert_array_equal(Ya.cpu().numpy(), want)
        L.set_option("HALO_TAPSTACK", 0)
        Y0 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
        assert L.last_algo() != "halo_tapstack"
        scale = np.abs(Y).max()
        assert np.abs(Y0.cpu().numpy() - Y).max() <= 5e-5 * scale   # the accumulators round once per MMA, in a different order
    finally:
        L.set_option("HALO_TAPSTACK", old)


def test_tap_stacked_kernel_is_chosen_for_the_64_channel_layer(pkg, eng):
    """At the benchmark's batch the planner takes it for forward and deltaX in plain TF32, never in 3xTF32."""
    import torch
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    X = torch.zeros((256, 56, 56, 64), device=dev)
    W = torch.zeros((64, 3, 3, 64), device=dev)
    lib.set_math_mode("tf32")
    try:
        eng.conv3D(X, W, 1, 1, 1, 1)
        assert lib.last_algo() == "halo_tapstack", lib.last_plan()
        eng.dconv3D_deltaX(X, W, 56, 56, 1, 1, 1, 1)
        assert lib.last_algo() == "halo_tapstack", lib.last_plan()
    finally:
        lib.set_math_mode("3xtf32")
    eng.conv3D(X, W, 1, 1, 1, 1)
    assert lib.last_algo() != "halo_tapstack"
    assert lib.device_status() == 0


# CTA-pair kernel with accumulators of 4 rows x 32 patch columns (images at most 30 pixels wide).
FLAT32_CASES = {
    "flat_28x28x128": (4, 28, 28, 128, 128, 3, 3, 1, 1, 1, 1),     # the benchmark's second layer
    "flat_ragged_rows": (4, 13, 30, 64, 128, 3, 3, 1, 1, 1, 1),    # OH % 4 != 0, the widest image the form takes
    "flat_narrow": (6, 9, 5, 32, 64, 3, 3, 1, 1, 1, 1),
    "flat_nopad": (4, 18, 22, 64, 128, 3, 3, 1, 1, 0, 0),
    "flat_oc256": (2, 12, 28, 64, 256, 3, 3, 1, 1, 1, 1),
}
CASES.update(FLAT32_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(FLAT32_CASES))
def test_pair_kernel_with_flat_tiles(pkg, eng, oracle_mod, name, mode):
    """Forced (options HALO_PAIR, HALO_FLAT32) on shapes it would not always be chosen for, against the oracle, and
    bit for bit against the same kernel with 16 x 8 tiles in 3xTF32 (same products, same order per output)."""
    import torch
    L = pkg.submodule("lib")
    old_pair, old_flat = L.set_option("HALO_PAIR", 3 if mode == "3xtf32" else 1), L.set_option("HALO_FLAT32", 2)
    old_skinny = L.set_option("SKINNY", 0)     # at these batches the layers have few tiles; the benchmark's batch does not
    try:
        res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, mode)
        assert res["status"] == 0 and res["fwd_algo"].startswith("halo_pair"), res["fwd_algo"]
        tol = TOL[mode]
        for op in ("fwd", "dx"):
            m = res[op]
            assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, op, res[op + "_algo"], m)
        dev = torch.device("cuda:0")
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
        tX, tW, tB = (torch.from_numpy(a).to(dev) for a in (X, W, B))
        eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
        assert "flat32" in L.last_plan(), L.last_plan()
        L.set_option("HALO_FLAT32", 0)
        Y0 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw).cpu().numpy()
        assert "flat32" not in L.last_plan() and L.last_plan().startswith("halo_pair"), L.last_plan()
        if mode == "3xtf32":
            np.testing.assert_array_equal(Y0, Y)
        else:
            assert np.abs(Y0 - Y).max() <= 5e-5 * np.abs(Y).max()
    finally:
        L.set_option("HALO_PAIR", old_pair)
        L.set_option("HALO_FLAT32", old_flat)
        L.set_option("SKINNY", old_skinny)


def test_flat_tiles_are_chosen_for_28x28(pkg, eng):
    import torch
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    lib.set_math_mode("3xtf32")
    X = torch.zeros((256, 28, 28, 128), device=dev)
    W = torch.zeros((128, 3, 3, 128), device=dev)
    eng.conv3D(X, W, 1, 1, 1, 1)
    assert "halo_pair" in lib.last_plan() and "flat32" in lib.last_plan(), lib.last_plan()
    X = torch.zeros((256, 14, 14, 256), device=dev)
    W = torch.zeros((256, 3, 3, 256), device=dev)
    eng.conv3D(X, W, 1, 1, 1, 1)
    assert "halo_pair" in lib.last_plan() and "flat32" not in lib.last_plan(), lib.last_plan()
    assert lib.device_status() == 0


CASES["flat_odd_blocks"] = (3, 12, 28, 32, 64, 3, 3, 1, 1, 1, 1)     # 3 images x 3 four-row blocks: the last macro tile is half empty


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", [n for n in FLAT32_CASES if n != "flat_narrow"] + ["flat_odd_blocks"])   # flat_narrow fills too few lanes for this kernel
def test_single_cta_kernel_with_flat_tiles(pkg, eng, oracle_mod, name, mode):
    """The single-CTA halo kernel with two flat accumulators per W tile, each with its own patch (the pair kernel is
    switched off), against the oracle and against its 16 x 8 form."""
    import torch
    L = pkg.submodule("lib")
    old = {k: L.set_option(k, v) for k, v in (("HALO_PAIR", 0), ("HALO_FLAT32", 2), ("SKINNY", 0), ("HALO_TAPSTACK", 0))}
    try:
        res, (X, W, B, dY, Y, dX, dW) = _run_case(pkg, eng, oracle_mod, name, mode)
        assert res["status"] == 0 and res["fwd_algo"] in ("halo_row", "halo_tap"), res["fwd_algo"]
        tol = TOL[mode]
        for op in ("fwd", "dx"):
            m = res[op]
            assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, op, res[op + "_algo"], m)
        dev = torch.device("cuda:0")
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
        tX, tW, tB = (torch.from_numpy(a).to(dev) for a in (X, W, B))
        eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw)
        assert "flat32" in L.last_plan(), L.last_plan()
        L.set_option("HALO_FLAT32", 0)
        Y0 = eng.conv3D_biased(tX, tW, tB, sh, sw, ph, pw).cpu().numpy()
        assert "flat32" not in L.last_plan(), L.last_plan()
        if mode == "3xtf32":
            np.testing.assert_array_equal(Y0, Y)
        else:
            assert np.abs(Y0 - Y).max() <= 5e-5 * np.abs(Y).max()
    finally:
        for k, v in old.items():
            L.set_option(k, v)



# deltaW pixel tiles of 7 rows: exact cover of 7, 14, 21, 28 ... pixel high images.  Forced on shapes of every
# kernel form (plain, three-MMA and stacked 3xTF32, the diagonal TF32 form with two half tiles, 8- and 16-column
# tiles, a tile row that ends inside the tile), then the planner's own choice at the benchmark's 7x7x512 layer.
SEVEN_ROW_CASES = {
    "dw7_7x7x64_oc128": (4, 7, 7, 64, 128, 3, 3, 1, 1, 1, 1),
    "dw7_14x14x32_oc64": (3, 14, 14, 32, 64, 3, 3, 1, 1, 1, 1),
    "dw7_21x9x32_oc96": (2, 21, 9, 32, 96, 3, 3, 1, 1, 1, 1),
    "dw7_28x28x32_oc64": (2, 28, 28, 32, 64, 3, 3, 1, 1, 1, 1),
    "dw7_10x12x32": (3, 10, 12, 32, 32, 3, 3, 1, 1, 1, 1),
}
CASES.update(SEVEN_ROW_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(SEVEN_ROW_CASES))
def test_deltaW_with_seven_row_tiles(pkg, eng, oracle_mod, name, mode):
    import torch
    O, lib = oracle_mod, pkg.submodule("lib")
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    X, dY = gen((N, IH, IW, IC), "relu", rng), gen((N, IH, IW, OC), "n01", rng)
    dev = torch.device("cuda:0")
    lib.set_math_mode(mode)
    old = lib.set_option("DW_R", 7)
    try:
        dW = eng.dconv3D_deltaW(torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev), FH, FW, sh, sw, ph, pw).cpu().numpy()
        plan = lib.last_plan()
    finally:
        lib.set_option("DW_R", old)
        lib.set_math_mode("3xtf32")
    assert lib.device_status() == 0
    assert plan.startswith("dw_halo") and "R=7" in plan, plan
    dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
    m = metrics(dW, dW64, SW)
    record(dict(case=name, mode=mode, tile="dw R=7", dw=m))
    assert m["finite"] and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= TOL[mode]["comp"], (plan, m)


def test_seven_row_tiles_are_chosen_where_they_cover_the_image(pkg, eng):
    import torch
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    lib.set_math_mode("tf32")
    try:
        for (N, HW, Cc), want in (((256, 7, 512), "R=7"), ((256, 56, 64), "R=7"), ((256, 14, 256), "R=4"), ((256, 28, 128), "R=4")):
            X, dY = torch.zeros((N, HW, HW, Cc), device=dev), torch.zeros((N, HW, HW, Cc), device=dev)
            dW = eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1)
            plan = lib.last_plan()
            assert plan.startswith("dw_halo") and want in plan, plan
            assert float(dW.abs().max()) == 0.0
    finally:
        lib.set_math_mode("3xtf32")
    assert lib.device_status() == 0


# Strided deltaW on the halo-tile kernel: X through one tensor map per phase of the stride lattice.  Two column
# phases (3x3, 4x4 and 5x5 stride 2), one (1x1 stride 2; stride 2 along H only), odd image sizes whose lattices
# differ in length, no padding, and the stacked / diagonal / three-MMA forms of both math modes.
STRIDED_DW_CASES = {
    "sdw_3x3_s2_16x16x32": (4, 16, 16, 32, 32, 3, 3, 2, 2, 1, 1),
    "sdw_3x3_s2_15x17x32_oc64": (4, 15, 17, 32, 64, 3, 3, 2, 2, 1, 1),
    "sdw_3x3_s2x1_12x12x64_oc96": (3, 12, 12, 64, 96, 3, 3, 2, 1, 1, 1),
    "sdw_3x3_s1x2_12x12x64_oc96": (3, 12, 12, 64, 96, 3, 3, 1, 2, 1, 1),
    "sdw_4x4_s2_8x8x64_oc128": (4, 8, 8, 64, 128, 4, 4, 2, 2, 1, 1),
    "sdw_4x4_s2_32x32x32_oc64": (2, 32, 32, 32, 64, 4, 4, 2, 2, 1, 1),
    "sdw_1x1_s2_16x16x64_oc128": (4, 16, 16, 64, 128, 1, 1, 2, 2, 0, 0),
    "sdw_5x5_s2_20x20x32": (2, 20, 20, 32, 32, 5, 5, 2, 2, 2, 2),
    "sdw_3x3_s2_nopad_9x9x32": (2, 9, 9, 32, 32, 3, 3, 2, 2, 0, 0),
    "sdw_3x3_s2_14x14x256": (2, 14, 14, 256, 256, 3, 3, 2, 2, 1, 1),
}
CASES.update(STRIDED_DW_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(STRIDED_DW_CASES))
def test_strided_deltaW_on_the_halo_kernel(pkg, eng, oracle_mod, name, mode):
    import torch
    O, lib = oracle_mod, pkg.submodule("lib")
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    X, dY = gen((N, IH, IW, IC), "relu", rng), gen((N, OH, OW, OC), "n01", rng)
    dev = torch.device("cuda:0")
    lib.set_math_mode(mode)
    old = lib.set_option("DW_STRIDED", 2)     # also where the planner would leave few-pixel images to the split-K kernel
    try:
        tX, tdY = torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev)
        dW = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw).cpu().numpy()
        plan = lib.last_plan()
        lib.set_option("DW_STRIDED", 0)
        other = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw).cpu().numpy()
    finally:
        lib.set_option("DW_STRIDED", old)
        lib.set_math_mode("3xtf32")
    assert lib.device_status() == 0
    assert plan.startswith("dw_halo") and "strided" in plan, plan
    dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
    m = metrics(dW, dW64, SW)
    record(dict(case=name, mode=mode, tile="dw strided", dw=m))
    assert m["finite"] and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= TOL[mode]["comp"], (plan, m)
    # and against the split-K im2col kernel on the same tensors
    assert np.abs(dW - other).max() <= TOL[mode]["norm"] * np.abs(other).max(), plan


def test_strided_deltaW_plan_choice(pkg, eng):
    """Down-sampling layers at the benchmark's batch take the halo kernel; images of a few pixels stay on the split-K kernel in 3xTF32."""
    import torch
    lib = pkg.submodule("lib")
    dev = torch.device("cuda:0")
    lib.set_math_mode("3xtf32")
    for (N, IH, IC, OC, F, p), halo in (((512, 32, 64, 128, 3, 1), True), ((512, 16, 128, 256, 3, 1), True), ((512, 8, 256, 512, 3, 1), False),
                                        ((512, 32, 64, 128, 1, 0), True), ((256, 16, 128, 256, 4, 1), True)):
        OH = (IH + 2 * p - F) // 2 + 1
        X, dY = torch.zeros((N, IH, IH, IC), device=dev), torch.zeros((N, OH, OH, OC), device=dev)
        dW = eng.dconv3D_deltaW(X, dY, F, F, 2, 2, p, p)
        algo, plan = lib.last_algo(), lib.last_plan()
        assert (algo.startswith("dw_halo") and "strided" in plan) == halo, (IH, IC, OC, F, algo, plan)
        assert float(dW.abs().max()) == 0.0
    assert lib.device_status() == 0


# deltaW filter rows of more than three taps split over CTAs of three taps each (5x5: taps 0-2 and 3-4 with a spare
# accumulator; 7x7: three groups), in the stacked, three-MMA and plain forms, with and without padding, against the
# oracle and against whole-row CTAs; the fused bias gradient must come from one tap group only.
TAPGROUP_CASES = {
    "tg_5x5_16x16x64_oc128": (3, 16, 16, 64, 128, 5, 5, 1, 1, 2, 2),
    "tg_5x5_12x20x128": (2, 12, 20, 128, 128, 5, 5, 1, 1, 2, 2),
    "tg_5x5_nopad_14x14x32_oc64": (2, 14, 14, 32, 64, 5, 5, 1, 1, 0, 0),
    "tg_7x7_14x14x128_oc64": (2, 14, 14, 128, 64, 7, 7, 1, 1, 3, 3),
    "tg_3x5_10x12x64": (3, 10, 12, 64, 64, 3, 5, 1, 1, 1, 2),
}
CASES.update(TAPGROUP_CASES)


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(TAPGROUP_CASES))
def test_deltaW_with_tap_groups(pkg, eng, oracle_mod, name, mode):
    import torch
    O, lib = oracle_mod, pkg.submodule("lib")
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    X, dY = gen((N, IH, IW, IC), "relu", rng), gen((N, OH, OW, OC), "n01", rng)
    dev = torch.device("cuda:0")
    tX, tdY = torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev)
    lib.set_math_mode(mode)
    old = lib.set_option("DW_TAPGROUPS", 2)
    try:
        dW, dB = eng.dconv3D_deltaW_bias(tX, tdY, FH, FW, sh, sw, ph, pw)
        plan = lib.last_plan()
        dW, dB = dW.cpu().numpy(), dB.cpu().numpy()
        lib.set_option("DW_TAPGROUPS", 0)
        whole = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw).cpu().numpy()
        plan0 = lib.last_plan()
    finally:
        lib.set_option("DW_TAPGROUPS", old)
        lib.set_math_mode("3xtf32")
    assert lib.device_status() == 0
    assert "tap groups" in plan and "tap groups" not in plan0, (plan, plan0)
    dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
    m = metrics(dW, dW64, SW)
    record(dict(case=name, mode=mode, tile="dw tap groups", dw=m))
    assert m["finite"] and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= TOL[mode]["comp"], (plan, m)
    assert np.abs(dW - whole).max() <= TOL[mode]["norm"] * np.abs(whole).max(), (plan, plan0)
    ref_b = dY.astype(np.float64).sum(axis=(0, 1, 2))
    assert np.abs(dB - ref_b).max() <= 1e-5 * np.abs(dY).astype(np.float64).sum(axis=(0, 1, 2)).max(), plan
