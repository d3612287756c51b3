"""GPU parity on the layer shapes of the benchmark configurations that are not bench lines:
the ResNet-18-shaped conv stack (config 3), the DCGAN-style transposed-conv stack (config 4) and
the large-shape stress convolutions (config 5).  Batches are cut down so that the CPU oracle
finishes in seconds; the full-size cases are tied down by size-independent identities."""
import zlib

import numpy as np
import pytest

from helpers import TOL, gen, metrics, out_hw, record

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng(pkg):
    import torch
    torch.cuda.set_device(0)
    return pkg.submodule("engine").Engine()


def _check_layer(pkg, eng, O, tag, N, IH, IC, OC, F, s, p, dists=("relu", "n01", "n01"), ops=("fwd", "dx", "dw")):
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    OH, OW = out_hw(IH, IH, F, F, s, s, p, p)
    rng = np.random.default_rng(zlib.crc32(tag.encode()))
    X = gen((N, IH, IH, IC), dists[0], rng)
    W = (gen((OC, F, F, IC), dists[1], rng) * np.float32(np.sqrt(2.0 / (F * F * IC)))).astype(np.float32)
    dY = gen((N, OH, OW, OC), dists[2], rng)
    dev = torch.device("cuda:0")
    tX, tW, tdY = (torch.from_numpy(a).to(dev) for a in (X, W, dY))
    out = {}
    if "fwd" in ops:
        Y = eng.conv3D(tX, tW, s, s, p, p).cpu().numpy()
        out["fwd"] = (lib.last_algo(), metrics(Y, *O.conv3D_f64(X, W, s, s, p, p, threads=8)))
    if "dx" in ops:
        dX = eng.dconv3D_deltaX(tdY, tW, IH, IH, s, s, p, p).cpu().numpy()
        out["dx"] = (lib.last_algo(), metrics(dX, *O.deconv3D_deltaX_f64(dY, W, IH, IH, s, s, p, p, threads=8)))
    if "dw" in ops:
        dW = eng.dconv3D_deltaW(tX, tdY, F, F, s, s, p, p).cpu().numpy()
        out["dw"] = (lib.last_algo(), metrics(dW, *O.deconv3D_deltaW_f64(X, dY, F, F, s, s, p, p, threads=8)))
    assert lib.device_status() == 0
    record(dict(case=tag, mode="3xtf32", **{k: dict(algo=v[0], **v[1]) for k, v in out.items()}))
    for op, (algo, m) in out.items():
        assert m["finite"] and m["norm"] <= TOL["3xtf32"]["norm"] and m["comp"] <= TOL["3xtf32"]["comp"], (tag, op, algo, m)
    return out


def test_resnet18_conv_stack(pkg, eng, oracle_mod):
    """All 20 convolutions of the CIFAR ResNet-18 (stem 7x7 s2 on 4 padded channels, 3x3 s1/s2,
    1x1 s2 shortcuts), batch 8: forward, deltaX and deltaW of every layer."""
    synth = pkg.submodule("synth")
    seen = set()
    assert len(synth.RESNET18_CONVS) == 20
    for i, (IH, IC, OC, F, s, p) in enumerate(list(synth.RESNET18_CONVS) + synth.SHORTCUT_1X1_CONVS):
        if (IH, IC, OC, F, s, p) in seen:
            continue
        seen.add((IH, IC, OC, F, s, p))
        _check_layer(pkg, eng, oracle_mod, "resnet18_%d" % i, 8, IH, IC, OC, F, s, p)


def test_dcgan_deconv_stack(pkg, eng, oracle_mod):
    """The generator's transposed convolutions (4x4, stride 2, pad 1): Deconv3D forward is
    dconv3D_deltaX with W[IC_in, 4, 4, OC_out]; as conv shapes OC = C_in, IC = C_out, image = output."""
    import torch
    synth = pkg.submodule("synth")
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    for (hin, cin, cout) in synth.DCGAN_DECONVS:
        rng = np.random.default_rng(hin * 1000 + cin)
        N, hout = 4, 2 * hin
        Z = gen((N, hin, hin, cin), "n01", rng)
        W = (rng.standard_normal((cin, 4, 4, cout)) * 0.02).astype(np.float32)
        out = eng.dconv3D(torch.from_numpy(Z).to(dev), torch.from_numpy(W).to(dev), 2, 2, 1, 1).cpu().numpy()
        assert out.shape == (N, hout, hout, cout)
        ref, S = O.deconv3D_deltaX_f64(Z, W, hout, hout, 2, 2, 1, 1, threads=8)
        m = metrics(out, ref, S)
        record(dict(case="dcgan_%d_%d_%d" % (hin, cin, cout), mode="3xtf32", algo=lib.last_algo(), dx=m))
        assert lib.device_status() == 0
        assert m["finite"] and m["norm"] <= 1e-4 and m["comp"] <= 1e-5, (hin, cin, cout, lib.last_algo(), m)
        # and the two backward passes of the same layer
        _check_layer(pkg, eng, O, "dcgan_bwd_%d" % hin, 4, hout, cout, cin, 4, 2, 1, dists=("n01", "n01", "n01"), ops=("fwd", "dw"))


@pytest.mark.parametrize("case", [
    ("stress_3x3_s1", 2, 112, 64, 64, 3, 1, 1),
    ("stress_5x5_s1", 1, 112, 64, 128, 5, 1, 2),
    ("stress_3x3_s2", 2, 112, 128, 64, 3, 2, 1),
    ("stress_1x1_1024", 4, 14, 1024, 1024, 1, 1, 0),
])
def test_large_shape_layers_reduced_batch(pkg, eng, oracle_mod, case):
    tag, N, IH, IC, OC, F, s, p = case
    _check_layer(pkg, eng, oracle_mod, tag, N, IH, IC, OC, F, s, p, dists=("u11", "u11", "u11"))


def test_large_tensor_beyond_4gib_offsets(pkg, eng):
    """X[128,112,112,256]: 1.6 GB per tensor, byte offsets beyond 2^32.  Too large for the oracle;
    the three kernels are checked against each other through the adjoint identity, and the last
    image against the first (same input, so the same output, at offsets 127/128 of the tensor)."""
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    N, HW, IC, OC = 128, 112, 256, 64
    X = torch.empty((N, HW, HW, IC), device=dev).uniform_(-1, 1, generator=g)
    X[N - 1] = X[0]
    W = torch.empty((OC, 3, 3, IC), device=dev).uniform_(-1, 1, generator=g) * 0.02
    Y = eng.conv3D(X, W, 1, 1, 1, 1)
    assert lib.device_status() == 0
    assert torch.equal(Y[N - 1], Y[0])
    dY = torch.empty_like(Y).uniform_(-1, 1, generator=g)
    dX = eng.dconv3D_deltaX(dY, W, HW, HW, 1, 1, 1, 1)
    dW = eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1)
    assert lib.device_status() == 0

    def dot(a, b):
        acc = 0.0
        for i in range(0, a.shape[0], 16):
            acc += float((a[i:i + 16].double() * b[i:i + 16].double()).sum())
        return acc
    a, b, c = dot(Y, dY), dot(X, dX), dot(W, dW)
    # <Y,dY> and <X,dX>: element errors of relative size 1e-4 of the rms, signs independent
    tol_b = 1e-4 * float(Y.double().norm() * dY.double().norm()) / (Y.numel() ** 0.5)
    # <W,dW>: each dW element sums K = N*OH*OW products in fp32; its error is bounded by
    # 1e-6 * sum|x||dy| (a tenth of the componentwise bar), again with independent signs
    S_dw = N * HW * HW * 0.25
    tol_c = 1e-6 * S_dw * float(W.double().norm())
    assert abs(a - b) <= tol_b and abs(a - c) <= tol_c, (a, b, c, tol_b, tol_c)


@pytest.mark.parametrize("shape", [(8, 14, 128, 128), (4, 7, 512, 256)])
def test_positive_inputs_long_reduction(pkg, eng, oracle_mod, shape):
    """All-positive inputs (the reference's own test data, uniform [0,1)) with long reductions.
    Tensor-core accumulation truncates, so a sum of K positive products carries a bias of about
    (K / 8) * 2^-25 relative per MMA that adds into the main sum (one per step in the wide form, three
    otherwise): 2e-5 to 6e-5 at K = 4608.  The stated bar (max relative error 1e-4) must hold."""
    import torch
    N, H, IC, OC = shape
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    rng = np.random.default_rng(17)
    X = gen((N, H, H, IC), "u01", rng); W = gen((OC, 3, 3, IC), "u01", rng); dY = gen((N, H, H, OC), "u01", rng)
    dev = torch.device("cuda:0")
    tX, tW, tdY = (torch.from_numpy(a).to(dev) for a in (X, W, dY))
    O = oracle_mod
    res = {}
    res["fwd"] = metrics(eng.conv3D(tX, tW, 1, 1, 1, 1).cpu().numpy(), *O.conv3D_f64(X, W, 1, 1, 1, 1, threads=8))
    res["dx"] = metrics(eng.dconv3D_deltaX(tdY, tW, H, H, 1, 1, 1, 1).cpu().numpy(), *O.deconv3D_deltaX_f64(dY, W, H, H, 1, 1, 1, 1, threads=8))
    res["dw"] = metrics(eng.dconv3D_deltaW(tX, tdY, 3, 3, 1, 1, 1, 1).cpu().numpy(), *O.deconv3D_deltaW_f64(X, dY, 3, 3, 1, 1, 1, 1, threads=8))
    record(dict(case="positive_%dx%d_ic%d_oc%d" % (H, H, IC, OC), mode="3xtf32", **res))
    assert lib.device_status() == 0
    for op, m in res.items():
        assert m["finite"] and m["norm"] <= 1e-4 and m["comp"] <= 1e-4, (op, m)


@pytest.mark.parametrize("case", [
    ("stress_3x3_s2_full", 128, 112, 128, 64, 3, 2, 1),       # strided forward, phase deltaX, strided halo-tile deltaW
    ("dcgan_8x8_to_16x16_full", 1024, 16, 128, 256, 4, 2, 1),  # generator layer: deltaX through the dense product + col2im
    ("dcgan_16x16_to_32x32_full", 1024, 32, 64, 128, 4, 2, 1),
    ("resnet_1x1_s2_full", 512, 32, 64, 128, 1, 2, 0),
])
def test_strided_layers_full_size_adjoint_identity(pkg, eng, case):
    """The strided layers of the large-shape and generator configurations at their full batch, where the oracle is
    too slow: forward, deltaX and deltaW run on three different kernel families (im2col, phases or dense product +
    col2im, halo tiles over the stride lattice) and are tied together by
    <conv(X,W), dY> = <X, deltaX(dY,W)> = <W, deltaW(X,dY)>; deltaW also against the split-K kernel."""
    import torch
    tag, N, IH, IC, OC, F, s, p = case
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(zlib.crc32(tag.encode()))
    OH, _ = out_hw(IH, IH, F, F, s, s, p, p)
    X = torch.empty((N, IH, IH, IC), device=dev).uniform_(-1, 1, generator=g)
    W = torch.empty((OC, F, F, IC), device=dev).uniform_(-1, 1, generator=g) * 0.05
    dY = torch.empty((N, OH, OH, OC), device=dev).uniform_(-1, 1, generator=g)
    Y = eng.conv3D(X, W, s, s, p, p)
    dX = eng.dconv3D_deltaX(dY, W, IH, IH, s, s, p, p)
    dx_algo = lib.last_algo()
    dW = eng.dconv3D_deltaW(X, dY, F, F, s, s, p, p)
    dw_plan = lib.last_plan()
    old = lib.set_option("DW_STRIDED", 0)
    try:
        dW_split = eng.dconv3D_deltaW(X, dY, F, F, s, s, p, p)
    finally:
        lib.set_option("DW_STRIDED", old)
    assert lib.device_status() == 0
    assert "strided" in dw_plan, dw_plan
    if tag.startswith("dcgan_8x8"):
        assert dx_algo == "dx_col2im", dx_algo

    def dot(a, b):
        acc = 0.0
        for i in range(0, a.shape[0], 16):
            acc += float((a[i:i + 16].double() * b[i:i + 16].double()).sum())
        return acc
    a, b, c = dot(Y, dY), dot(X, dX), dot(W, dW)
    tol_b = 1e-4 * float(Y.double().norm() * dY.double().norm()) / (Y.numel() ** 0.5)
    tol_c = 1e-6 * (N * OH * OH * 0.25) * float(W.double().norm())
    assert abs(a - b) <= tol_b and abs(a - c) <= tol_c, (a, b, c, tol_b, tol_c)
    assert float((dW - dW_split).abs().max()) <= 1e-4 * float(dW_split.abs().max())
