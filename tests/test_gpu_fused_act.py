"""conv + bias + LeakyReLU in one kernel (alpha_conv3d_forward_leakyRelu) against the oracle's conv
followed by the reference's activation formula, on shapes that reach every forward kernel."""
import numpy as np
import pytest

from helpers import metrics

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng(pkg):
    return pkg.submodule("engine").Engine()


def leaky_relu_ref(x, k):
    """x * ((x > 0) + k * (x < 0)), Cuda_function/type4_leakyRelu2D.cuh:32."""
    return x * ((x > 0) + k * (x < 0))


# (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, kernel the forward is expected to take)
CASES = [
    (4, 32, 32, 16, 32, 3, 3, 1, 1, 1, 1, None),        # the reference's small test shape
    (8, 28, 28, 64, 64, 3, 3, 1, 1, 1, 1, "halo"),       # single-CTA halo kernel
    (8, 14, 14, 64, 128, 3, 3, 1, 1, 1, 1, "halo_pair"),  # CTA-pair kernel (128-channel block)
    (4, 16, 16, 32, 48, 3, 3, 2, 2, 1, 1, "igemm"),      # strided: im2col kernel
    (4, 16, 16, 4, 32, 3, 3, 1, 1, 1, 1, None),          # IC = 4: patch-matrix path
    (2, 9, 9, 6, 10, 3, 3, 1, 1, 1, 1, None),            # odd channels: padded / SIMT
    (3, 12, 12, 32, 32, 1, 1, 1, 1, 0, 0, None),         # 1x1
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("k", [0.0, 0.2])
def test_fused_leaky_relu(pkg, eng, oracle_mod, case, k):
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, want = case
    rng = np.random.default_rng(IH * 131 + IC)
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = (rng.standard_normal((OC, FH, FW, IC)) / np.sqrt(FH * FW * IC)).astype(np.float32)
    B = rng.standard_normal(OC).astype(np.float32)
    dev = torch.device("cuda:0")
    Y = eng.conv3D_leakyRelu(torch.from_numpy(X).to(dev), torch.from_numpy(W).to(dev), torch.from_numpy(B).to(dev),
                             k, sh, sw, ph, pw)
    assert lib.device_status() == 0
    if want:
        assert lib.last_algo().startswith(want), lib.last_algo()
    Y64, SY = oracle_mod.conv3D_f64(X, W, sh, sw, ph, pw, threads=8)
    pre = Y64 + B.astype(np.float64)
    ref = leaky_relu_ref(pre, k)
    m = metrics(Y.cpu().numpy(), ref, SY + np.abs(B).astype(np.float64))
    assert m["finite"] and m["norm"] <= 1e-4 and m["comp"] <= 1e-4, (lib.last_algo(), m)
    # same bits as the unfused pair of operators
    Y2 = eng.conv3D_biased(torch.from_numpy(X).to(dev), torch.from_numpy(W).to(dev), torch.from_numpy(B).to(dev),
                           sh, sw, ph, pw)
    Y2 = torch.where(Y2 > 0, Y2, Y2 * k)
    assert torch.equal(Y, Y2) or float((Y - Y2).abs().max()) == 0.0


def test_fused_relu_without_bias(pkg, eng):
    import torch
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(2)
    X = torch.randn((8, 14, 14, 64), device=dev, generator=gen)
    W = torch.randn((64, 3, 3, 64), device=dev, generator=gen) * 0.05
    Y = eng.conv3D_leakyRelu(X, W, None, 0.0, 1, 1, 1, 1)
    Y2 = eng.conv3D(X, W, 1, 1, 1, 1)
    assert float(Y.min()) >= 0.0
    assert torch.equal(Y, torch.where(Y2 > 0, Y2, Y2 * 0.0))
