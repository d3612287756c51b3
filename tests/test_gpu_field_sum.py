"""Bias gradient (Engine.field_sum of deltaY, nn/unit/simple/Conv3D.java:160) on the GPU against the
oracle's double-precision column sums, through the C ABI entry point alpha_conv_bias_grad."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng(pkg):
    return pkg.submodule("engine").Engine()


# fp32 accumulation in a tree of (rows / CTAs / 64 lanes) levels: far below this bound in practice
REL = 2e-6


@pytest.mark.parametrize("shape", [
    (1, 1, 1, 4),          # a single row
    (4, 32, 32, 32),       # the reference's own small test shape
    (3, 7, 5, 12),         # ragged rows, 3 float4 columns
    (2, 9, 9, 6),          # channels padded to 8 by the engine layer
    (5, 3, 3, 1028),       # more float4 columns than threads in a CTA
    (16, 28, 28, 96),      # row lanes do not divide the CTA (24 float4 columns)
    (256, 56, 56, 64),     # benchmark size: 205 MB
])
def test_field_sum_matches_oracle(pkg, eng, oracle_mod, shape):
    import torch
    lib = pkg.submodule("lib")
    gen = torch.Generator(device="cuda:0").manual_seed(sum(shape))
    dY = torch.randn(shape, device="cuda:0", generator=gen)
    got = eng.field_sum(dY, shape[-1]).cpu().numpy()
    assert lib.device_status() == 0 and got.shape == (shape[-1],)
    ref, mag = oracle_mod.field_sum_f64(dY.cpu().numpy(), shape[-1])
    assert np.all(np.abs(got - ref) <= REL * mag + 1e-30), float(np.max(np.abs(got - ref) / (mag + 1e-30)))
    if dY.numel() <= 1 << 20:
        # the reference's sequential float loop agrees to its own rounding error
        seq = oracle_mod.field_sum(dY.cpu().numpy(), shape[-1])
        assert np.all(np.abs(seq - ref) <= 1e-4 * mag + 1e-30)


@pytest.mark.parametrize("shape", [(4, 32, 32, 32), (3, 7, 5, 12), (16, 28, 28, 96), (64, 56, 56, 64), (5, 3, 3, 1028), (2, 2, 2, 8)])
def test_field_sum_against_the_reference_gpu_kernel(pkg, eng, oracle_mod, shape):
    """Pin against the reference itself: its Cuda_reduce.field_linear (Cuda_reduce/A.cu:117-131, what
    Engine.field_sum runs), rebuilt for sm_100 from its checkout, on the same device tensor.  Both results
    are fp32 sums in different orders: they agree within the rounding of such sums, and each agrees with
    the double-precision sum."""
    import torch
    from oracle import cu32_ref
    if not cu32_ref.reduce_available():
        pytest.skip("oracle/_ref/libcu32_Cuda_reduce.so not built (needs the reference checkout)")
    gen = torch.Generator(device="cuda:0").manual_seed(sum(shape) + 1)
    dY = torch.randn(shape, device="cuda:0", generator=gen)
    OC = shape[-1]
    ours = eng.field_sum(dY, OC).cpu().numpy()
    theirs = cu32_ref.field_linear(dY.view(-1, OC)).cpu().numpy()
    ref, mag = oracle_mod.field_sum_f64(dY.cpu().numpy(), OC)
    assert np.isfinite(theirs).all()
    assert np.all(np.abs(theirs - ref) <= 1e-5 * mag + 1e-30), float(np.max(np.abs(theirs - ref) / (mag + 1e-30)))
    assert np.all(np.abs(ours - theirs) <= 1e-5 * mag + 1e-30), float(np.max(np.abs(ours - theirs) / (mag + 1e-30)))
    assert np.all(np.abs(ours - ref) <= REL * mag + 1e-30)


def test_field_sum_positive_inputs_and_reproducibility(pkg, eng, oracle_mod):
    """All-positive input (a long sum without cancellation) and bit-identical repeats."""
    import torch
    gen = torch.Generator(device="cuda:0").manual_seed(3)
    dY = torch.rand((64, 56, 56, 64), device="cuda:0", generator=gen)
    a = eng.field_sum(dY, 64)
    b = eng.field_sum(dY, 64)
    assert torch.equal(a, b)
    ref, mag = oracle_mod.field_sum_f64(dY.cpu().numpy(), 64)
    assert np.all(np.abs(a.cpu().numpy() - ref) <= REL * mag)


def test_bias_grad_of_a_biased_layer(pkg, eng, oracle_mod):
    """The three gradients of Conv3D.__backward__ (deltaW, deltaB, deltaX) of one biased layer tie together:
    <Y(X, W, B), dY> = <X, deltaX> + <B, deltaB> = <W, deltaW> + <B, deltaB>."""
    import torch
    gen = torch.Generator(device="cuda:0").manual_seed(5)
    N, HW, IC, OC = 8, 14, 32, 64
    X = torch.randn((N, HW, HW, IC), device="cuda:0", generator=gen)
    W = torch.randn((OC, 3, 3, IC), device="cuda:0", generator=gen) * 0.1
    B = torch.randn((OC,), device="cuda:0", generator=gen)
    dY = torch.randn((N, HW, HW, OC), device="cuda:0", generator=gen)
    Y = eng.conv3D_biased(X, W, B, 1, 1, 1, 1)
    dX = eng.dconv3D_deltaX(dY, W, HW, HW, 1, 1, 1, 1)
    dW = eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1)
    dB = eng.field_sum(dY, OC)

    def dot(a, b):
        return float((a.double() * b.double()).sum())
    lhs = dot(Y, dY)
    scale = float(Y.double().norm() * dY.double().norm())
    assert abs(lhs - (dot(X, dX) + dot(B, dB))) <= 1e-5 * scale
    assert abs(lhs - (dot(W, dW) + dot(B, dB))) <= 1e-5 * scale


# (N, IH, IW, IC, OC, F, stride, pad): shapes of every form of the deltaW halo kernel, and some it does not take
FUSED_CASES = [
    (16, 28, 28, 128, 128, 3, 1, 1),    # three MMAs per step (3xTF32) / plain
    (8, 56, 56, 64, 64, 3, 1, 1),       # stacked planes (3xTF32) / diagonal half tiles (TF32)
    (8, 14, 14, 256, 256, 3, 1, 1),     # two output-channel tiles
    (4, 12, 12, 32, 96, 3, 1, 1),       # output channels do not fill the 128-channel tile
    (4, 9, 7, 32, 36, 5, 1, 2),         # ragged image, 5x5, OC = 36
    (16, 7, 7, 64, 72, 1, 1, 0),        # 1x1 (flat pixel view)
    (8, 16, 16, 32, 64, 3, 2, 1),       # stride 2: not fused, two passes
    (8, 32, 32, 4, 64, 7, 2, 3),        # IC = 4 stem: patch-matrix path, two passes
    (32, 2, 2, 64, 64, 3, 1, 1),        # tiny images: patch-matrix path
]


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("case", FUSED_CASES)
def test_bias_gradient_inside_the_deltaW_pass(pkg, eng, oracle_mod, case, mode):
    """alpha_conv3d_deltaW_bias: deltaW equals alpha_conv3d_deltaW's bit for bit (the bias columns are summed
    beside the MMAs, not in them), deltaB agrees with the double-precision column sums and with the
    stand-alone bias-gradient kernel to fp32 summation order, and repeats are bit-identical."""
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    N, IH, IW, IC, OC, F, s, p = case
    OH, OW = (IH + 2 * p - F) // s + 1, (IW + 2 * p - F) // s + 1
    gen = torch.Generator(device="cuda:0").manual_seed(sum(case))
    X = torch.randn((N, IH, IW, IC), device="cuda:0", generator=gen)
    dY = torch.randn((N, OH, OW, OC), device="cuda:0", generator=gen)
    try:
        dW_ref = eng.dconv3D_deltaW(X, dY, F, F, s, s, p, p)
        dB_ref = eng.field_sum(dY, OC)
        dW, dB = eng.dconv3D_deltaW_bias(X, dY, F, F, s, s, p, p)
        dW2, dB2 = eng.dconv3D_deltaW_bias(X, dY, F, F, s, s, p, p)
        assert lib.device_status() == 0
    finally:
        lib.set_math_mode("3xtf32")
    assert torch.equal(dW, dW_ref) and torch.equal(dW, dW2) and torch.equal(dB, dB2)
    ref, mag = oracle_mod.field_sum_f64(dY.cpu().numpy(), OC)
    got = dB.cpu().numpy()
    assert np.all(np.abs(got - ref) <= REL * mag + 1e-30), float(np.max(np.abs(got - ref) / (mag + 1e-30)))
    assert np.all(np.abs(got - dB_ref.cpu().numpy()) <= 2 * REL * mag + 1e-30)
