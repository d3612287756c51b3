"""CPU tests of the oracle: against the committed golden vectors (outputs of the reference's own
C++ loops), against the reference's loops themselves where they were built on this machine, and
against its own fp64 variant."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv_golden.npz")


@pytest.fixture(scope="module")
def golden():
    g = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in g.files})
    return g, names


def _case(g, name):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = (int(v) for v in g[name + "/shape"])
    return (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), g[name + "/X"], g[name + "/W"], g[name + "/dY"]


def test_golden_file_has_cases(golden):
    g, names = golden
    assert len(names) >= 7


def test_float_loops_match_reference_outputs_bit_for_bit(golden, oracle_mod):
    """The float-accumulator restatements reproduce the reference's compiled loops exactly."""
    O = oracle_mod
    g, names = golden
    for name in names:
        (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), X, W, dY = _case(g, name)
        assert np.array_equal(O.conv3D_naive_f32(X, W, sh, sw, ph, pw), g[name + "/ref_Y"]), name
        assert np.array_equal(O.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw), g[name + "/ref_dX"]), name
        assert np.array_equal(O.deconv3D_deltaW_img2col2(X, dY, FH, FW, sh, sw, ph, pw), g[name + "/ref_dW"]), name


def test_threads_do_not_change_results(golden, oracle_mod):
    O = oracle_mod
    g, names = golden
    for name in names[:3]:
        (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), X, W, dY = _case(g, name)
        assert np.array_equal(O.conv3D_naive(X, W, sh, sw, ph, pw, threads=1), O.conv3D_naive(X, W, sh, sw, ph, pw, threads=4))
        assert np.array_equal(O.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw, threads=1),
                              O.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw, threads=4))
        assert np.array_equal(O.deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw, threads=1),
                              O.deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw, threads=4))


def test_double_accumulator_loops(golden, oracle_mod):
    """The Java double-accumulator loops: stable against the stored values and within one fp32
    rounding of the fp64 result."""
    O = oracle_mod
    g, names = golden
    for name in names:
        (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), X, W, dY = _case(g, name)
        Y = O.conv3D_naive(X, W, sh, sw, ph, pw)
        dW = O.deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw)
        assert np.array_equal(Y, g[name + "/java_Y"]), name
        assert np.array_equal(dW, g[name + "/java_dW"]), name
        Y64, SY = O.conv3D_f64(X, W, sh, sw, ph, pw)
        dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw)
        # float products carry 2^-24 each; the double sum adds nothing visible; the final cast 2^-24
        assert (np.abs(Y - Y64) <= 1.3e-7 * SY + 1e-30).all(), name
        assert (np.abs(dW - dW64) <= 1.3e-7 * SW + 1e-30).all(), name


def test_deltaX_forms_agree(golden, oracle_mod):
    """img2col (gather) and crossAdd (scatter) forms of deltaX agree up to summation order."""
    O = oracle_mod
    g, names = golden
    for name in names:
        (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), X, W, dY = _case(g, name)
        a = O.deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)
        b = O.deconv3D_deltaX_crossAdd(dY, W, IH, IW, sh, sw, ph, pw)
        d64, S = O.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw)
        assert (np.abs(a - d64) <= 1e-5 * S + 1e-30).all(), name
        assert (np.abs(b - d64) <= 1e-5 * S + 1e-30).all(), name


def test_adjoint_identity(oracle_mod):
    """<conv(X, W), dY> = <X, deltaX(dY, W)> = <W, deltaW(X, dY)> in fp64: the three loops describe
    one bilinear form (a size-independent property of the path)."""
    O = oracle_mod
    rng = np.random.default_rng(5)
    for (sh, ph, F) in [(1, 1, 3), (2, 1, 3), (2, 1, 4), (1, 0, 1)]:
        X = rng.standard_normal((2, 9, 8, 4)).astype(np.float32)
        W = rng.standard_normal((8, F, F, 4)).astype(np.float32)
        OH, OW = O.out_hw(9, 8, F, F, sh, sh, ph, ph)
        dY = rng.standard_normal((2, OH, OW, 8)).astype(np.float32)
        Y, _ = O.conv3D_f64(X, W, sh, sh, ph, ph)
        dX, _ = O.deconv3D_deltaX_f64(dY, W, 9, 8, sh, sh, ph, ph)
        dW, _ = O.deconv3D_deltaW_f64(X, dY, F, F, sh, sh, ph, ph)
        a, b, c = (Y * dY).sum(), (dX * X).sum(), (dW * W).sum()
        assert abs(a - b) <= 1e-9 * abs(a) + 1e-9 and abs(a - c) <= 1e-9 * abs(a) + 1e-9


def test_same_percent_relative(oracle_mod):
    O = oracle_mod
    a = np.array([1.0, 2.0, 0.0, np.nan, 1.0], np.float32)
    b = np.array([1.0, 2.00001, 0.0, np.nan, 1.1], np.float32)
    assert abs(O.samePercentRelative(a, b, 1e-4) - 0.8) < 1e-6


def test_reference_loops_when_built(golden, oracle_mod):
    """Where the reference's loops were compiled on this machine, the golden file is reproducible."""
    O = oracle_mod
    if O.ref_lib() is None:
        pytest.skip("oracle/_ref was not built here (no reference checkout)")
    g, names = golden
    for name in names:
        (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw), X, W, dY = _case(g, name)
        assert np.array_equal(O.ref_CONV_3D_NAIVE(X, W, sh, sw, ph, pw), g[name + "/ref_Y"])
        assert np.array_equal(O.ref_deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw), g[name + "/ref_dX"])
        assert np.array_equal(O.ref_deconv3D_deltaW_img2col2(X, dY, FH, FW, sh, sw, ph, pw), g[name + "/ref_dW"])


def test_field_sum_follows_the_reference_loop(oracle_mod):
    """field_sum restates Matrix.field_linear (alpha = 1, beta = 0): V[j] = sum over rows, in float,
    row after row."""
    rng = np.random.default_rng(9)
    A = rng.standard_normal((37, 12)).astype(np.float32)
    want = np.zeros(12, np.float32)
    for j in range(12):
        v = np.float32(0)
        for i in range(37):
            v = np.float32(v + A[i, j])
        want[j] = v
    got = oracle_mod.field_sum(A, 12)
    assert np.array_equal(got, want)
    d, mag = oracle_mod.field_sum_f64(A, 12)
    assert np.all(np.abs(d - want) <= 1e-5 * mag)


def test_matmul_oracle_against_the_reference_loops(oracle_mod):
    """The float loops of the three matrix products reproduce the stored outputs of the reference's own
    multiply / multiplyT1 / multiplyT2 (tests/golden/matmul_golden.npz) bit for bit, and sit within fp32
    rounding of the double-precision product."""
    import os
    O = oracle_mod
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "matmul_golden.npz"))
    keys = sorted({k.rsplit("/", 1)[0] for k in g.files})
    assert len(keys) == 12
    for key in keys:
        variant = key.split("/")[1]
        A, B, ref = g[key + "/A"], g[key + "/B"], g[key + "/ref_C"]
        got = O.matmul(A, B, variant)
        assert np.array_equal(got, ref), key
        c64, S = O.matmul_f64(A, B, variant)
        assert (np.abs(got - c64) <= 1e-5 * S + 1e-30).all(), key
        if O.ref_lib() is not None:
            assert np.array_equal(O.ref_matmul(A, B, variant), ref), key


def _golden(name):
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


def test_batched_matmul_oracle_against_the_reference_loops(oracle_mod):
    """The float loops of the three batched products, on the engine's padded memory layout, reproduce the stored
    outputs of the reference's own bmm / bmmT1 / bmmT2 (tests/golden/bmm_golden.npz) bit for bit."""
    O = oracle_mod
    g = _golden("bmm_golden.npz")
    keys = sorted({k.rsplit("/", 1)[0] for k in g.files})
    assert len(keys) == 9
    for key in keys:
        variant = key.split("/")[1]
        A, B, ref, rows = g[key + "/A"], g[key + "/B"], g[key + "/ref_C"], int(g[key + "/rows"])
        got = O.batch_matmul(A, B, variant, rows=rows)
        assert np.array_equal(got, ref), key
        c64, S = O.batch_matmul(A, B, variant, rows=rows, f64=True)
        assert (np.abs(got - c64) <= 1e-5 * S + 1e-30).all(), key
        if O.ref_lib() is not None:
            assert np.array_equal(O.ref_batch_matmul(A, B, variant, rows=rows), ref), key


def test_pooling_oracle_against_the_reference_loops(oracle_mod):
    """Forward max / average (padding ignored) and their gradients reproduce the stored outputs of the reference's own
    CPU loops (tests/golden/pool_golden.npz) bit for bit on inputs with ties; the variants those loops do not have are
    tied to them by identities: the index points at an element equal to the maximum, the indexed gradient hands
    every output gradient to exactly one input element, the plain average equals the padded-count one where no
    window leaves the image."""
    O = oracle_mod
    g = _golden("pool_golden.npz")
    names = sorted({k.split("/")[0] for k in g.files})
    assert len(names) == 6
    for name in names:
        N, IH, IW, IC, FH, FW, sh, sw, ph, pw = (int(v) for v in g[name + "/shape"])
        X, dY = g[name + "/X"], g[name + "/dY"]
        win = (FH, FW, sh, sw, ph, pw)
        Y = O.pool2D(X, *win, op="max")
        assert np.array_equal(Y, g[name + "/ref_max"]), name
        assert np.array_equal(O.pool2D(X, *win, op="avg_ignore_padding"), g[name + "/ref_avg_ip"]), name
        assert np.array_equal(O.upool2D(dY, IH, IW, *win, op="max", Y=Y, X=X), g[name + "/ref_d_max"]), name
        assert np.array_equal(O.upool2D(dY, IH, IW, *win, op="avg_ignore_padding"), g[name + "/ref_d_avg_ip"]), name
        Yi, Index = O.pool2D(X, *win, op="max_indexed")
        assert np.array_equal(Yi, Y) and np.array_equal(X.reshape(-1)[Index], Y), name
        dXi = O.upool2D(dY, IH, IW, *win, op="max_indexed", Index=Index)
        assert abs(float(dXi.astype(np.float64).sum()) - float(dY.astype(np.float64).sum())) <= 1e-4 * np.abs(dY).sum()
        assert np.count_nonzero(dXi) <= dY.size
        if ph == 0 and pw == 0:
            assert np.array_equal(O.pool2D(X, *win, op="avg"), O.pool2D(X, *win, op="avg_ignore_padding")), name
            a, b = O.upool2D(dY, IH, IW, *win, op="avg"), O.upool2D(dY, IH, IW, *win, op="avg_ignore_padding")
            assert np.abs(a - b).max() <= 1e-6 * np.abs(b).max(), name
        if O.ref_lib() is not None:
            assert np.array_equal(O.ref_pool2D(X, *win, op="max"), g[name + "/ref_max"]), name
            assert np.array_equal(O.ref_upool2D(dY, IH, IW, *win, op="avg"), g[name + "/ref_d_avg_ip"]), name
