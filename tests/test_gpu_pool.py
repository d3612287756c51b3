"""GPU parity of the 2D pooling operators (Engine.pool2D_max / pool2D_avg and their gradients; the reference's
Cuda_pool2D / Cuda_upool2D natives) against the oracle - which equals the reference's own CPU loops bit for bit
(tests/test_oracle.py) - and, where they were built, the reference's kernels rebuilt for sm_100.
max / max_indexed and their gradients are compared bit for bit (selection and ordered sums of the same numbers),
the averages to 1e-6 relative (one division, placed as in the reference's kernels)."""
import zlib

import numpy as np
import pytest

from helpers import gen

pytestmark = pytest.mark.gpu

# (N, IH, IW, IC, FH, FW, sh, sw, ph, pw)
CASES = {
    "resnet_stem_3x3_s2": (4, 56, 56, 64, 3, 3, 2, 2, 1, 1),      # ImageNet ResNet: max pool after the stem
    "2x2_s2": (4, 32, 32, 64, 2, 2, 2, 2, 0, 0),                  # window == stride (the reference's tiled gradient)
    "2x2_s2_odd_image": (4, 7, 9, 32, 2, 2, 2, 2, 0, 0),          # last row / column not covered by any window
    "ref_test_3x3_s1x2_p1": (8, 31, 31, 12, 3, 3, 1, 2, 1, 1),    # Cuda_pool2D.java:94-95
    "ref_test_4x4_s2_p1": (8, 62, 62, 16, 4, 4, 2, 2, 1, 1),      # Cuda_pool2D.java:97-98
    "overlap_3x3_s1": (4, 10, 12, 8, 3, 3, 1, 1, 1, 1),
    "global_avg_7x7": (4, 7, 7, 512, 7, 7, 1, 1, 0, 0),           # the head of a ResNet
    "ic_not_multiple_of_4": (2, 9, 9, 6, 3, 3, 2, 2, 1, 1),       # the engine pads the channels to 8
    "rect_5x2": (4, 16, 10, 4, 5, 2, 3, 1, 2, 1),
}
OPS = ("max", "max_indexed", "avg", "avg_ignore_padding")


@pytest.fixture(scope="module")
def eng(pkg):
    import torch
    torch.cuda.set_device(0)
    return pkg.submodule("engine").Engine()


def _inputs(name, ties):
    N, IH, IW, IC, FH, FW, sh, sw, ph, pw = CASES[name]
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    X = gen((N, IH, IW, IC), "n01", rng)
    if ties:
        X = (np.round(X * 2) / 2).astype(np.float32)      # many equal values inside every window
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    dY = gen((N, OH, OW, IC), "n01", rng)
    return X, dY


@pytest.mark.parametrize("ties", [False, True])
@pytest.mark.parametrize("name", list(CASES))
def test_forward_and_gradients_against_the_oracle(pkg, eng, oracle_mod, name, ties):
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    N, IH, IW, IC, FH, FW, sh, sw, ph, pw = CASES[name]
    X, dY = _inputs(name, ties)
    dev = torch.device("cuda:0")
    tX, tdY = torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev)
    win = (FH, FW, sh, sw, ph, pw)
    # forward
    Y = eng.pool2D_max(tX, *win)
    Yi, Index = eng.pool2D_max(tX, *win, indexed=True)
    Ya = eng.pool2D_avg(tX, *win)
    Yp = eng.pool2D_avg(tX, *win, ignore_padding=True)
    oY = O.pool2D(X, *win, op="max")
    np.testing.assert_array_equal(Y.cpu().numpy(), oY)
    np.testing.assert_array_equal(Yi.cpu().numpy(), oY)
    ic4 = Index.shape[3]
    Xp = np.zeros(X.shape[:3] + (ic4,), np.float32)
    Xp[..., :IC] = X
    _, oIdx = O.pool2D(Xp, *win, op="max_indexed")              # the index counts in the padded tensor
    np.testing.assert_array_equal(Index.cpu().numpy(), oIdx)
    np.testing.assert_array_equal(Xp.reshape(-1)[Index.cpu().numpy()[..., :IC]], oY)
    for got, op in ((Ya, "avg"), (Yp, "avg_ignore_padding")):
        want = O.pool2D(X, *win, op=op)
        assert np.abs(got.cpu().numpy() - want).max() <= 1e-6 * np.abs(want).max(), op
    # gradients
    dXm = eng.upool2D_max(tdY, Y, tX, *win)
    np.testing.assert_array_equal(dXm.cpu().numpy(), O.upool2D(dY, IH, IW, *win, op="max", Y=oY, X=X))
    dXi = eng.upool2D_max_indexed(tdY, Index, IH, IW, *win)
    dYp = np.zeros(dY.shape[:3] + (ic4,), np.float32)
    dYp[..., :IC] = dY
    np.testing.assert_array_equal(dXi.cpu().numpy(), O.upool2D(dYp, IH, IW, *win, op="max_indexed", Index=oIdx)[..., :IC])
    # every output element hands its gradient to exactly one input element
    assert abs(float(dXi.double().sum()) - float(dY.astype(np.float64).sum())) <= 1e-3 * (1 + np.abs(dY).sum() * 1e-4)
    for ip, op in ((False, "avg"), (True, "avg_ignore_padding")):
        got = eng.upool2D_avg(tdY, IH, IW, *win, ignore_padding=ip).cpu().numpy()
        want = O.upool2D(dY, IH, IW, *win, op=op)
        assert np.abs(got - want).max() <= 1e-6 * max(np.abs(want).max(), 1e-30), op
    assert lib.last_algo() == "pool_bwd"


def test_golden_vectors_of_the_reference_loops(pkg, eng):
    """The committed outputs of the reference's own CPU loops (tests/golden/pool_golden.npz)."""
    import os
    import torch
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pool_golden.npz"))
    dev = torch.device("cuda:0")
    for name in sorted({k.split("/")[0] for k in g.files}):
        N, IH, IW, IC, FH, FW, sh, sw, ph, pw = (int(v) for v in g[name + "/shape"])
        win = (FH, FW, sh, sw, ph, pw)
        tX, tdY = torch.from_numpy(g[name + "/X"]).to(dev), torch.from_numpy(g[name + "/dY"]).to(dev)
        Y = eng.pool2D_max(tX, *win)
        np.testing.assert_array_equal(Y.cpu().numpy(), g[name + "/ref_max"])
        np.testing.assert_array_equal(eng.upool2D_max(tdY, Y, tX, *win).cpu().numpy(), g[name + "/ref_d_max"])
        for got, key in ((eng.pool2D_avg(tX, *win, ignore_padding=True), "/ref_avg_ip"),
                         (eng.upool2D_avg(tdY, IH, IW, *win, ignore_padding=True), "/ref_d_avg_ip")):
            want = g[name + key]
            assert np.abs(got.cpu().numpy() - want).max() <= 1e-6 * np.abs(want).max(), (name, key)


def test_engine_base_methods_in_the_java_argument_order(pkg, eng, oracle_mod):
    """CudaFloat32EngineBase.pool2D_* / upool2D_* with the reference's argument order (CudaFloat32EngineBase.java:2012-2215)."""
    import torch
    O = oracle_mod
    base = eng.base
    dev = torch.device("cuda:0")
    N, IH, IW, IC, FH, FW, sh, sw, ph, pw = CASES["overlap_3x3_s1"]
    X, dY = _inputs("overlap_3x3_s1", ties=True)
    OH, OW = dY.shape[1:3]
    win = (FH, FW, sh, sw, ph, pw)
    tX, tdY = torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev)
    Y = torch.empty((N, OH, OW, IC), device=dev)
    Index = torch.empty((N, OH, OW, IC), device=dev, dtype=torch.int32)
    dX = torch.empty_like(tX)
    dims = (FH, FW, N, IC, sh, sw, ph, pw)
    base.pool2D_max(Y, OH, OW, tX, IH, IW, *dims)
    oY = O.pool2D(X, *win, op="max")
    np.testing.assert_array_equal(Y.cpu().numpy(), oY)
    base.pool2D_max_indexed(Y, Index, OH, OW, tX, IH, IW, *dims)
    np.testing.assert_array_equal(Index.cpu().numpy(), O.pool2D(X, *win, op="max_indexed")[1])
    base.upool2D_max(dX, tX, IH, IW, tdY, Y, OH, OW, *dims)
    np.testing.assert_array_equal(dX.cpu().numpy(), O.upool2D(dY, IH, IW, *win, op="max", Y=oY, X=X))
    base.upool2D_max_Indexed(dX, IH, IW, tdY, Index, OH, OW, *dims)
    np.testing.assert_array_equal(dX.cpu().numpy(), O.upool2D(dY, IH, IW, *win, op="max_indexed", Index=Index.cpu().numpy()))
    for fwd, bwd, op in ((base.pool2D_avg, base.upool2D_avg, "avg"),
                         (base.pool2D_avg_ignore_padding, base.upool2D_avg_ignore_padding, "avg_ignore_padding")):
        fwd(Y, OH, OW, tX, IH, IW, *dims)
        want = O.pool2D(X, *win, op=op)
        assert np.abs(Y.cpu().numpy() - want).max() <= 1e-6 * np.abs(want).max(), op
        bwd(dX, IH, IW, tdY, OH, OW, *dims)
        want = O.upool2D(dY, IH, IW, *win, op=op)
        assert np.abs(dX.cpu().numpy() - want).max() <= 1e-6 * np.abs(want).max(), op


def test_adjoint_identity_of_the_average(pkg, eng):
    """<pool_avg(X), dY> == <X, upool_avg(dY)> at a size the oracle would not finish (a property of the pair)."""
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    X = torch.randn((64, 112, 112, 64), device=dev, generator=g)
    win = (3, 3, 2, 2, 1, 1)
    for ip in (False, True):
        Y = eng.pool2D_avg(X, *win, ignore_padding=ip)
        dY = torch.randn(Y.shape, device=dev, generator=g)
        dX = eng.upool2D_avg(dY, 112, 112, *win, ignore_padding=ip)
        a, b = float((Y.double() * dY.double()).sum()), float((X.double() * dX.double()).sum())
        assert abs(a - b) <= 1e-5 * (abs(a) + abs(b) + 1), (ip, a, b)


def test_natives_against_the_rebuilt_reference(pkg, oracle_mod):
    """Both implementations of the ten natives under one harness (the engine's call shapes: channels and batch padded to 4,
    the tiled average gradient when the window equals the stride), on identical device tensors."""
    import torch
    from oracle import cu32_ref
    from test_gpu_jni import FakeEnv
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    env = FakeEnv([])
    ours = cu32_ref.Cu32Pool(libs=(L.load(), L.load()), env=env)
    theirs = cu32_ref.Cu32Pool() if cu32_ref.pool_available() else None
    O = oracle_mod
    for name in ("resnet_stem_3x3_s2", "2x2_s2", "2x2_s2_odd_image", "ref_test_3x3_s1x2_p1", "ref_test_4x4_s2_p1", "overlap_3x3_s1", "rect_5x2"):
        N, IH, IW, IC, FH, FW, sh, sw, ph, pw = CASES[name]
        assert IC % 4 == 0 and (N * IH * IW) % 4 == 0
        X, dY = _inputs(name, ties=True)
        tX, tdY = torch.from_numpy(X).to(dev), torch.from_numpy(dY).to(dev)
        win = (FH, FW, sh, sw, ph, pw)
        res = {}
        for who, impl in (("ours", ours), ("theirs", theirs)):
            if impl is None:
                continue
            r = {}
            r["max"] = impl.pool2D(tX, *win, op="max")
            r["max_i"], r["index"] = impl.pool2D(tX, *win, op="max_indexed")
            r["avg"] = impl.pool2D(tX, *win, op="avg")
            r["avg_ip"] = impl.pool2D(tX, *win, op="avg_ignore_padding")
            r["d_max"] = impl.upool2D(tdY, IH, IW, *win, op="max", Y=r["max"], X=tX)
            r["d_max_i"] = impl.upool2D(tdY, IH, IW, *win, op="max_indexed", Index=r["index"])
            r["d_avg"] = impl.upool2D(tdY, IH, IW, *win, op="avg")
            r["d_avg_ip"] = impl.upool2D(tdY, IH, IW, *win, op="avg_ignore_padding")
            res[who] = {k: v.cpu().numpy() for k, v in r.items()}
        assert env.thrown is None, env.thrown
        mine = res["ours"]
        np.testing.assert_array_equal(mine["max"], O.pool2D(X, *win, op="max"))
        if "theirs" in res:
            ref = res["theirs"]
            for k in ("max", "max_i", "index", "d_max"):
                np.testing.assert_array_equal(mine[k], ref[k], err_msg="%s %s" % (name, k))
            # The reference's indexed gradient is wrong in the corner its remainder kernels take (channels beyond the
            # last multiple of 8 x positions beyond the last multiple of 8: upool2D.cuh:152-171 -> the 1 x 1 kernel;
            # 8 x 31 x 31 x 12: a dozen elements of the last row of the last image), where its own CPU loop, its
            # non-indexed kernel and the oracle agree with this library.  Everywhere else the two must be equal.
            np.testing.assert_array_equal(mine["d_max_i"], O.upool2D(dY, IH, IW, *win, op="max_indexed", Index=mine["index"]))
            bad = np.argwhere(mine["d_max_i"] != ref["d_max_i"])
            assert len(bad) <= 16 and all(b[0] == N - 1 and b[1] == IH - 1 and b[3] >= IC - IC % 8 for b in bad), (name, bad[:8])
            for k in ("avg", "avg_ip", "d_avg", "d_avg_ip"):
                assert np.isfinite(ref[k]).all(), (name, k)
                assert np.abs(mine[k] - ref[k]).max() <= 1e-6 * max(np.abs(ref[k]).max(), 1e-30), (name, k)
    want = {"pool2D_1max", "pool2D_1max_1indexed", "pool2D_1avg", "pool2D_1avg_1ignore_1padding", "upool2D_1max",
            "upool2D_1max_1Indexed", "upool2D_1avg", "upool2D_1avg_1tiled", "upool2D_1avg_1ignore_1padding",
            "upool2D_1avg_1ignore_1padding_1tiled"}
    assert want <= set(ours.called), want - set(ours.called)


def test_argument_errors(pkg):
    import ctypes as C
    import torch
    L = pkg.submodule("lib")
    lib = L.load()
    t = torch.zeros(4096, device="cuda:0")
    p = C.c_void_p(t.data_ptr())
    ok = L.AlphaPoolShape(1, 8, 8, 4, 2, 2, 4, 4, 2, 2, 0, 0)
    assert lib.alpha_pool2D_max(C.byref(ok), p, p, None) == 0
    bad = L.AlphaPoolShape(1, 8, 8, 4, 2, 2, 5, 4, 2, 2, 0, 0)                       # OH does not follow
    assert lib.alpha_pool2D_max(C.byref(bad), p, p, None) == -1 and b"does not follow" in lib.alpha_conv_last_error()
    pad = L.AlphaPoolShape(1, 8, 8, 4, 2, 2, 5, 5, 2, 2, 2, 2)                       # padding as large as the window
    assert lib.alpha_pool2D_avg(C.byref(pad), p, p, 0, None) == -1 and b"padding" in lib.alpha_conv_last_error()
    assert lib.alpha_upool2D_max(C.byref(ok), p, None, p, p, None) == -1 and b"forward pass" in lib.alpha_conv_last_error()
    assert lib.alpha_pool2D_max_indexed(C.byref(ok), p, p, None, None) == -1 and b"index" in lib.alpha_conv_last_error()
    torch.cuda.synchronize()
