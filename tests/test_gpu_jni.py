"""The JNI entry points themselves on the GPU: the symbols the Java classes bind, called with a
fake JNIEnv (function table at the specification's slots) and device addresses, in the order the
engine calls them (CudaFloat32EngineBase.conv3D / dconv3D_deltaX / dconv3D_deltaW)."""
import ctypes as C

import numpy as np
import pytest

from helpers import TOL, gen, metrics

pytestmark = pytest.mark.gpu
PFX = "Java_z_dragon_engine_cuda_impl_math_"


class FakeEnv:
    def __init__(self, streams):
        self.thrown = None
        self.streams = list(streams)
        FINDCLASS = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p)
        THROWNEW = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_char_p)
        GETREGION = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64))
        EXCCHECK = C.CFUNCTYPE(C.c_uint8, C.c_void_p)

        def throw_new(env, cls, msg):
            self.thrown = msg
            return 0

        def get_region(env, arr, start, n, buf):
            for i in range(n):
                buf[i] = self.streams[start + i]
        self._cbs = [FINDCLASS(lambda env, name: 0x77), THROWNEW(throw_new), GETREGION(get_region), EXCCHECK(lambda env: 0)]
        self._table = (C.c_void_p * 235)()
        for slot, cb in zip((6, 14, 204, 228), self._cbs):
            self._table[slot] = C.cast(cb, C.c_void_p)
        self._envp = C.c_void_p(C.addressof(self._table))
        self.env = C.pointer(self._envp)


def _fn(lib, name, argtypes):
    f = getattr(lib, PFX + name)
    f.restype = None
    f.argtypes = [C.c_void_p, C.c_void_p] + argtypes
    return f


def test_jni_natives_compute_on_the_gpu(pkg, oracle_mod):
    import torch
    L = pkg.submodule("lib")
    lib = L.load()
    L.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    O = oracle_mod
    N, IH, IC, OC, F = 8, 16, 32, 64, 3
    rng = np.random.default_rng(3)
    X = gen((N, IH, IH, IC), "u11", rng); W = gen((OC, F, F, IC), "u11", rng); dY = gen((N, IH, IH, OC), "n01", rng)
    tX, tW, tdY = (torch.from_numpy(a).to(dev) for a in (X, W, dY))
    tCW = torch.empty_like(tW)
    tY = torch.empty((N, IH, IH, OC), device=dev); tdX = torch.empty_like(tX); tdW = torch.empty_like(tW)
    GridZ = 4
    tbuf = torch.full(((GridZ - 1) * tW.numel(),), 7.0, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    env = FakeEnv([stream, stream, stream, stream])
    I, J = C.c_int, C.c_int64
    arr = C.c_void_p(0x1000)   # opaque jlongArray handle, only passed back to GetLongArrayRegion

    remode = _fn(lib, "Cuda_1conv3D_kernel_1remode", [J, J, J, I, I, I, I])
    remode(env.env, None, stream, tW.data_ptr(), tCW.data_ptr(), F, F, OC, IC)
    fwd = _fn(lib, "Cuda_1conv3D_conv3D_1GemmR", [C.c_void_p, I, J, I, I, J, J, I, I, J, I, I, I, I, I, I, I, I, I])
    fwd(env.env, None, arr, 4, tX.data_ptr(), IH, IH, tW.data_ptr(), tCW.data_ptr(), F, F, tY.data_ptr(), IH, IH, N, IC, OC, 1, 1, 1, 1)
    dx = _fn(lib, "Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1", [C.c_void_p, I, J, I, I, J, I, I, J, I, I, I, I, I, I, I])
    dx(env.env, None, arr, 4, tdY.data_ptr(), IH, IH, tW.data_ptr(), F, F, tdX.data_ptr(), IH, IH, N, IC, OC, 1, 1)
    dw = _fn(lib, "Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmSK",
             [C.c_void_p, I, I, J, I, I, J, I, I, J, J, I, I, I, I, I, I, I, I, I])
    dw(env.env, None, arr, 4, GridZ, tX.data_ptr(), IH, IH, tdY.data_ptr(), IH, IH, tdW.data_ptr(), tbuf.data_ptr(), F, F, N, IC, OC,
       1, 1, 1, 1)
    summ = _fn(lib, "Cuda_1dconv3D_1deltaW_buf_1summary", [J, J, J, I, I])
    summ(env.env, None, stream, tbuf.data_ptr(), tdW.data_ptr(), GridZ - 1, tW.numel())
    torch.cuda.synchronize()
    assert env.thrown is None, env.thrown
    assert L.device_status() == 0
    tol = TOL["3xtf32"]
    for name, got, ref in (("fwd", tY, O.conv3D_f64(X, W, 1, 1, 1, 1, threads=8)),
                           ("dx", tdX, O.deconv3D_deltaX_f64(dY, W, IH, IH, 1, 1, 1, 1, threads=8)),
                           ("dw", tdW, O.deconv3D_deltaW_f64(X, dY, F, F, 1, 1, 1, 1, threads=8))):
        m = metrics(got.cpu().numpy(), *ref)
        assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (name, m)


def test_jni_native_reports_a_bad_call_as_exception(pkg):
    import torch
    L = pkg.submodule("lib")
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    env = FakeEnv([stream])
    I, J = C.c_int, C.c_int64
    fwd = _fn(lib, "Cuda_1conv3D_conv3D_1GemmR", [C.c_void_p, I, J, I, I, J, J, I, I, J, I, I, I, I, I, I, I, I, I])
    fwd(env.env, None, C.c_void_p(1), 1, 0, 8, 8, 0, 0, 3, 3, 0, 8, 8, 4, 8, 8, 1, 1, 1, 1)   # null tensors
    assert env.thrown is not None and b"null" in env.thrown


# ---- every native, in the order and with the selection rules of the Java engine --------------------------
#
# oracle.cu32_ref.Cu32Reference mirrors CudaFloat32EngineBase.conv3D / dconv3D_deltaX / dconv3D_deltaW
# (:1355-1474, 1666-1762, 1796-2005): which native is called for which shape, with kernel_remode /
# ks_remodev2 before the consumers and buf_summary after the split-K natives.  Given this library
# instead of the rebuilt reference it drives the same chains through our Java_... symbols.
# Shapes: (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw) -> the native the engine picks.
FWD_CASES = {
    "conv3D_GemmR_W1": (8, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "conv3D_GemmV2R": (64, 7, 7, 32, 64, 3, 3, 1, 1, 1, 1),
    "conv3D_GemmR_texture": (8, 16, 16, 32, 64, 3, 3, 1, 1, 1, 1),
    "conv3D_W1": (8, 8, 8, 32, 16, 1, 1, 1, 1, 0, 0),
    "conv3D_np": (4, 10, 10, 32, 16, 3, 3, 1, 1, 0, 0),
    "conv3D_texture": (4, 12, 12, 16, 16, 3, 3, 1, 1, 1, 1),
    "conv3D": (4, 12, 12, 16, 8, 3, 3, 1, 1, 1, 1),
}
DX_CASES = {
    "dconv3D_deltaX_crossAdd": (4, 16, 16, 4, 32, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaX_crossAdd/stem": (4, 32, 32, 4, 64, 7, 7, 2, 2, 3, 3),
    "dconv3D_deltaX_W1": (8, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "dconv3D_deltaX_V2_s1": (64, 7, 7, 64, 64, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaX_s1_texture": (8, 14, 14, 64, 64, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaX_s1": (4, 12, 12, 12, 32, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaX_ksV2_Ims2R": (64, 8, 8, 64, 64, 3, 3, 2, 2, 1, 1),
    "dconv3D_deltaX_ksIms2R": (8, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
    "dconv3D_deltaX_ksIms2R/4x4": (8, 16, 16, 32, 64, 4, 4, 2, 2, 1, 1),
    "dconv3D_deltaX_ksImsR": (4, 12, 12, 32, 32, 3, 3, 3, 3, 0, 0),
    "dconv3D_deltaX_kernelSplit": (4, 11, 11, 32, 32, 3, 3, 2, 2, 1, 1),
}
DW_CASES = {
    "dconv3D_deltaW_W1": (4, 8, 8, 32, 32, 1, 1, 1, 1, 0, 0),
    "dconv3D_deltaW": (4, 8, 8, 32, 32, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaW_GemmSK_W1": (8, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "dconv3D_deltaW_GemmV2SK": (16, 7, 7, 64, 64, 3, 3, 1, 1, 1, 1),
    "dconv3D_deltaW_GemmSK": (8, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
}
_EXECUTED = set()


@pytest.fixture(scope="module")
def jni(pkg):
    import torch
    from oracle.cu32_ref import Cu32Reference
    torch.cuda.set_device(0)
    L = pkg.submodule("lib")
    lib = L.load()
    env = FakeEnv([])
    return Cu32Reference(libs=(lib, lib, lib), env=env, fill=float("nan")), env, L


def _mangled(native):
    return native.replace("_", "_1")


def _check(L, env, got, ref64, what):
    assert env.thrown is None, (what, env.thrown)
    assert L.device_status() == 0
    m = metrics(got.cpu().numpy(), *ref64)
    tol = TOL["3xtf32"]
    assert m["finite"] and m["norm"] <= tol["norm"] and m["comp"] <= tol["comp"], (what, m)


def _inputs(case, seed):
    import torch
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    rng = np.random.default_rng(seed)
    X, W, dY = gen((N, IH, IW, IC), "u11", rng), gen((OC, FH, FW, IC), "u11", rng), gen((N, OH, OW, OC), "n01", rng)
    dev = torch.device("cuda:0")
    return X, W, dY, [torch.from_numpy(a).to(dev) for a in (X, W, dY)]


@pytest.mark.parametrize("native", list(FWD_CASES))
def test_forward_natives_in_engine_order(jni, oracle_mod, native):
    eng, env, L = jni
    L.set_math_mode("3xtf32")
    case = FWD_CASES[native]
    X, W, dY, (tX, tW, tdY) = _inputs(case, 11)
    sh, sw, ph, pw = case[7:]
    n0 = len(eng.called)
    Y = eng.conv3D(tX, tW, sh, sw, ph, pw)
    assert eng.called[-1] == "Cuda_1conv3D_" + _mangled(native), eng.called[n0:]
    _EXECUTED.update(eng.called[n0:])
    _check(L, env, Y, oracle_mod.conv3D_f64(X, W, sh, sw, ph, pw, threads=8), native)


@pytest.mark.parametrize("name", list(DX_CASES))
def test_deltaX_natives_in_engine_order(jni, oracle_mod, name):
    eng, env, L = jni
    L.set_math_mode("3xtf32")
    case = DX_CASES[name]
    X, W, dY, (tX, tW, tdY) = _inputs(case, 12)
    IH, IW = case[1], case[2]
    sh, sw, ph, pw = case[7:]
    n0 = len(eng.called)
    dX = eng.dconv3D_deltaX(tdY, tW, IH, IW, sh, sw, ph, pw)
    native = name.split("/")[0]
    assert eng.called[-1] == "Cuda_1dconv3D_1deltaX_" + _mangled(native), eng.called[n0:]
    if sh * sw > 1 and case[3] > 16:
        assert eng.called[-2].endswith("ks_1remodev2")      # the consumer only ever saw CW
    _EXECUTED.update(eng.called[n0:])
    _check(L, env, dX, oracle_mod.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=8), name)


@pytest.mark.parametrize("native", list(DW_CASES))
def test_deltaW_natives_in_engine_order(jni, oracle_mod, native):
    eng, env, L = jni
    L.set_math_mode("3xtf32")
    case = DW_CASES[native]
    X, W, dY, (tX, tW, tdY) = _inputs(case, 13)
    FH, FW, sh, sw, ph, pw = case[5:]
    n0 = len(eng.called)
    dW = eng.dconv3D_deltaW(tX, tdY, FH, FW, sh, sw, ph, pw)
    names = eng.called[n0:]
    assert "Cuda_1dconv3D_1deltaW_" + _mangled(native) in names, names
    if "SK" in native:
        assert names[-1].endswith("buf_1summary")
    _EXECUTED.update(names)
    _check(L, env, dW, oracle_mod.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8), native)


def test_natives_the_default_flags_never_pick(jni, oracle_mod):
    """conv3DV2, conv3D_GemmR, ks_remode -> ksImsR_texture / ksIms2R_texture: reached in the Java engine only
    with non-default option flags (conv3D_remode(false), conv3D_useTexture(false), dconv3D_deltaX_ks_useTexture(true))."""
    import torch
    eng, env, L = jni
    L.set_math_mode("3xtf32")
    O = oracle_mod
    S = "streams"
    n0 = len(eng.called)
    # forward, 3x3: non-remode V2 entry, remode entry without texture
    case = (8, 16, 16, 32, 64, 3, 3, 1, 1, 1, 1)
    X, W, dY, (tX, tW, tdY) = _inputs(case, 14)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    ref = O.conv3D_f64(X, W, sh, sw, ph, pw, threads=8)
    Y = torch.full((N, IH, IW, OC), float("nan"), device=tX.device)
    eng._call(eng.c3, "Cuda_1conv3D_conv3DV2", True, S, 10, tX, IH, IW, tW, FH, FW, Y, IH, IW, N, IC, OC, sh, sw, ph, pw)
    torch.cuda.synchronize()
    _check(L, env, Y, ref, "conv3DV2")
    CW = torch.empty_like(tW)
    Y.fill_(float("nan"))
    eng._call(eng.c3, "Cuda_1conv3D_kernel_1remode", ("long", eng.streams[0].cuda_stream), tW, CW, FH, FW, OC, IC)
    torch.cuda.synchronize()
    eng._call(eng.c3, "Cuda_1conv3D_conv3D_1GemmR", S, 10, tX, IH, IW, tW, CW, FH, FW, Y, IH, IW, N, IC, OC, sh, sw, ph, pw)
    torch.cuda.synchronize()
    _check(L, env, Y, ref, "conv3D_GemmR")
    # strided deltaX through ks_remode (first version) and the texture consumers
    P = "Cuda_1dconv3D_1deltaX_"
    for native, case in (("dconv3D_1deltaX_1ksIms2R_1texture", (8, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1)),
                         ("dconv3D_1deltaX_1ksImsR_1texture", (4, 12, 12, 32, 32, 5, 5, 3, 3, 1, 1))):
        X, W, dY, (tX, tW, tdY) = _inputs(case, 15)
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        OH, OW = tdY.shape[1], tdY.shape[2]
        CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
        CW = torch.full((OC * CFH * CFW * IC * sh * sw,), float("nan"), device=tX.device)
        dX = torch.full((N, IH, IW, IC), float("nan"), device=tX.device)
        eng._call(eng.dx, P + "ks_1remode", ("long", eng.streams[0].cuda_stream), tW, FH, FW, CW, CFH, CFW, OC, IC, sh, sw)
        torch.cuda.synchronize()
        tW_gone = torch.full_like(tW, float("nan"))   # the consumer must not need W any more
        if "Ims2R" in native:
            eng._call(eng.dx, P + native, S, 10, tdY, OH, OW, CW, FH, FW, dX, IH, IW, N, IC, OC, ph, pw)
        else:
            eng._call(eng.dx, P + native, S, 10, tdY, OH, OW, CW, FH, FW, dX, IH, IW, N, IC, OC, sh, sw, ph, pw)
        torch.cuda.synchronize()
        del tW_gone
        _check(L, env, dX, O.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=8), native)
    _EXECUTED.update(eng.called[n0:])


def test_buf_summary_adds_nonzero_buffers(jni):
    """deltaW += sum of `part` buffers (Cuda_dconv3D_deltaW/A.cu:66, dconv3d_dW_GemmSK_bufSum.cuh:32-67),
    on buffers that hold numbers: compared with the sum formed in double precision."""
    import torch
    eng, env, L = jni
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(21)
    for part, sizeW in ((1, 64 * 9 * 32), (3, 96 * 64), (15, 128 * 9 * 128), (127, 2304)):
        dW = torch.randn(sizeW, device=dev, generator=g)
        buf = torch.randn(part * sizeW, device=dev, generator=g) * 3.0
        want = dW.double() + buf.double().view(part, sizeW).sum(0)
        scale = dW.abs().double() + buf.abs().double().view(part, sizeW).sum(0)
        eng._call(eng.dw, "Cuda_1dconv3D_1deltaW_buf_1summary", ("long", eng.streams[0].cuda_stream), buf, dW, part, sizeW)
        torch.cuda.synchronize()
        assert env.thrown is None, env.thrown
        # a compensated fp32 sum is within an ulp or two of the rounded exact sum
        assert float(((dW.double() - want).abs() / scale).max()) <= 2.5e-7, (part, sizeW)
    _EXECUTED.add("Cuda_1dconv3D_1deltaW_buf_1summary")


def test_zz_at_least_twenty_natives_ran_on_the_gpu():
    """Runs last in this file: the tests above must have executed most of the 29 natives."""
    assert len(_EXECUTED) >= 26, sorted(_EXECUTED)
