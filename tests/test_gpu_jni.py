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
        FINDCLASS = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p)
        THROWNEW = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_char_p)
        GETREGION = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64))
        EXCCHECK = C.CFUNCTYPE(C.c_uint8, C.c_void_p)

        def throw_new(env, cls, msg):
            self.thrown = msg
            return 0

        def get_region(env, arr, start, n, buf):
            for i in range(n):
                buf[i] = streams[start + i]
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
