"""Driver of the reference's own cu32 CUDA kernels, rebuilt for sm_100 (TEST INFRASTRUCTURE).

`oracle/build_ref_gpu.sh` compiles the reference's Cuda_conv3D, Cuda_dconv3D_deltaX and
Cuda_dconv3D_deltaW libraries from its checkout into oracle/_ref/libcu32_*.so with their original JNI
entry points.  This module calls those entry points through a hand-made JNIEnv function table and
mirrors the kernel-family selection of CudaFloat32EngineBase
(src/alpha_src/z/dragon/engine/cuda/CudaFloat32EngineBase.java:1355-1474, 1666-1762, 1796-2005), so
that the tests can compare this repository's kernels with "what cu32 itself computes" on the same
GPU and the benchmark can time the reference's SIMT kernels on the same box.  Only tests/ and
bench.py may import it.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {}


def available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", "libcu32_%s.so" % n))
               for n in ("Cuda_conv3D", "Cuda_dconv3D_deltaX", "Cuda_dconv3D_deltaW"))


def reduce_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libcu32_Cuda_reduce.so"))


def field_nextN(N, M):
    """Rows of the partial-sum block the next stage reads (Cuda_reduce.java:35-45)."""
    if M > 15:
        if N > 63:
            return N >> 6
        if N > 15:
            return 1
    if M > 7:
        if N > 127:
            return N >> 7
        if N > 31:
            return 1
    return (N + 63) >> 6


def field_linear(X2d, alpha=1.0, beta=0.0):
    """The reference's Engine.field_sum on the GPU: CudaFloat32EngineBase.field_linear (:5811-5834) ->
    Cuda_reduce.field_linear (Cuda_reduce/A.cu:117-131): column sums of alpha * X + beta over the rows
    of X2d [N, M] (M a multiple of 4), with the partial-sum block V the Java side allocates."""
    lib = _lib("Cuda_reduce")
    f = lib.Java_z_dragon_engine_cuda_impl_math_Cuda_1reduce_field_1linear
    f.restype = C.c_int
    N, M = X2d.shape
    nxt = field_nextN(N, M)
    V = torch.empty(max(1, nxt * M), device=X2d.device, dtype=torch.float32)
    Y = torch.full((M,), float("nan"), device=X2d.device, dtype=torch.float32)
    torch.cuda.synchronize()
    f(None, None, C.c_int64(torch.cuda.current_stream().cuda_stream), C.c_int64(X2d.data_ptr()), C.c_float(alpha), C.c_float(beta),
      C.c_int(N), C.c_int(M), C.c_int64(V.data_ptr() if nxt != 1 else 0), C.c_int64(Y.data_ptr()), C.c_int(M), C.c_int(M), C.c_int(1))
    torch.cuda.synchronize()
    return Y


def matmul_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libcu32_Cuda_matMul.so"))


class Cu32MatMul:
    """The reference's matMul / matMulT1 / matMulT2 on the GPU, natives called as CudaFloat32EngineBase
    does (:1129-1245): matMulT1 switches to the split-K native plus SKbuf_summary from K = 512 on.
    `lib` is the rebuilt reference library by default; a test passes another implementation of the natives."""

    def __init__(self, lib=None, env=None):
        self.lib = lib if lib is not None else _lib("Cuda_matMul")
        self.env = env if env is not None else _FakeEnv()
        self.streams = [torch.cuda.Stream() for _ in range(10)]
        self.env.streams = [s.cuda_stream for s in self.streams]
        self.called = []

    def _call(self, name, *args):
        f = getattr(self.lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_" + name)
        f.restype = None
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(C.c_int64(a.data_ptr()))
            elif a == "streams":
                conv.append(C.c_void_p(0x5EED))
            elif isinstance(a, tuple) and a[0] == "long":
                conv.append(C.c_int64(a[1]))
            else:
                conv.append(C.c_int(int(a)))
        f(self.env.env, None, *conv)
        self.called.append(name)

    def matMul(self, A, B):
        (N, K), (_, M) = A.shape, B.shape
        Cm = torch.full((N, M), float("nan"), device=A.device, dtype=torch.float32)
        torch.cuda.synchronize()
        self._call("matMul", "streams", 10, A, B, Cm, N, M, K)
        torch.cuda.synchronize()
        return Cm

    def matMulT2(self, A, B):
        (N, K), (M, _) = A.shape, B.shape
        Cm = torch.full((N, M), float("nan"), device=A.device, dtype=torch.float32)
        torch.cuda.synchronize()
        self._call("matMulT2", "streams", 10, A, B, Cm, N, M, K)
        torch.cuda.synchronize()
        return Cm

    def matMulT1(self, A, B, threshold=512, max_part=16):
        (K, N), (_, M) = A.shape, B.shape
        Cm = torch.full((N, M), float("nan"), device=A.device, dtype=torch.float32)
        torch.cuda.synchronize()
        if K < threshold:
            self._call("matMulT1", "streams", 10, A, B, Cm, N, M, K)
        else:
            GridZ = K >> 8 if K < 1024 else (K >> 9 if K < 2048 else K >> 10)
            GridZ = min(GridZ, max_part)
            buf = torch.empty(max(1, N * M * (GridZ - 1)), device=A.device, dtype=torch.float32)
            self._call("matMulT1SK", "streams", 10, GridZ, A, B, Cm, buf, N, M, K)
            torch.cuda.synchronize()
            self._call("SKbuf_1summary", ("long", self.streams[0].cuda_stream), buf, Cm, GridZ - 1, N * M)
        torch.cuda.synchronize()
        return Cm


def _lib(name):
    if name not in _LIBS:
        _LIBS[name] = C.CDLL(os.path.join(_HERE, "_ref", "libcu32_%s.so" % name))
    return _LIBS[name]


class _FakeEnv:
    """JNIEnv whose GetLongArrayRegion (slot 204) hands out the stream handles of the current call."""

    def __init__(self):
        self.streams = []
        GETREGION = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64))
        FINDCLASS = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p)

        def get_region(env, arr, start, n, buf):
            for i in range(n):
                buf[i] = self.streams[start + i]

        def find_class(env, name):
            raise RuntimeError("the reference library raised a CUDA error (FindClass %r)" % name)
        self._cbs = [GETREGION(get_region), FINDCLASS(find_class)]
        self.table = (C.c_void_p * 235)()
        self.table[204] = C.cast(self._cbs[0], C.c_void_p)
        self.table[6] = C.cast(self._cbs[1], C.c_void_p)
        self.env = C.pointer(C.c_void_p(C.addressof(self.table)))


def _tile_count(g):
    """One factor of the Java blockNum helpers (Cuda_conv3D.java:19-42): tiles of 128..4 along g."""
    b = 0
    if g > 127:
        b += g >> 7
    g &= 127
    for t in (63, 31, 15, 7):
        if g == 0:
            return b
        if g > t:
            b += 1
        g &= t
    if g > 3:
        b += 1
    return b


class Cu32Reference:
    """The reference's conv3D / dconv3D_deltaX / dconv3D_deltaW on torch CUDA tensors (NHWC fp32,
    N, IC, OC multiples of 4).  Every call synchronises the device before and after."""

    N_STREAMS = 10

    def __init__(self, libs=None, env=None, fill=None):
        """libs: (conv3D, deltaX, deltaW) libraries that export the reference's JNI symbols - the
        rebuilt reference by default; a test passes another implementation of the same natives to
        drive it in the engine's call order.  env: a JNIEnv stand-in with `.env` and `.streams`.
        fill: value the output tensors hold before the natives run (NaN shows what a kernel left
        unwritten); None leaves them uninitialised."""
        if libs is None:
            if not available():
                raise ImportError("oracle/_ref/libcu32_*.so missing: run oracle/build_ref_gpu.sh where the reference is")
            libs = (_lib("Cuda_conv3D"), _lib("Cuda_dconv3D_deltaX"), _lib("Cuda_dconv3D_deltaW"))
        self.env = env if env is not None else _FakeEnv()
        self.streams = [torch.cuda.Stream() for _ in range(self.N_STREAMS)]
        self.env.streams = [s.cuda_stream for s in self.streams]
        self.c3, self.dx, self.dw = libs
        self.fill = fill
        self.last = ""
        self.called = []     # every native called so far, in order

    def _out(self, shape, device):
        if self.fill is None:
            return torch.empty(shape, device=device, dtype=torch.float32)
        return torch.full(shape, float(self.fill), device=device, dtype=torch.float32)

    # -- helpers -----------------------------------------------------------------------------------
    def _call(self, lib, name, *args):
        f = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_" + name)
        f.restype = None
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(C.c_int64(a.data_ptr()))
            elif isinstance(a, bool):
                conv.append(C.c_uint8(1 if a else 0))
            elif a == "streams":
                conv.append(C.c_void_p(0x5EED))  # the jlongArray handle; only the fake env looks at it
            elif isinstance(a, tuple) and a[0] == "long":
                conv.append(C.c_int64(a[1]))
            else:
                conv.append(C.c_int(int(a)))
        f(self.env.env, None, *conv)
        self.last = name
        self.called.append(name)

    @staticmethod
    def _scale_up(IH, IW, OH, OW, FH, FW, sh, sw):
        return ((OH - 1) * sh + FH) * ((OW - 1) * sw + FW) / float(IH * IW)

    # -- operators ---------------------------------------------------------------------------------
    def conv3D(self, X, W, sh, sw, ph, pw):
        """CudaFloat32EngineBase.conv3D (:1355-1474) with the default flags (remode, texture)."""
        N, IH, IW, IC = X.shape
        OC, FH, FW, _ = W.shape
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        Y = self._out((N, OH, OW, OC), X.device)
        L = self.N_STREAMS
        torch.cuda.synchronize()
        if OC > 31 and N * OH * OW > 31:
            V2 = N > 63 and OC > 63 and self._scale_up(IH, IW, OH, OW, FH, FW, sh, sw) > 1.05
            CW = torch.empty(FH * FW * IC * OC, device=X.device, dtype=torch.float32)
            self._call(self.c3, "Cuda_1conv3D_kernel_1remode", ("long", self.streams[0].cuda_stream), W, CW, FH, FW, OC, IC)
            torch.cuda.synchronize()
            if FH == 1 and FW == 1:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1GemmR_1W1", "streams", L, X, IH, IW, W, CW, Y, N, IC, OC)
            elif V2:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1GemmV2R", True, "streams", L, X, IH, IW, W, CW, FH, FW, Y, OH, OW,
                           N, IC, OC, sh, sw, ph, pw)
            else:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1GemmR_1texture", "streams", L, X, IH, IW, W, CW, FH, FW, Y, OH, OW,
                           N, IC, OC, sh, sw, ph, pw)
        else:
            V2 = N > 127 and OC > 127 and self._scale_up(IH, IW, OH, OW, FH, FW, sh, sw) >= 1.25
            tex = OC > 15
            if FH == 1 and FW == 1:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1W1", "streams", L, X, IH, IW, W, Y, N, IC, OC)
            elif ph == 0 and pw == 0:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1np", "streams", L, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw)
            elif V2:
                self._call(self.c3, "Cuda_1conv3D_conv3DV2", tex, "streams", L, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC,
                           sh, sw, ph, pw)
            elif tex:
                self._call(self.c3, "Cuda_1conv3D_conv3D_1texture", "streams", L, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC,
                           sh, sw, ph, pw)
            else:
                self._call(self.c3, "Cuda_1conv3D_conv3D", "streams", L, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw)
        torch.cuda.synchronize()
        return Y

    def dconv3D_deltaX(self, dY, W, IH, IW, sh, sw, ph, pw):
        """CudaFloat32EngineBase.dconv3D_deltaX (:1796-2005) with the default flags."""
        N, OH, OW, OC = dY.shape
        _, FH, FW, IC = W.shape
        dX = self._out((N, IH, IW, IC), dY.device)
        L = self.N_STREAMS
        P = "Cuda_1dconv3D_1deltaX_"
        torch.cuda.synchronize()
        if IC <= 8 or (IC <= 16 and sh * sw >= 4):
            self._call(self.dx, P + "dconv3D_1deltaX_1crossAdd", "streams", 7, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC,
                       sh, sw, ph, pw)
        elif FH == 1 and FW == 1:
            self._call(self.dx, P + "dconv3D_1deltaX_1W1", "streams", L, dY, W, dX, IH, IW, N, IC, OC)
        elif sh == 1 and sw == 1:
            V2 = N > 63 and IC > 63 and ((IH - 1 + FH) * (IW - 1 + FW)) / float(OH * OW) > 1.1
            tex = IC > 15
            if V2:
                self._call(self.dx, P + "dconv3D_1deltaX_1V2_1s1", tex, "streams", L, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw)
            elif tex:
                self._call(self.dx, P + "dconv3D_1deltaX_1s1_1texture", "streams", L, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw)
            else:
                self._call(self.dx, P + "dconv3D_1deltaX_1s1", "streams", L, dY, OH, OW, W, FH, FW, dX, IH, IW, N, IC, OC, ph, pw)
        else:
            CFH, CFW = (FH + sh - 1) // sh, (FW + sw - 1) // sw
            CW = torch.empty(OC * CFH * CFW * IC * sh * sw, device=dY.device, dtype=torch.float32)
            self._call(self.dx, P + "ks_1remodev2", ("long", self.streams[0].cuda_stream), W, FH, FW, CW, CFH, CFW, OC, IC, sh, sw)
            torch.cuda.synchronize()
            if sh == 2 and sw == 2 and IH % 2 == 0 and IW % 2 == 0:
                OH0, OW0 = (IH >> 1) + ((FH + 1) >> 1) - 1, (IW >> 1) + ((FW + 1) >> 1) - 1
                OH1, OW1 = (IH >> 1) + (FH >> 1) - 1, (IW >> 1) + (FW >> 1) - 1
                V2 = N > 63 and IC > 63 and 0.25 * ((OH0 + OH1) * (OW0 + OW1)) / (OH * OW) > 1.1
                if V2:
                    self._call(self.dx, P + "dconv3D_1deltaX_1ksV2_1Ims2R", False, "streams", L, dY, OH, OW, CW, FH, FW, dX, IH, IW,
                               N, IC, OC, ph, pw)
                else:
                    self._call(self.dx, P + "dconv3D_1deltaX_1ksIms2R", "streams", L, dY, OH, OW, CW, FH, FW, dX, IH, IW, N, IC, OC, ph, pw)
            elif IH % sh == 0 and IW % sw == 0:
                self._call(self.dx, P + "dconv3D_1deltaX_1ksImsR", "streams", L, dY, OH, OW, CW, FH, FW, dX, IH, IW, N, IC, OC,
                           sh, sw, ph, pw)
            else:
                self._call(self.dx, P + "dconv3D_1deltaX_1kernelSplit", "streams", L, dY, OH, OW, CW, FH, FW, dX, IH, IW, N, IC, OC,
                           sh, sw, ph, pw)
        torch.cuda.synchronize()
        return dX

    def dconv3D_deltaW(self, X, dY, FH, FW, sh, sw, ph, pw):
        """CudaFloat32EngineBase.dconv3D_deltaW (:1666-1762): split-K with GridZ from the block counts."""
        N, IH, IW, IC = X.shape
        _, OH, OW, OC = dY.shape
        dW = self._out((OC, FH, FW, IC), X.device)
        L = self.N_STREAMS
        P = "Cuda_1dconv3D_1deltaW_"
        GK = N * OH * OW
        torch.cuda.synchronize()
        if GK < 512:
            if FH == 1 and FW == 1:
                self._call(self.dw, P + "dconv3D_1deltaW_1W1", "streams", L, X, IH, IW, dY, dW, N, IC, OC)
            else:
                self._call(self.dw, P + "dconv3D_1deltaW", "streams", L, X, IH, IW, dY, OH, OW, dW, FH, FW, N, IC, OC, sh, sw, ph, pw)
        else:
            V2 = OC > 63 and IC > 63 and self._scale_up(IH, IW, OH, OW, FH, FW, sh, sw) >= 1.15
            if V2:
                b1 = _tile_count(OC) * _tile_count(N) * OH * OW
                b2 = _tile_count(IC) * _tile_count(N) * IH * IW
                b3 = _tile_count(OC) * _tile_count(IC) * FH * FW
            else:
                b1 = _tile_count(OC) * _tile_count(N * OH * OW)
                b2 = _tile_count(IC) * _tile_count(N * IH * IW)
                b3 = _tile_count(OC) * _tile_count(FH * FW * IC)
            GridZ = max(2, (b1 + b2) // (b3 << 1))
            GridZ = min(GridZ, 16, GK >> 8)
            sizeW = OC * FH * FW * IC
            buf = torch.empty(max(1, sizeW * (GridZ - 1)), device=X.device, dtype=torch.float32)
            if FH == 1 and FW == 1:
                self._call(self.dw, P + "dconv3D_1deltaW_1GemmSK_1W1", "streams", L, GridZ, X, IH, IW, dY, dW, buf, N, IC, OC)
            elif V2:
                self._call(self.dw, P + "dconv3D_1deltaW_1GemmV2SK", "streams", L, GridZ, X, IH, IW, dY, OH, OW, dW, buf, FH, FW,
                           N, IC, OC, sh, sw, ph, pw)
            else:
                self._call(self.dw, P + "dconv3D_1deltaW_1GemmSK", "streams", L, GridZ, X, IH, IW, dY, OH, OW, dW, buf, FH, FW,
                           N, IC, OC, sh, sw, ph, pw)
            torch.cuda.synchronize()
            self._call(self.dw, P + "buf_1summary", ("long", self.streams[0].cuda_stream), buf, dW, GridZ - 1, sizeW)
        torch.cuda.synchronize()
        return dW


def batch_matmul_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libcu32_Cuda_batchMatMul.so"))


class Cu32BatchMatMul(Cu32MatMul):
    """The reference's batchMatMul / batchMatMulT1 / batchMatMulT2 on the GPU, natives and texture switch as in
    CudaFloat32EngineBase (:1256-1318), on tensors in the engine's memory layout (last dimension padded to 4)."""

    def __init__(self, lib=None, env=None):
        super().__init__(lib if lib is not None else _lib("Cuda_batchMatMul"), env)

    def _call(self, name, *args):
        f = getattr(self.lib, "Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_" + name)
        f.restype = None
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(C.c_int64(a.data_ptr()))
            elif a == "streams":
                conv.append(C.c_void_p(0x5EED))
            else:
                conv.append(C.c_int(int(a)))
        f(self.env.env, None, *conv)
        self.called.append(name)

    def batchMatMul(self, A, B, texture=True):
        """A [Batch, N, AK], B [Batch, BK, M] -> C [Batch, N, M]."""
        (Bt, N, AK), (_, BK, M) = A.shape, B.shape
        Cm = torch.full((Bt, N, M), float("nan"), device=A.device, dtype=torch.float32)
        torch.cuda.synchronize()
        name = "batchMatMul_1texture" if (texture and N > 47 and M > 47) else "batchMatMul"
        self._call(name, "streams", 10, A, B, Cm, Bt, N, M, BK, AK)
        torch.cuda.synchronize()
        return Cm

    def batchMatMulT1(self, A, B, CN=None):
        """A [Batch, K, AN], B [Batch, K, M] -> C [Batch, CN, M]."""
        (Bt, K, AN), (_, _, M) = A.shape, B.shape
        CN = AN if CN is None else CN
        Cm = torch.full((Bt, CN, M), float("nan"), device=A.device, dtype=torch.float32)
        torch.cuda.synchronize()
        self._call("batchMatMulT1", "streams", 10, A, B, Cm, Bt, CN, AN, M, K)
        torch.cuda.synchronize()
        return Cm

    def batchMatMulT2(self, A, B, texture=True):
        """A [Batch, N, K], B [Batch, BM, K] -> C [Batch, N, CM], CM = BM rounded up to 4 (padding columns zero on entry)."""
        (Bt, N, K), (_, BM, _) = A.shape, B.shape
        CM = (BM + 3) & ~3
        Cm = torch.zeros((Bt, N, CM), device=A.device, dtype=torch.float32)
        Cm[..., :BM] = float("nan")
        torch.cuda.synchronize()
        name = "batchMatMulT2_1texture" if (texture and N > 47 and CM > 47) else "batchMatMulT2"
        self._call(name, "streams", 10, A, B, Cm, Bt, N, CM, BM, K)
        torch.cuda.synchronize()
        return Cm


def pool_available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", "libcu32_%s.so" % n)) for n in ("Cuda_pool2D", "Cuda_upool2D"))


class Cu32Pool:
    """The reference's pooling natives on the GPU (Cuda_pool2D, Cuda_upool2D) with the engine's choice of the tiled
    average gradient (CudaFloat32EngineBase.java:2147-2215).  The natives copy at most 4 stream handles
    (Cuda_pool2D/A.cu:18), so the harness passes 4.  Their kernels want IC % 4 == 0 and N * IH * IW % 4 == 0, which the
    engine's padding provides; callers of this class pad the same way.
    `libs` = (pool library, upool library), the rebuilt reference by default."""

    def __init__(self, libs=None, env=None):
        self.pool, self.upool = libs if libs is not None else (_lib("Cuda_pool2D"), _lib("Cuda_upool2D"))
        self.env = env if env is not None else _FakeEnv()
        self.streams = [torch.cuda.Stream() for _ in range(4)]
        self.env.streams = [s.cuda_stream for s in self.streams]
        self.called = []

    def _call(self, lib, cls, name, *args):
        f = getattr(lib, "Java_z_dragon_engine_cuda_impl_math_%s_%s" % (cls, name))
        f.restype = None
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                conv.append(C.c_int64(a.data_ptr()))
            elif a == "streams":
                conv.append(C.c_void_p(0x5EED))
            else:
                conv.append(C.c_int(int(a)))
        torch.cuda.synchronize()
        f(self.env.env, None, *conv)
        torch.cuda.synchronize()
        self.called.append(name)

    @staticmethod
    def _out_hw(IH, IW, FH, FW, sh, sw, ph, pw):
        return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1

    def pool2D(self, X, FH, FW, sh, sw, ph, pw, op="max"):
        N, IH, IW, IC = X.shape
        OH, OW = self._out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
        Y = torch.full((N, OH, OW, IC), float("nan"), device=X.device, dtype=torch.float32)
        if op == "max_indexed":
            Index = torch.full((N, OH, OW, IC), -1, device=X.device, dtype=torch.int32)
            self._call(self.pool, "Cuda_1pool2D", "pool2D_1max_1indexed", "streams", 4, X, IH, IW, FH, FW, Y, Index, OH, OW, N, IC, sh, sw, ph, pw)
            return Y, Index
        name = {"max": "pool2D_1max", "avg": "pool2D_1avg", "avg_ignore_padding": "pool2D_1avg_1ignore_1padding"}[op]
        self._call(self.pool, "Cuda_1pool2D", name, "streams", 4, X, IH, IW, FH, FW, Y, OH, OW, N, IC, sh, sw, ph, pw)
        return Y

    def upool2D(self, deltaY, IH, IW, FH, FW, sh, sw, ph, pw, op="max", Y=None, X=None, Index=None):
        N, OH, OW, IC = deltaY.shape
        # the tiled kernels write only the elements a window covers: the engine hands them a zeroed tensor
        dX = torch.zeros((N, IH, IW, IC), device=deltaY.device, dtype=torch.float32)
        if op == "max":
            self._call(self.upool, "Cuda_1upool2D", "upool2D_1max", "streams", 4, deltaY, Y, OH, OW, FH, FW, dX, X, IH, IW, N, IC, sh, sw, ph, pw)
        elif op == "max_indexed":
            self._call(self.upool, "Cuda_1upool2D", "upool2D_1max_1Indexed", "streams", 4, deltaY, Index, OH, OW, FH, FW, dX, IH, IW, N, IC, sh, sw, ph, pw)
        else:
            name = "upool2D_1avg" if op == "avg" else "upool2D_1avg_1ignore_1padding"
            if FH == sh and FW == sw:
                name += "_1tiled"
            self._call(self.upool, "Cuda_1upool2D", name, "streams", 4, deltaY, OH, OW, FH, FW, dX, IH, IW, N, IC, sh, sw, ph, pw)
        return dX
