"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

`liboracle.so` is the plain-C restatement of the reference's Java CPU loops
(src/zutil_src/z/util/math/vector/Tense.java); `_ref/libref_cpu.so`, when it has been built from a
reference checkout, holds the reference project's own C++ loops (test.cuh of each cu32 library).
Only the test suite, the smoke check and the benchmark's CPU-baseline legs may import this module.

All arrays are C-contiguous float32 NHWC: X[N,IH,IW,IC], W[OC,FH,FW,IC], Y[N,OH,OW,OC].
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_F = C.POINTER(C.c_float)
_D = C.POINTER(C.c_double)
_i = C.c_int


def build(ref_root="/root/reference"):
    """Compile liboracle.so, and _ref/libref_cpu.so when a reference checkout is present."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    if os.path.isdir(os.path.join(ref_root, "src", "cu32_src")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REF=" + ref_root])


def _load(path):
    if not os.path.exists(path):
        return None
    return C.CDLL(path)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _lib = C.CDLL(path)
        _lib.oracle_samePercentRelative.restype = C.c_float
        _lib.oracle_max_threads.restype = C.c_int
    return _lib


def ref_lib():
    """The reference's own C++ loops, or None when they were never built on this machine."""
    global _ref
    if _ref is None:
        _ref = _load(os.path.join(_HERE, "_ref", "libref_cpu.so"))
    return _ref


def max_threads():
    return int(lib().oracle_max_threads())


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_F)


def out_hw(IH, IW, FH, FW, sh, sw, ph, pw):
    """OH, OW as Cuda_conv3D.java:154-155 computes them."""
    return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1


def conv3D_naive(X, W, sh, sw, ph, pw, threads=1):
    """Tense.conv3D_naive (Tense.java:143-173): double accumulator over float products."""
    N, IH, IW, IC = X.shape
    OC, FH, FW, _ = W.shape
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    X, px = _f(X)
    W, pw_ = _f(W)
    Y = np.zeros((N, OH, OW, OC), np.float32)
    lib().oracle_conv3D_naive(px, _i(IH), _i(IW), pw_, _i(FH), _i(FW), Y.ctypes.data_as(_F),
                              _i(OH), _i(OW), _i(N), _i(IC), _i(OC), _i(sh), _i(sw), _i(ph),
                              _i(pw), _i(threads))
    return Y


def conv3D_naive_f32(X, W, sh, sw, ph, pw, threads=1):
    """CONV_3D_NAIVE restated (Cuda_conv3D/test.cuh:80-110): float accumulator."""
    N, IH, IW, IC = X.shape
    OC, FH, FW, _ = W.shape
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    X, px = _f(X)
    W, pw_ = _f(W)
    Y = np.zeros((N, OH, OW, OC), np.float32)
    lib().oracle_conv3D_naive_f32(px, _i(IH), _i(IW), pw_, _i(FH), _i(FW), Y.ctypes.data_as(_F),
                                  _i(OH), _i(OW), _i(N), _i(IC), _i(OC), _i(sh), _i(sw), _i(ph),
                                  _i(pw), _i(threads))
    return Y


def conv3D_f64(X, W, sh, sw, ph, pw, threads=1):
    """fp64 forward conv and S = sum|x||w| per output (error analysis)."""
    N, IH, IW, IC = X.shape
    OC, FH, FW, _ = W.shape
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    X, px = _f(X)
    W, pw_ = _f(W)
    Y = np.zeros((N, OH, OW, OC), np.float64)
    S = np.zeros((N, OH, OW, OC), np.float64)
    lib().oracle_conv3D_f64(px, _i(IH), _i(IW), pw_, _i(FH), _i(FW), Y.ctypes.data_as(_D),
                            S.ctypes.data_as(_D), _i(OH), _i(OW), _i(N), _i(IC), _i(OC), _i(sh),
                            _i(sw), _i(ph), _i(pw), _i(threads))
    return Y, S


def add_bias_row(Y, bias):
    """Y[..., oc] += bias[oc] in float (conv3D_biased's linear_dual2D_row stage)."""
    Y = np.ascontiguousarray(Y, np.float32).copy()
    b, pb = _f(bias)
    lib().oracle_add_bias_row(Y.ctypes.data_as(_F), pb, C.c_size_t(Y.size // Y.shape[-1]),
                              _i(Y.shape[-1]))
    return Y


def field_sum(X, row_length=-1):
    """Column sums of X seen as [rows][row_length], accumulated row after row in float as the
    reference's CPU loop does (z/util/math/vector/Matrix.java:2119-2127, field_linear with alpha = 1,
    beta = 0; Engine.field_sum, Engine.java:6945, is the GPU operator Conv3D's backward pass calls
    for the bias gradient).  The reference holds no golden vector for it; it is pinned on the GPU box
    against the reference's own Cuda_reduce.field_linear kernel rebuilt from its checkout
    (oracle/cu32_ref.field_linear, tests/test_gpu_field_sum.py)."""
    X = np.ascontiguousarray(X, np.float32)
    if row_length == -1:
        row_length = X.shape[-1]
    A = X.reshape(-1, row_length)
    return np.cumsum(A, axis=0, dtype=np.float32)[-1].copy()


def field_sum_f64(X, row_length=-1):
    """The same sums in double, and the sums of magnitudes that scale the error bound."""
    X = np.ascontiguousarray(X, np.float32)
    if row_length == -1:
        row_length = X.shape[-1]
    A = X.reshape(-1, row_length).astype(np.float64)
    return A.sum(axis=0), np.abs(A).sum(axis=0)


def deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw, threads=1):
    """Tense.deconv3D_deltaX_img2col (Tense.java:334-375): float accumulator."""
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    dY, pdy = _f(dY)
    W, pw_ = _f(W)
    dX = np.zeros((N, IH, IW, IC), np.float32)
    lib().oracle_deconv3D_deltaX_img2col(pdy, _i(OH), _i(OW), pw_, _i(FH), _i(FW),
                                         dX.ctypes.data_as(_F), _i(IH), _i(IW), _i(N), _i(IC),
                                         _i(OC), _i(sh), _i(sw), _i(ph), _i(pw), _i(threads))
    return dX


def deconv3D_deltaX_crossAdd(dY, W, IH, IW, sh, sw, ph, pw):
    """Tense.deconv3D_deltaX_crossAdd (Tense.java:441-469): scatter form, float adds."""
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    dY, pdy = _f(dY)
    W, pw_ = _f(W)
    dX = np.zeros((N, IH, IW, IC), np.float32)
    lib().oracle_deconv3D_deltaX_crossAdd(pdy, _i(OH), _i(OW), pw_, _i(FH), _i(FW),
                                          dX.ctypes.data_as(_F), _i(IH), _i(IW), _i(N), _i(IC),
                                          _i(OC), _i(sh), _i(sw), _i(ph), _i(pw))
    return dX


def deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=1):
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    dY, pdy = _f(dY)
    W, pw_ = _f(W)
    dX = np.zeros((N, IH, IW, IC), np.float64)
    S = np.zeros((N, IH, IW, IC), np.float64)
    lib().oracle_deconv3D_deltaX_f64(pdy, _i(OH), _i(OW), pw_, _i(FH), _i(FW),
                                     dX.ctypes.data_as(_D), S.ctypes.data_as(_D), _i(IH), _i(IW),
                                     _i(N), _i(IC), _i(OC), _i(sh), _i(sw), _i(ph), _i(pw),
                                     _i(threads))
    return dX, S


def deconv3D_deltaW_img2col2(X, dY, FH, FW, sh, sw, ph, pw, threads=1):
    """Tense.deconv3D_deltaW_img2col2 (Tense.java:1364-1401): float accumulator."""
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = dY.shape
    X, px = _f(X)
    dY, pdy = _f(dY)
    dW = np.zeros((OC, FH, FW, IC), np.float32)
    lib().oracle_deconv3D_deltaW_img2col2(px, _i(IH), _i(IW), pdy, _i(OH), _i(OW),
                                          dW.ctypes.data_as(_F), _i(FH), _i(FW), _i(N), _i(IC),
                                          _i(OC), _i(sh), _i(sw), _i(ph), _i(pw), _i(threads))
    return dW


def deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw, threads=1):
    """Tense.deconv3d_deltaW_naive (Tense.java:1277-1319): double accumulator."""
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = dY.shape
    X, px = _f(X)
    dY, pdy = _f(dY)
    dW = np.zeros((OC, FH, FW, IC), np.float32)
    lib().oracle_deconv3d_deltaW_naive(px, _i(IH), _i(IW), pdy, _i(OH), _i(OW),
                                       dW.ctypes.data_as(_F), _i(FH), _i(FW), _i(N), _i(IC),
                                       _i(OC), _i(sh), _i(sw), _i(ph), _i(pw), _i(threads))
    return dW


def deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=1):
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = dY.shape
    X, px = _f(X)
    dY, pdy = _f(dY)
    dW = np.zeros((OC, FH, FW, IC), np.float64)
    S = np.zeros((OC, FH, FW, IC), np.float64)
    lib().oracle_deconv3D_deltaW_f64(px, _i(IH), _i(IW), pdy, _i(OH), _i(OW),
                                     dW.ctypes.data_as(_D), S.ctypes.data_as(_D), _i(FH), _i(FW),
                                     _i(N), _i(IC), _i(OC), _i(sh), _i(sw), _i(ph), _i(pw),
                                     _i(threads))
    return dW, S


def samePercentRelative(A, B, threshold):
    """Vector.samePercentRelative (Vector.java:4109-4125)."""
    A, pa = _f(np.ravel(A))
    B, pb = _f(np.ravel(B))
    return float(lib().oracle_samePercentRelative(pa, pb, C.c_size_t(A.size), C.c_float(threshold)))


# ---- the reference's own C++ loops (only where _ref/libref_cpu.so was built) -------------------

def ref_CONV_3D_NAIVE(X, W, sh, sw, ph, pw):
    """CONV_3D_NAIVE, src/cu32_src/Cuda_conv3D/Cuda_conv3D/test.cuh:80-110 (float accumulator)."""
    N, IH, IW, IC = X.shape
    OC, FH, FW, _ = W.shape
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    X, px = _f(X)
    W, pw_ = _f(W)
    Y = np.zeros((N, OH, OW, OC), np.float32)
    ref_lib().ref_CONV_3D_NAIVE(px, _i(IH), _i(IW), pw_, _i(FH), _i(FW), Y.ctypes.data_as(_F),
                                _i(OH), _i(OW), _i(N), _i(IC), _i(OC), _i(sh), _i(sw), _i(ph),
                                _i(pw))
    return Y


def ref_deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw):
    """deconv3D_deltaX_img2col, src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/test.cuh:89-131."""
    N, OH, OW, OC = dY.shape
    _, FH, FW, IC = W.shape
    dY, pdy = _f(dY)
    W, pw_ = _f(W)
    dX = np.zeros((N, IH, IW, IC), np.float32)
    ref_lib().ref_deconv3D_deltaX_img2col(pdy, _i(OH), _i(OW), pw_, _i(FH), _i(FW),
                                          dX.ctypes.data_as(_F), _i(IH), _i(IW), _i(N), _i(IC),
                                          _i(OC), _i(sh), _i(sw), _i(ph), _i(pw))
    return dX


def ref_deconv3D_deltaW_img2col2(X, dY, FH, FW, sh, sw, ph, pw):
    """deconv3D_deltaW_img2col2, src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/test.cuh:77-121."""
    N, IH, IW, IC = X.shape
    _, OH, OW, OC = dY.shape
    X, px = _f(X)
    dY, pdy = _f(dY)
    dW = np.zeros((OC, FH, FW, IC), np.float32)
    ref_lib().ref_deconv3D_deltaW_img2col2(px, _i(IH), _i(IW), pdy, _i(OH), _i(OW),
                                           dW.ctypes.data_as(_F), _i(FH), _i(FW), _i(N), _i(IC),
                                           _i(OC), _i(sh), _i(sw), _i(ph), _i(pw))
    return dW


# ---- matrix products (FullConnect path) ----------------------------------------------------------

_MM_VARIANT = {"matMul": 0, "matMulT1": 1, "matMulT2": 2}


def _mm_dims(A, B, variant):
    if variant == 0:
        (N, K), (K2, M) = A.shape, B.shape
    elif variant == 1:
        (K, N), (K2, M) = A.shape, B.shape
    else:
        (N, K), (M, K2) = A.shape, B.shape
    if K != K2:
        raise ValueError("inner dimensions differ: %d, %d" % (K, K2))
    return N, M, K


def matmul(A, B, variant="matMul"):
    """C = A*B ('matMul', A[N,K], B[K,M]), A^T*B ('matMulT1', A[K,N], B[K,M]) or A*B^T ('matMulT2', A[N,K], B[M,K]) with
    the float loops of the reference's own tests (Cuda_matMul_test*.java:27-36; Cuda_matMul/test.cuh:59-81)."""
    v = _MM_VARIANT[variant]
    A, pa = _f(A)
    B, pb = _f(B)
    N, M, K = _mm_dims(A, B, v)
    Cm = np.empty((N, M), np.float32)
    lib().oracle_matmul(pa, pb, Cm.ctypes.data_as(_F), _i(N), _i(M), _i(K), _i(v))
    return Cm


def matmul_f64(A, B, variant="matMul", threads=1):
    """The same product in double, and S = sum_k |a||b| per element."""
    v = _MM_VARIANT[variant]
    A, pa = _f(A)
    B, pb = _f(B)
    N, M, K = _mm_dims(A, B, v)
    Cm, S = np.empty((N, M), np.float64), np.empty((N, M), np.float64)
    lib().oracle_matmul_f64(pa, pb, Cm.ctypes.data_as(_D), S.ctypes.data_as(_D), _i(N), _i(M), _i(K), _i(v), _i(threads))
    return Cm, S


def ref_matmul(A, B, variant="matMul"):
    """The reference project's own C++ loop (multiply / multiplyT1 / multiplyT2 of Cuda_matMul/test.cuh)."""
    v = _MM_VARIANT[variant]
    A, pa = _f(A)
    B, pb = _f(B)
    N, M, K = _mm_dims(A, B, v)
    Cm = np.zeros((N, M), np.float32)
    fn = getattr(ref_lib(), ("ref_multiply", "ref_multiplyT1", "ref_multiplyT2")[v])
    fn(pa, pb, Cm.ctypes.data_as(_F), _i(N), _i(M), _i(K))
    return Cm


_BMM_VARIANT = {"batchMatMul": 0, "batchMatMulT1": 1, "batchMatMulT2": 2}


def _bmm_dims(A, B, v, M):
    """Logical (Batch, N, M, K) and the padded pitch p of a batched product from the MEMORY shapes of A and B
    (last dimension padded to 4 by the engine) and the logical M (variant 2: rows of B = M)."""
    if v == 0:      # A [Batch, N, AK], B [Batch, K, M]
        (Bt, N, p), (_, K, M) = A.shape, B.shape
    elif v == 1:    # A [Batch, K, AN], B [Batch, K, M]; N given through M's slot is not needed: C rows = CN
        (Bt, K, p), (_, _, M) = A.shape, B.shape
        N = None
    else:           # A [Batch, N, K], B [Batch, BM, K]; p = CM
        (Bt, N, K), (_, M, _) = A.shape, B.shape
        p = (M + 3) & ~3
    return Bt, N, M, K, p


def batch_matmul(A, B, variant="batchMatMul", rows=None, threads=1, f64=False):
    """The reference's batched products on the engine's memory layout (Cuda_batchMatMul/test.cuh:95-140):
    'batchMatMul'   C[b][N, M]  = A[b][N, AK](:, :K) * B[b][K, M]          (K = B.shape[1])
    'batchMatMulT1' C[b][CN, M] = (A[b][K, AN](:, :CN))^T * B[b][K, M]     (CN = rows, default AN)
    'batchMatMulT2' C[b][N, CM](:, :BM) = A[b][N, K] * B[b][BM, K]^T       (CM = BM rounded up to 4)
    float loops by default; f64=True returns (C, S) in double with S = sum_k |a||b|."""
    v = _BMM_VARIANT[variant]
    A, pa = _f(A)
    B, pb = _f(B)
    Bt, N, M, K, p = _bmm_dims(A, B, v, None)
    if v == 1:
        N = p if rows is None else rows
    cm = p if v == 2 else M
    if f64:
        Cm, S = np.empty((Bt, N, cm), np.float64), np.empty((Bt, N, cm), np.float64)
        lib().oracle_bmm_f64(pa, pb, Cm.ctypes.data_as(_D), S.ctypes.data_as(_D), _i(Bt), _i(N), _i(M), _i(K), _i(p), _i(v), _i(threads))
        return Cm, S
    Cm = np.empty((Bt, N, cm), np.float32)
    lib().oracle_bmm(pa, pb, Cm.ctypes.data_as(_F), _i(Bt), _i(N), _i(M), _i(K), _i(p), _i(v))
    return Cm


def ref_batch_matmul(A, B, variant="batchMatMul", rows=None):
    """The reference project's own C++ loops bmm / bmmT1 / bmmT2 (Cuda_batchMatMul/test.cuh:95-140)."""
    v = _BMM_VARIANT[variant]
    A, pa = _f(A)
    B, pb = _f(B)
    Bt, N, M, K, p = _bmm_dims(A, B, v, None)
    if v == 1:
        N = p if rows is None else rows
    cm = p if v == 2 else M
    Cm = np.zeros((Bt, N, cm), np.float32)
    L = ref_lib()
    if v == 0:
        L.ref_bmm(pa, pb, Cm.ctypes.data_as(_F), _i(Bt), _i(N), _i(M), _i(K), _i(p))
    elif v == 1:
        L.ref_bmmT1(pa, pb, Cm.ctypes.data_as(_F), _i(Bt), _i(N), _i(p), _i(M), _i(K))
    else:
        L.ref_bmmT2(pa, pb, Cm.ctypes.data_as(_F), _i(Bt), _i(N), _i(cm), _i(M), _i(K))
    return Cm


_POOL_OP = {"max": 0, "max_indexed": 1, "avg": 2, "avg_ignore_padding": 3}
_I32 = C.POINTER(C.c_int)


def pool_out_hw(IH, IW, FH, FW, sh, sw, ph, pw):
    return (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1


def pool2D(X, FH, FW, sh, sw, ph, pw, op="max"):
    """Forward pooling of X[N, IH, IW, IC] (Cuda_pool2D/test.cuh:79-157 and the avg / indexed kernels beside it);
    'max_indexed' returns (Y, Index)."""
    X, px = _f(X)
    N, IH, IW, IC = X.shape
    OH, OW = pool_out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    Y = np.empty((N, OH, OW, IC), np.float32)
    Index = np.zeros((N, OH, OW, IC), np.int32)
    lib().oracle_pool2D(px, Y.ctypes.data_as(_F), Index.ctypes.data_as(_I32), _i(N), _i(IH), _i(IW), _i(IC), _i(FH), _i(FW),
                        _i(OH), _i(OW), _i(sh), _i(sw), _i(ph), _i(pw), _i(_POOL_OP[op]))
    return (Y, Index) if op == "max_indexed" else Y


def upool2D(deltaY, IH, IW, FH, FW, sh, sw, ph, pw, op="max", Y=None, X=None, Index=None):
    """Gradient of the pooling operators (Cuda_upool2D/test.cuh:90-229 and the avg / indexed kernels beside it)."""
    deltaY, pdy = _f(deltaY)
    N, OH, OW, IC = deltaY.shape
    dX = np.empty((N, IH, IW, IC), np.float32)
    null = C.cast(None, _F)
    py = px = null
    pidx = C.cast(None, _I32)
    if op == "max":
        Y, py = _f(Y)
        X, px = _f(X)
    if op == "max_indexed":
        Index = np.ascontiguousarray(Index, np.int32)
        pidx = Index.ctypes.data_as(_I32)
    lib().oracle_upool2D(pdy, py, px, pidx, dX.ctypes.data_as(_F), _i(N), _i(IH), _i(IW), _i(IC), _i(FH), _i(FW), _i(OH), _i(OW),
                         _i(sh), _i(sw), _i(ph), _i(pw), _i(_POOL_OP[op]))
    return dX


def ref_pool2D(X, FH, FW, sh, sw, ph, pw, op="max"):
    """The reference project's own C++ loops Pool2D_max_img2col / Pool2D_avg_img2col (the latter ignores padding)."""
    X, px = _f(X)
    N, IH, IW, IC = X.shape
    OH, OW = pool_out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    Y = np.empty((N, OH, OW, IC), np.float32)
    fn = {"max": ref_lib().ref_Pool2D_max, "avg_ignore_padding": ref_lib().ref_Pool2D_avg}[op]
    fn(px, _i(IH), _i(IW), _i(FH), _i(FW), Y.ctypes.data_as(_F), _i(OH), _i(OW), _i(N), _i(IC), _i(sh), _i(sw), _i(ph), _i(pw))
    return Y


def ref_upool2D(deltaY, IH, IW, FH, FW, sh, sw, ph, pw, op="max", Y=None, X=None):
    """The reference project's own C++ loops unpool2D_max_img2col_plus / unpooling_avg_img2col_plus (ignores padding)."""
    deltaY, pdy = _f(deltaY)
    N, OH, OW, IC = deltaY.shape
    dX = np.empty((N, IH, IW, IC), np.float32)
    if op == "max":
        Y, py = _f(Y)
        X, px = _f(X)
        ref_lib().ref_unpool2D_max(pdy, py, _i(OH), _i(OW), _i(FH), _i(FW), dX.ctypes.data_as(_F), px, _i(IH), _i(IW), _i(N), _i(IC),
                                   _i(sh), _i(sw), _i(ph), _i(pw))
    else:
        ref_lib().ref_unpool2D_avg(pdy, _i(OH), _i(OW), _i(FH), _i(FW), dX.ctypes.data_as(_F), _i(IH), _i(IW), _i(N), _i(IC),
                                   _i(sh), _i(sw), _i(ph), _i(pw))
    return dX
