"""Host-side mirror of the conv section of Dragon-Alpha's CudaFloat32EngineBase.

`CudaFloat32EngineBase` keeps the reference's address-level operator methods (same names, same
argument order, same option setters and the same IllegalArgument checks, raised as ValueError):
src/alpha_src/z/dragon/engine/cuda/CudaFloat32EngineBase.java:1322-2007.  `Engine` adds the
tensor-level calls with the shape inference of src/alpha_src/z/dragon/engine/Engine.java:1541-1829
and the pad-to-4 memory rule of src/alpha_src/z/dragon/engine/Tensor.java:208-221.

PyTorch only provides device memory and streams here; every contraction runs in
libalpha_conv_b200.so.  There is no CPU or PyTorch fallback: a missing library raises ImportError.
"""
import ctypes as C

import torch

from . import lib as _l


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


class CudaFloat32EngineBase:
    """Address-level operators.  Arguments are device addresses (ints) or torch CUDA tensors."""

    def __init__(self, stream=None, math=None, algo=None):
        """math ('3xtf32' / 'tf32') and algo ('auto' / 'tensor' / 'simt' / 'winograd') are this engine's own
        settings, passed with every call; None follows the process-wide default of lib.set_math_mode /
        lib.set_algo.  Two engines of one process may differ."""
        self._lib = _l.load()
        self._stream = stream
        self._math = -1 if math is None else {"3xtf32": _l.ALPHA_MATH_3XTF32, "tf32": _l.ALPHA_MATH_TF32}[math]
        self._algo = -1 if algo is None else {"auto": 0, "tensor": 1, "simt": 2, "winograd": 3}[algo]
        # Option flags of the reference.  There they choose among SIMT kernel families (texture loads,
        # remoded weights, the V2 tilings, split-K part counts); every family maps onto the same
        # tensor-core kernels here, so the setters below only store the value: they exist so that host
        # code written against the reference's engine runs unchanged, and nothing reads them.
        self._conv3D_useTexture = True
        self._conv3D_remode = True
        self._conv3D_remode_V2_Q = 1.05
        self._conv3D_V2_Q = 1.25
        self._dW_SplitKThreshold = 512
        self._dW_SK_MaxPartNum = 16
        self._dW_SK_V2_Q = 1.15
        self._dX_s1_useTexture = True
        self._dX_ks_useTexture = False
        self._dX_ks_V2_Q = 1.1
        self._dX_s1_V2_Q = 1.1

    # ---- fluent option setters (CudaFloat32EngineBase.java:1324-1352, 1630-1663, 1765-1793) ----
    def conv3D_useTexture(self, flag=None):
        if flag is None:
            return self._conv3D_useTexture
        self._conv3D_useTexture = bool(flag)
        return self

    def conv3D_remode(self, flag=None):
        if flag is None:
            return self._conv3D_remode
        self._conv3D_remode = bool(flag)
        return self

    def conv3D_remode_V2_Q(self, Q=None):
        if Q is None:
            return self._conv3D_remode_V2_Q
        if Q < 1.04999:
            raise ValueError("Q must >= 1.05")
        self._conv3D_remode_V2_Q = float(Q)
        return self

    def conv3D_V2_Q(self, Q=None):
        if Q is None:
            return self._conv3D_V2_Q
        if Q < 1.09999:
            raise ValueError("Q must >= 1.1")
        self._conv3D_V2_Q = float(Q)
        return self

    def dconv3D_deltaW_SplitKThreshold(self, threshold=None):
        if threshold is None:
            return self._dW_SplitKThreshold
        if threshold & (threshold - 1):
            raise ValueError("threshold must be a power of 2")
        if threshold < 256:
            raise ValueError("threshold must >= 256")
        self._dW_SplitKThreshold = int(threshold)
        return self

    def dconv3D_deltaW_SK_MaxPartNum(self, maxPartNum=None):
        if maxPartNum is None:
            return self._dW_SK_MaxPartNum
        if maxPartNum < 4:
            raise ValueError("maxPartNum must >= 4")
        self._dW_SK_MaxPartNum = int(maxPartNum)
        return self

    def dconv3DdeltaW_SK_V2_Q(self, Q=None):
        if Q is None:
            return self._dW_SK_V2_Q
        if Q < 1.1:
            raise ValueError("Q >= 1.1")
        self._dW_SK_V2_Q = float(Q)
        return self

    def dconv3D_deltaX_s1_useTexture(self, flag=None):
        if flag is None:
            return self._dX_s1_useTexture
        self._dX_s1_useTexture = bool(flag)
        return self

    def dconv3D_deltaX_ks_useTexture(self, flag=None):
        if flag is None:
            return self._dX_ks_useTexture
        self._dX_ks_useTexture = bool(flag)
        return self

    # ---- operators ------------------------------------------------------------------------------
    def _own_settings(self):
        return self._math >= 0 or self._algo >= 0

    @staticmethod
    def _addr(a):
        return C.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else C.c_void_p(int(a))

    def conv3D(self, Y_address, OH, OW, X_address, IH, IW, W_address, FH, FW, N, IC, OC, sh, sw, ph, pw):
        """CudaFloat32EngineBase.conv3D (:1355-1474)."""
        a = self._addr
        if self._own_settings():
            shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
            return _l.check(self._lib.alpha_conv3d_forward_ex(C.byref(shp), a(X_address), a(W_address), None, a(Y_address),
                                                              self._math, self._algo, _stream(self._stream)))
        _l.check(self._lib.alpha_engine_conv3D(a(Y_address), OH, OW, a(X_address), IH, IW, a(W_address),
                                               FH, FW, N, IC, OC, sh, sw, ph, pw, _stream(self._stream)))

    def conv3D_biased(self, Y_address, OH, OW, X_address, IH, IW, W_address, FH, FW, Bias_address, N, IC,
                      OC, sh, sw, ph, pw):
        """CudaFloat32EngineBase.conv3D_biased (:1478-1627); the bias add is fused in the epilogue."""
        a = self._addr
        if self._own_settings():
            shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
            return _l.check(self._lib.alpha_conv3d_forward_ex(C.byref(shp), a(X_address), a(W_address), a(Bias_address),
                                                              a(Y_address), self._math, self._algo, _stream(self._stream)))
        _l.check(self._lib.alpha_engine_conv3D_biased(a(Y_address), OH, OW, a(X_address), IH, IW,
                                                      a(W_address), FH, FW, a(Bias_address), N, IC, OC,
                                                      sh, sw, ph, pw, _stream(self._stream)))

    def dconv3D_deltaW(self, deltaW_address, FH, FW, X_address, IH, IW, deltaY_address, OH, OW, N, IC, OC,
                       sh, sw, ph, pw):
        """CudaFloat32EngineBase.dconv3D_deltaW (:1666-1762)."""
        a = self._addr
        if self._own_settings():
            shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
            return _l.check(self._lib.alpha_conv3d_deltaW_ex(C.byref(shp), a(X_address), a(deltaY_address), a(deltaW_address),
                                                             self._math, self._algo, _stream(self._stream)))
        _l.check(self._lib.alpha_engine_dconv3D_deltaW(a(deltaW_address), FH, FW, a(X_address), IH, IW,
                                                       a(deltaY_address), OH, OW, N, IC, OC, sh, sw, ph,
                                                       pw, _stream(self._stream)))

    def dconv3D_deltaX(self, deltaX_address, IH, IW, deltaY_address, OH, OW, W_address, FH, FW, N, IC, OC,
                       sh, sw, ph, pw):
        """CudaFloat32EngineBase.dconv3D_deltaX (:1796-2005)."""
        a = self._addr
        if self._own_settings():
            shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
            return _l.check(self._lib.alpha_conv3d_deltaX_ex(C.byref(shp), a(deltaY_address), a(W_address), a(deltaX_address),
                                                             self._math, self._algo, _stream(self._stream)))
        _l.check(self._lib.alpha_engine_dconv3D_deltaX(a(deltaX_address), IH, IW, a(deltaY_address), OH,
                                                       OW, a(W_address), FH, FW, N, IC, OC, sh, sw, ph,
                                                       pw, _stream(self._stream)))


    # ---- weight-side transforms in caller-owned memory --------------------------------------------------
    def prepare_weights(self, op, W_address, FH, FW, N, IH, IW, OH, OW, IC, OC, sh, sw, ph, pw, stream=None):
        """Enqueues the transform of W that `op` ('forward' / 'deltaX') needs for this layer on `stream` and returns
        the block (a torch uint8 tensor, or None when the operator needs none).  A training loop runs these for
        all layers on a side stream after the optimizer step; conv3D / dconv3D_deltaX then take the block through
        their `prepared` argument.  The caller orders prepare before use."""
        shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
        nbytes = _l.prepared_weights_bytes(shp, op)
        if nbytes == 0:
            return None
        W = W_address if isinstance(W_address, torch.Tensor) else None
        block = torch.empty(nbytes, dtype=torch.uint8, device=W.device if W is not None else "cuda")
        self.prepare_weights_into(block, op, W_address, FH, FW, N, IH, IW, OH, OW, IC, OC, sh, sw, ph, pw, stream)
        return block

    def prepare_weights_into(self, block, op, W_address, FH, FW, N, IH, IW, OH, OW, IC, OC, sh, sw, ph, pw, stream=None):
        shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
        _l.check(self._lib.alpha_conv_prepare_weights(C.byref(shp), _l.OPS[op], self._addr(W_address), self._addr(block),
                                                      block.numel(), _stream(stream if stream is not None else self._stream)))

    def conv3D_prepared(self, Y_address, OH, OW, X_address, IH, IW, W_address, FH, FW, N, IC, OC, sh, sw, ph, pw, prepared):
        a = self._addr
        shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
        _l.check(self._lib.alpha_conv3d_forward_prepared(C.byref(shp), a(X_address), a(W_address),
                                                         a(prepared) if prepared is not None else None,
                                                         prepared.numel() if prepared is not None else 0, None, a(Y_address),
                                                         _stream(self._stream)))

    def dconv3D_deltaX_prepared(self, deltaX_address, IH, IW, deltaY_address, OH, OW, W_address, FH, FW, N, IC, OC, sh, sw, ph, pw,
                                prepared):
        a = self._addr
        shp = _l.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
        _l.check(self._lib.alpha_conv3d_deltaX_prepared(C.byref(shp), a(deltaY_address), a(W_address),
                                                        a(prepared) if prepared is not None else None,
                                                        prepared.numel() if prepared is not None else 0, a(deltaX_address),
                                                        _stream(self._stream)))

    # ---- matrix products (CudaFloat32EngineBase.java:1129-1245) ---------------------------------------
    def _mm(self, fn, *args):
        if self._math >= 0:
            old = self._lib.alpha_conv_get_math_mode()
            _l.check(self._lib.alpha_conv_set_math_mode(self._math))
            try:
                _l.check(fn(*args))
            finally:
                self._lib.alpha_conv_set_math_mode(old)
        else:
            _l.check(fn(*args))

    def matMul(self, C_address, A_address, B_address, N, M, K):
        """C[N,M] = A[N,K] * B[K,M] (CudaFloat32EngineBase.matMul, :1129-1139)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_matMul, a(C_address), a(A_address), a(B_address), N, M, K, _stream(self._stream))

    def matMul_biased(self, C_address, A_address, B_address, N, M, K, Bias_address):
        """C = A * B + Bias per row (CudaFloat32EngineBase.matMul_biased, :1142-1168)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_matMul_biased, a(C_address), a(A_address), a(B_address), N, M, K, a(Bias_address),
                 _stream(self._stream))

    def matMulT1(self, C_address, A_address, B_address, N, M, K):
        """C[N,M] = A[K,N]^T * B[K,M] (CudaFloat32EngineBase.matMulT1, :1185-1230)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_matMulT1, a(C_address), a(A_address), a(B_address), N, M, K, _stream(self._stream))

    def matMulT2(self, C_address, A_address, B_address, N, M, K):
        """C[N,M] = A[N,K] * B[M,K]^T (CudaFloat32EngineBase.matMulT2, :1233-1245)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_matMulT2, a(C_address), a(A_address), a(B_address), N, M, K, _stream(self._stream))

    def batchMatMul(self, C_address, A_address, B_address, Batch, N, M, BK, AK):
        """C[b] = A[b][N, AK](:, :BK) * B[b][BK, M] (CudaFloat32EngineBase.batchMatMul, :1256-1272)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_batchMatMul, a(C_address), a(A_address), a(B_address), Batch, N, M, BK, AK,
                 _stream(self._stream))

    def batchMatMulT1(self, C_address, A_address, B_address, Batch, CN, AN, M, K):
        """C[b][CN, M] = (A[b][K, AN](:, :CN))^T * B[b][K, M] (CudaFloat32EngineBase.batchMatMulT1, :1277-1287)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_batchMatMulT1, a(C_address), a(A_address), a(B_address), Batch, CN, AN, M, K,
                 _stream(self._stream))

    def batchMatMulT2(self, C_address, A_address, B_address, Batch, N, CM, BM, K):
        """C[b][N, CM](:, :BM) = A[b][N, K] * B[b][BM, K]^T (CudaFloat32EngineBase.batchMatMulT2, :1298-1318)."""
        a = self._addr
        self._mm(self._lib.alpha_engine_batchMatMulT2, a(C_address), a(A_address), a(B_address), Batch, N, CM, BM, K,
                 _stream(self._stream))

    # ---- pooling, Java argument order (CudaFloat32EngineBase.java:2012-2215) ----
    def _pool(self, fn, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, *ptrs_and_flags):
        s = _l.AlphaPoolShape(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw)
        _l.check(fn(C.byref(s), *ptrs_and_flags, _stream(self._stream)))

    def pool2D_max(self, Y_address, OH, OW, X_address, IH, IW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_pool2D_max, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(X_address), a(Y_address))

    def pool2D_max_indexed(self, Y_address, Index_address, OH, OW, X_address, IH, IW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_pool2D_max_indexed, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(X_address), a(Y_address),
                   a(Index_address))

    def pool2D_avg(self, Y_address, OH, OW, X_address, IH, IW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_pool2D_avg, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(X_address), a(Y_address), 0)

    def pool2D_avg_ignore_padding(self, Y_address, OH, OW, X_address, IH, IW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_pool2D_avg, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(X_address), a(Y_address), 1)

    def upool2D_max(self, deltaX_address, X_address, IH, IW, deltaY_address, Y_address, OH, OW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_upool2D_max, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(deltaY_address), a(Y_address),
                   a(X_address), a(deltaX_address))

    def upool2D_max_Indexed(self, deltaX_address, IH, IW, deltaY_address, Index_address, OH, OW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_upool2D_max_indexed, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(deltaY_address),
                   a(Index_address), a(deltaX_address))

    def upool2D_avg(self, deltaX_address, IH, IW, deltaY_address, OH, OW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_upool2D_avg, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(deltaY_address), a(deltaX_address), 0)

    def upool2D_avg_ignore_padding(self, deltaX_address, IH, IW, deltaY_address, OH, OW, FH, FW, N, IC, sh, sw, ph, pw):
        a = self._addr
        self._pool(self._lib.alpha_upool2D_avg, N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, a(deltaY_address), a(deltaX_address), 1)


def _pad4(n):
    return (n + 3) & ~3


def _pad_last(t, c4):
    """Copy of t whose last dimension is zero-padded to c4 (Tensor.java:208-221 memory rule)."""
    if t.shape[-1] == c4:
        return t.contiguous()
    out = torch.zeros(t.shape[:-1] + (c4,), dtype=t.dtype, device=t.device)
    out[..., : t.shape[-1]] = t
    return out


def _pad_first(t, n4):
    if t.shape[0] == n4:
        return t
    out = torch.zeros((n4,) + t.shape[1:], dtype=t.dtype, device=t.device)
    out[: t.shape[0]] = t
    return out


class Engine:
    """Tensor-level conv operators (Engine.java:1541, 1601, 1697, 1788) on torch CUDA tensors.

    Tensors are NHWC float32.  Channel counts and the batch that are not multiples of 4 are padded
    with zero lanes exactly as Dragon-Alpha's Tensor memory layout does, and sliced back.
    """

    def __init__(self, base=None):
        self.base = base if base is not None else CudaFloat32EngineBase()

    @staticmethod
    def out_size(IH, IW, FH, FW, sh, sw, ph, pw):
        return (IH - FH + 2 * ph) // sh + 1, (IW - FW + 2 * pw) // sw + 1

    def conv3D(self, X, W, sh, sw, ph, pw, Bias=None):
        N, IH, IW, IC = X.shape
        OC, FH, FW, WIC = W.shape
        if WIC != IC:
            raise ValueError("W.IC=%d != X.IC=%d" % (WIC, IC))
        OH, OW = self.out_size(IH, IW, FH, FW, sh, sw, ph, pw)
        ic4, oc4 = _pad4(IC), _pad4(OC)
        Xp = _pad_last(X, ic4)
        Wp = _pad_first(_pad_last(W, ic4), oc4)
        Y = torch.empty((N, OH, OW, oc4), dtype=torch.float32, device=X.device)
        if Bias is None:
            self.base.conv3D(Y, OH, OW, Xp, IH, IW, Wp, FH, FW, N, ic4, oc4, sh, sw, ph, pw)
        else:
            Bp = _pad_last(Bias.reshape(1, -1), oc4).reshape(-1)
            self.base.conv3D_biased(Y, OH, OW, Xp, IH, IW, Wp, FH, FW, Bp, N, ic4, oc4, sh, sw, ph, pw)
        return Y if oc4 == OC else Y[..., :OC]

    def conv3D_biased(self, X, W, Bias, sh, sw, ph, pw):
        return self.conv3D(X, W, sh, sw, ph, pw, Bias=Bias)

    def conv3D_leakyRelu(self, X, W, Bias, k, sh, sw, ph, pw):
        """leakyRelu(conv3D(_biased)(X, W[, Bias]), k) with the activation in the kernel's epilogue: what a
        Conv3D unit followed by a LeakyRelu unit computes (Engine.leakyRelu, Cuda_function's
        leakyRelu2D); k = 0 is relu."""
        N, IH, IW, IC = X.shape
        OC, FH, FW, WIC = W.shape
        if WIC != IC:
            raise ValueError("W.IC=%d != X.IC=%d" % (WIC, IC))
        OH, OW = self.out_size(IH, IW, FH, FW, sh, sw, ph, pw)
        ic4, oc4 = _pad4(IC), _pad4(OC)
        Xp = _pad_last(X, ic4)
        Wp = _pad_first(_pad_last(W, ic4), oc4)
        Bp = None if Bias is None else _pad_last(Bias.reshape(1, -1), oc4).reshape(-1)
        Y = torch.empty((N, OH, OW, oc4), dtype=torch.float32, device=X.device)
        shape = _l.AlphaConvShape(N, IH, IW, ic4, oc4, FH, FW, OH, OW, sh, sw, ph, pw)
        a = self.base._addr
        _l.check(self.base._lib.alpha_conv3d_forward_leakyRelu(C.byref(shape), a(Xp), a(Wp), a(Bp) if Bp is not None else None,
                                                               float(k), a(Y), _stream(self.base._stream)))
        return Y if oc4 == OC else Y[..., :OC]

    def field_sum(self, X, row_length=-1):
        """Engine.field_sum(X, row_length) (Engine.java:6945): sums the rows of X seen as a matrix of
        `row_length` columns; Conv3D.__backward__ calls it on deltaY with OC for the bias gradient."""
        if row_length == -1:
            row_length = X.shape[-1]
        if X.shape[-1] != row_length:
            raise ValueError("field_sum: row_length must be the last dimension")
        oc4 = _pad4(row_length)
        Xp = _pad_last(X, oc4).contiguous()
        out = torch.empty((oc4,), dtype=torch.float32, device=X.device)
        rows = Xp.numel() // oc4
        _l.check(self.base._lib.alpha_conv_bias_grad(self.base._addr(Xp), rows, oc4, self.base._addr(out),
                                                     _stream(self.base._stream)))
        return out if oc4 == row_length else out[:row_length]

    def dconv3D_deltaW(self, X, deltaY, FH, FW, sh, sw, ph, pw):
        N, IH, IW, IC = X.shape
        _, OH, OW, OC = deltaY.shape
        ic4, oc4 = _pad4(IC), _pad4(OC)
        Xp, dYp = _pad_last(X, ic4), _pad_last(deltaY, oc4)
        dW = torch.empty((oc4, FH, FW, ic4), dtype=torch.float32, device=X.device)
        self.base.dconv3D_deltaW(dW, FH, FW, Xp, IH, IW, dYp, OH, OW, N, ic4, oc4, sh, sw, ph, pw)
        return dW if (ic4 == IC and oc4 == OC) else dW[:OC, :, :, :IC]

    def dconv3D_deltaW_bias(self, X, deltaY, FH, FW, sh, sw, ph, pw):
        """(deltaW, deltaB) of a biased Conv3D unit in one call: dconv3D_deltaW and field_sum(deltaY, OC) of
        Conv3D.__backward__ (nn/unit/simple/Conv3D.java:150-160); stride-1 layers sum the bias columns inside
        the deltaW kernel's pass over deltaY."""
        N, IH, IW, IC = X.shape
        _, OH, OW, OC = deltaY.shape
        ic4, oc4 = _pad4(IC), _pad4(OC)
        Xp, dYp = _pad_last(X, ic4), _pad_last(deltaY, oc4)
        dW = torch.empty((oc4, FH, FW, ic4), dtype=torch.float32, device=X.device)
        dB = torch.empty((oc4,), dtype=torch.float32, device=X.device)
        shape = _l.AlphaConvShape(N, IH, IW, ic4, oc4, FH, FW, OH, OW, sh, sw, ph, pw)
        a = self.base._addr
        _l.check(self.base._lib.alpha_conv3d_deltaW_bias(C.byref(shape), a(Xp), a(dYp), a(dW), a(dB), _stream(self.base._stream)))
        return (dW if (ic4 == IC and oc4 == OC) else dW[:OC, :, :, :IC]), (dB if oc4 == OC else dB[:OC])

    def dconv3D_deltaX(self, deltaY, W, IH, IW, sh, sw, ph, pw):
        N, OH, OW, OC = deltaY.shape
        _, FH, FW, IC = W.shape
        ic4, oc4 = _pad4(IC), _pad4(OC)
        dYp = _pad_last(deltaY, oc4)
        Wp = _pad_first(_pad_last(W, ic4), oc4)
        dX = torch.empty((N, IH, IW, ic4), dtype=torch.float32, device=deltaY.device)
        self.base.dconv3D_deltaX(dX, IH, IW, dYp, OH, OW, Wp, FH, FW, N, ic4, oc4, sh, sw, ph, pw)
        return dX if ic4 == IC else dX[..., :IC]

    # ---- matrix products (Engine.matMul / matMulT1 / matMulT2, Engine.java) -------------------------------
    @staticmethod
    def _pad2(t):
        r4, c4 = _pad4(t.shape[0]), _pad4(t.shape[1])
        if (r4, c4) == tuple(t.shape):
            return t.contiguous()
        out = torch.zeros((r4, c4), dtype=t.dtype, device=t.device)
        out[: t.shape[0], : t.shape[1]] = t
        return out

    def matMul(self, A, B, Bias=None):
        """C[N,M] = A[N,K] * B[K,M] (+ Bias[M] per row); dimensions are zero-padded to multiples of 4 as the
        engine's tensor memory is, and sliced back."""
        (N, K), (K2, M) = A.shape, B.shape
        if K != K2:
            raise ValueError("A.width=%d != B.height=%d" % (K, K2))
        Ap, Bp = self._pad2(A), self._pad2(B)
        C = torch.empty((Ap.shape[0], Bp.shape[1]), dtype=torch.float32, device=A.device)
        if Bias is None:
            self.base.matMul(C, Ap, Bp, Ap.shape[0], Bp.shape[1], Ap.shape[1])
        else:
            bp = _pad_last(Bias.reshape(1, -1), Bp.shape[1]).reshape(-1)
            self.base.matMul_biased(C, Ap, Bp, Ap.shape[0], Bp.shape[1], Ap.shape[1], bp)
        return C[:N, :M]

    def matMulT1(self, A, B):
        """C[N,M] = A[K,N]^T * B[K,M]."""
        (K, N), (K2, M) = A.shape, B.shape
        if K != K2:
            raise ValueError("A.height=%d != B.height=%d" % (K, K2))
        Ap, Bp = self._pad2(A), self._pad2(B)
        C = torch.empty((Ap.shape[1], Bp.shape[1]), dtype=torch.float32, device=A.device)
        self.base.matMulT1(C, Ap, Bp, Ap.shape[1], Bp.shape[1], Ap.shape[0])
        return C[:N, :M]

    def matMulT2(self, A, B):
        """C[N,M] = A[N,K] * B[M,K]^T."""
        (N, K), (M, K2) = A.shape, B.shape
        if K != K2:
            raise ValueError("A.width=%d != B.width=%d" % (K, K2))
        Ap, Bp = self._pad2(A), self._pad2(B)
        C = torch.empty((Ap.shape[0], Bp.shape[0]), dtype=torch.float32, device=A.device)
        self.base.matMulT2(C, Ap, Bp, Ap.shape[0], Bp.shape[0], Ap.shape[1])
        return C[:N, :M]

    # Batched products with the engine's memory rule (only the last dimension of a tensor is padded to a multiple
    # of 4) and EngineCore's argument mapping (EngineCore.java:579-623): the row pitch and the logical row length
    # go down separately.  The batch itself is not padded here (the reference rounds it up over zero matrices).
    def batchMatMul(self, A, B):
        """C[b] = A[b] * B[b]; A [Batch, N, K], B [Batch, K, M]."""
        (Bt, N, K), (Bt2, K2, M) = A.shape, B.shape
        if Bt != Bt2 or K != K2:
            raise ValueError("batchMatMul: A %s against B %s" % (tuple(A.shape), tuple(B.shape)))
        Ap, Bp = _pad_last(A, _pad4(K)), _pad_last(B, _pad4(M))
        C = torch.zeros((Bt, N, _pad4(M)), dtype=torch.float32, device=A.device)
        self.base.batchMatMul(C, Ap, Bp, Bt, N, _pad4(M), K, _pad4(K))
        return C[..., :M]

    def batchMatMulT1(self, A, B):
        """C[b] = A[b]^T * B[b]; A [Batch, K, N], B [Batch, K, M]."""
        (Bt, K, N), (Bt2, K2, M) = A.shape, B.shape
        if Bt != Bt2 or K != K2:
            raise ValueError("batchMatMulT1: A %s against B %s" % (tuple(A.shape), tuple(B.shape)))
        Ap, Bp = _pad_last(A, _pad4(N)), _pad_last(B, _pad4(M))
        C = torch.zeros((Bt, N, _pad4(M)), dtype=torch.float32, device=A.device)
        self.base.batchMatMulT1(C, Ap, Bp, Bt, N, _pad4(N), _pad4(M), K)
        return C[..., :M]

    def batchMatMulT2(self, A, B):
        """C[b] = A[b] * B[b]^T; A [Batch, N, K], B [Batch, M, K]."""
        (Bt, N, K), (Bt2, M, K2) = A.shape, B.shape
        if Bt != Bt2 or K != K2:
            raise ValueError("batchMatMulT2: A %s against B %s" % (tuple(A.shape), tuple(B.shape)))
        Ap, Bp = _pad_last(A, _pad4(K)), _pad_last(B, _pad4(K))
        C = torch.zeros((Bt, N, _pad4(M)), dtype=torch.float32, device=A.device)
        self.base.batchMatMulT2(C, Ap, Bp, Bt, N, _pad4(M), M, _pad4(K))
        return C[..., :M]

    # ---- 2D pooling (Engine.pool2D_max / pool2D_avg and their gradients; CudaFloat32EngineBase.java:2012-2215) ----
    def _pool_shape(self, X, FH, FW, sh, sw, ph, pw):
        N, IH, IW, IC = X.shape
        OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
        return _l.AlphaPoolShape(N, IH, IW, _pad4(IC), FH, FW, OH, OW, sh, sw, ph, pw), OH, OW

    def pool2D_max(self, X, FH, FW, sh, sw, ph, pw, indexed=False):
        """Y (and, with indexed=True, the int32 index tensor the indexed gradient reads)."""
        s, OH, OW = self._pool_shape(X, FH, FW, sh, sw, ph, pw)
        IC = X.shape[3]
        Xp = _pad_last(X, s.IC)
        Y = torch.empty((s.N, OH, OW, s.IC), dtype=torch.float32, device=X.device)
        if indexed:
            Index = torch.empty((s.N, OH, OW, s.IC), dtype=torch.int32, device=X.device)
            self.base.pool2D_max_indexed(Y, Index, OH, OW, Xp, s.IH, s.IW, FH, FW, s.N, s.IC, sh, sw, ph, pw)
            return (Y if s.IC == IC else Y[..., :IC]), Index
        self.base.pool2D_max(Y, OH, OW, Xp, s.IH, s.IW, FH, FW, s.N, s.IC, sh, sw, ph, pw)
        return Y if s.IC == IC else Y[..., :IC]

    def pool2D_avg(self, X, FH, FW, sh, sw, ph, pw, ignore_padding=False):
        s, OH, OW = self._pool_shape(X, FH, FW, sh, sw, ph, pw)
        IC = X.shape[3]
        Xp = _pad_last(X, s.IC)
        Y = torch.empty((s.N, OH, OW, s.IC), dtype=torch.float32, device=X.device)
        a = self.base._addr
        _l.check(self.base._lib.alpha_pool2D_avg(C.byref(s), a(Xp), a(Y), int(bool(ignore_padding)), _stream(self.base._stream)))
        return Y if s.IC == IC else Y[..., :IC]

    def upool2D_max(self, deltaY, Y, X, FH, FW, sh, sw, ph, pw):
        """deltaX of pool2D_max from X and Y of the forward pass."""
        s, OH, OW = self._pool_shape(X, FH, FW, sh, sw, ph, pw)
        IC = X.shape[3]
        Xp, Yp, dYp = _pad_last(X, s.IC), _pad_last(Y, s.IC), _pad_last(deltaY, s.IC)
        dX = torch.empty_like(Xp)
        a = self.base._addr
        _l.check(self.base._lib.alpha_upool2D_max(C.byref(s), a(dYp), a(Yp), a(Xp), a(dX), _stream(self.base._stream)))
        return dX if s.IC == IC else dX[..., :IC]

    def upool2D_max_indexed(self, deltaY, Index, IH, IW, FH, FW, sh, sw, ph, pw):
        """deltaX of pool2D_max from the index tensor of the forward pass (its channel count is the padded one)."""
        N, OH, OW, IC = deltaY.shape
        ic4 = Index.shape[3]
        s = _l.AlphaPoolShape(N, IH, IW, ic4, FH, FW, OH, OW, sh, sw, ph, pw)
        dYp = _pad_last(deltaY, ic4)
        dX = torch.empty((N, IH, IW, ic4), dtype=torch.float32, device=deltaY.device)
        a = self.base._addr
        _l.check(self.base._lib.alpha_upool2D_max_indexed(C.byref(s), a(dYp), a(Index), a(dX), _stream(self.base._stream)))
        return dX if ic4 == IC else dX[..., :IC]

    def upool2D_avg(self, deltaY, IH, IW, FH, FW, sh, sw, ph, pw, ignore_padding=False):
        N, OH, OW, IC = deltaY.shape
        ic4 = _pad4(IC)
        s = _l.AlphaPoolShape(N, IH, IW, ic4, FH, FW, OH, OW, sh, sw, ph, pw)
        dYp = _pad_last(deltaY, ic4)
        dX = torch.empty((N, IH, IW, ic4), dtype=torch.float32, device=deltaY.device)
        a = self.base._addr
        _l.check(self.base._lib.alpha_upool2D_avg(C.byref(s), a(dYp), a(dX), int(bool(ignore_padding)), _stream(self.base._stream)))
        return dX if ic4 == IC else dX[..., :IC]

    def dconv3D(self, X, W, sh, sw, ph, pw, OH=None, OW=None):
        """Deconv3D forward = dconv3D_deltaX with the roles of input and output swapped
        (Engine.java:1819-1829); W is [IC_in, FH, FW, OC_out]."""
        N, IH, IW, _ = X.shape
        _, FH, FW, _ = W.shape
        if OH is None:
            OH = (IH - 1) * sh + FH - 2 * ph
        if OW is None:
            OW = (IW - 1) * sw + FW - 2 * pw
        return self.dconv3D_deltaX(X, W, OH, OW, sh, sw, ph, pw)
