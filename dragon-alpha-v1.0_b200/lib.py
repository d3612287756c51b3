"""ctypes binding of libalpha_conv_b200.so (the C ABI declared in include/alpha_conv_b200.h)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libalpha_conv_b200.so")

ALPHA_MATH_3XTF32, ALPHA_MATH_TF32 = 0, 1
ALPHA_ALGO_AUTO, ALPHA_ALGO_TENSOR, ALPHA_ALGO_SIMT, ALPHA_ALGO_WINOGRAD = 0, 1, 2, 3


class AlphaConvShape(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("N", "IH", "IW", "IC", "OC", "FH", "FW", "OH", "OW", "sh", "sw", "ph", "pw")]


class AlphaPoolShape(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("N", "IH", "IW", "IC", "FH", "FW", "OH", "OW", "sh", "sw", "ph", "pw")]


class AlphaConvError(RuntimeError):
    """A call into the library returned a non-zero status; .code holds the ALPHA_E_* value."""

    def __init__(self, code, message):
        super().__init__("alpha_conv_b200 error %d: %s" % (code, message))
        self.code = code


_lib = None


def load():
    """Loads the shared library; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: run __graft_entry__.build() (nvcc, sm_100a) first" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    lib.alpha_conv_last_error.restype = C.c_char_p
    lib.alpha_conv_last_algo.restype = C.c_char_p
    lib.alpha_conv_last_plan.restype = C.c_char_p
    lib.alpha_conv_launch_count.restype = C.c_ulonglong
    P, V, I, L = C.POINTER(AlphaConvShape), C.c_void_p, C.c_int, C.c_int64
    lib.alpha_conv3d_forward.argtypes = [P, V, V, V, V, V]
    lib.alpha_conv3d_deltaX.argtypes = [P, V, V, V, V]
    lib.alpha_conv3d_forward_leakyRelu.argtypes = [P, V, V, V, C.c_float, V, V]
    lib.alpha_conv3d_deltaW.argtypes = [P, V, V, V, V]
    lib.alpha_conv_bias_grad.argtypes = [V, C.c_longlong, I, V, V]
    lib.alpha_conv3d_deltaW_bias.argtypes = [P, V, V, V, V, V]
    lib.alpha_conv3d_forward_ex.argtypes = [P, V, V, V, V, I, I, V]
    lib.alpha_conv3d_deltaX_ex.argtypes = [P, V, V, V, I, I, V]
    lib.alpha_conv3d_deltaW_ex.argtypes = [P, V, V, V, I, I, V]
    lib.alpha_conv3d_deltaW_noalloc.argtypes = [P, V, V, V, V]
    lib.alpha_conv3d_deltaW_noalloc_capacity.restype = C.c_size_t
    lib.alpha_conv_set_option.argtypes = [C.c_char_p, I]
    lib.alpha_conv_get_option.argtypes = [C.c_char_p, C.POINTER(I)]
    lib.alpha_conv_workspace_bytes.argtypes = [P, I, C.POINTER(C.c_size_t)]
    lib.alpha_conv_set_workspace.argtypes = [V, V, C.c_size_t]
    lib.alpha_conv_reserve_workspace.argtypes = [V, C.c_size_t]
    lib.alpha_conv_workspace_in_use.restype = C.c_size_t
    lib.alpha_conv_prepared_weights_bytes.argtypes = [P, I, C.POINTER(C.c_size_t)]
    lib.alpha_conv_prepare_weights.argtypes = [P, I, V, V, C.c_size_t, V]
    lib.alpha_conv3d_forward_prepared.argtypes = [P, V, V, V, C.c_size_t, V, V, V]
    lib.alpha_conv3d_deltaX_prepared.argtypes = [P, V, V, V, C.c_size_t, V, V]
    lib.alpha_conv_weight_cache.argtypes = [I]
    lib.alpha_conv_weights_updated.argtypes = [V]
    lib.alpha_engine_conv3D.argtypes = [V, I, I, V, I, I, V, I, I] + [I] * 7 + [V]
    lib.alpha_engine_conv3D_biased.argtypes = [V, I, I, V, I, I, V, I, I, V] + [I] * 7 + [V]
    lib.alpha_engine_dconv3D_deltaW.argtypes = [V, I, I, V, I, I, V, I, I] + [I] * 7 + [V]
    lib.alpha_engine_dconv3D_deltaX.argtypes = [V, I, I, V, I, I, V, I, I] + [I] * 7 + [V]
    SA = C.POINTER(C.c_int64)
    # Cuda_conv3D natives
    conv = [SA, I, V, I, I, V, I, I, V, I, I] + [I] * 7
    lib.alpha_Cuda_conv3D_conv3D.argtypes = conv
    lib.alpha_Cuda_conv3D_conv3D_texture.argtypes = conv
    lib.alpha_Cuda_conv3D_conv3DV2.argtypes = [I] + conv
    lib.alpha_Cuda_conv3D_conv3D_np.argtypes = [SA, I, V, I, I, V, I, I, V, I, I] + [I] * 5
    lib.alpha_Cuda_conv3D_conv3D_W1.argtypes = [SA, I, V, I, I, V, V, I, I, I]
    lib.alpha_Cuda_conv3D_kernel_remode.argtypes = [L, V, V, I, I, I, I]
    convR = [SA, I, V, I, I, V, V, I, I, V, I, I] + [I] * 7
    lib.alpha_Cuda_conv3D_conv3D_GemmR.argtypes = convR
    lib.alpha_Cuda_conv3D_conv3D_GemmR_texture.argtypes = convR
    lib.alpha_Cuda_conv3D_conv3D_GemmV2R.argtypes = [I] + convR
    lib.alpha_Cuda_conv3D_conv3D_GemmR_W1.argtypes = [SA, I, V, I, I, V, V, V, I, I, I]
    # Cuda_dconv3D_deltaX natives
    dxs1 = [SA, I, V, I, I, V, I, I, V, I, I] + [I] * 5
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1.argtypes = dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1_texture.argtypes = dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_V2_s1.argtypes = [I] + dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_W1.argtypes = [SA, I, V, V, V, I, I, I, I, I]
    rem = [L, V, I, I, V, I, I, I, I, I, I]
    lib.alpha_Cuda_dconv3D_deltaX_ks_remode.argtypes = rem
    lib.alpha_Cuda_dconv3D_deltaX_ks_remodev2.argtypes = rem
    dxks = [SA, I, V, I, I, V, I, I, V, I, I] + [I] * 7
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_kernelSplit.argtypes = dxks
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR.argtypes = dxks
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR_texture.argtypes = dxks
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R.argtypes = dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R_texture.argtypes = dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksV2_Ims2R.argtypes = [I] + dxs1
    lib.alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_crossAdd.argtypes = dxks
    # Cuda_dconv3D_deltaW natives
    lib.alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW.argtypes = [SA, I, V, I, I, V, I, I, V, I, I] + [I] * 7
    lib.alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_W1.argtypes = [SA, I, V, I, I, V, V, I, I, I]
    lib.alpha_Cuda_dconv3D_deltaW_buf_summary.argtypes = [L, V, V, I, I]
    sk = [SA, I, I, V, I, I, V, I, I, V, V, I, I] + [I] * 7
    lib.alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK.argtypes = sk
    lib.alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmV2SK.argtypes = sk
    lib.alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK_W1.argtypes = [SA, I, I, V, I, I, V, V, V, I, I, I]
    # matrix products
    lib.alpha_matMul.argtypes = [V, V, V, V, I, I, I, V]
    lib.alpha_matMulT1.argtypes = [V, V, V, I, I, I, V]
    lib.alpha_matMulT2.argtypes = [V, V, V, V, I, I, I, V]
    lib.alpha_engine_matMul.argtypes = [V, V, V, I, I, I, V]
    lib.alpha_engine_matMul_biased.argtypes = [V, V, V, I, I, I, V, V]
    lib.alpha_engine_matMulT1.argtypes = [V, V, V, I, I, I, V]
    lib.alpha_engine_matMulT2.argtypes = [V, V, V, I, I, I, V]
    mm = [SA, I, V, V, V, I, I, I]
    lib.alpha_Cuda_matMul_matMul.argtypes = mm
    lib.alpha_Cuda_matMul_matMulT1.argtypes = mm
    lib.alpha_Cuda_matMul_matMulT2.argtypes = mm
    lib.alpha_Cuda_matMul_matMulT1SK.argtypes = [SA, I, I, V, V, V, V, I, I, I]
    lib.alpha_Cuda_matMul_SKbuf_summary.argtypes = [L, V, V, I, I]
    # batched matrix products: (A, B, C, Batch, 4 dimensions, stream) / engine order (C, A, B, ...) / natives
    for name in ("alpha_batchMatMul", "alpha_batchMatMulT1", "alpha_batchMatMulT2",
                 "alpha_engine_batchMatMul", "alpha_engine_batchMatMulT1", "alpha_engine_batchMatMulT2"):
        getattr(lib, name).argtypes = [V, V, V, I, I, I, I, I, V]
    for name in ("batchMatMul", "batchMatMul_texture", "batchMatMulT1", "batchMatMulT2", "batchMatMulT2_texture"):
        getattr(lib, "alpha_Cuda_batchMatMul_" + name).argtypes = [SA, I, V, V, V, I, I, I, I, I]
    # pooling
    PS = C.POINTER(AlphaPoolShape)
    lib.alpha_pool2D_max.argtypes = [PS, V, V, V]
    lib.alpha_pool2D_max_indexed.argtypes = [PS, V, V, V, V]
    lib.alpha_pool2D_avg.argtypes = [PS, V, V, I, V]
    lib.alpha_upool2D_max.argtypes = [PS, V, V, V, V, V]
    lib.alpha_upool2D_max_indexed.argtypes = [PS, V, V, V, V]
    lib.alpha_upool2D_avg.argtypes = [PS, V, V, I, V]
    fwd = [SA, I, V, I, I, I, I, V, I, I, I, I, I, I, I, I]
    lib.alpha_Cuda_pool2D_pool2D_max.argtypes = fwd
    lib.alpha_Cuda_pool2D_pool2D_avg.argtypes = fwd
    lib.alpha_Cuda_pool2D_pool2D_avg_ignore_padding.argtypes = fwd
    lib.alpha_Cuda_pool2D_pool2D_max_indexed.argtypes = [SA, I, V, I, I, I, I, V, V, I, I, I, I, I, I, I, I]
    lib.alpha_Cuda_upool2D_upool2D_max.argtypes = [SA, I, V, V, I, I, I, I, V, V, I, I, I, I, I, I, I, I]
    lib.alpha_Cuda_upool2D_upool2D_max_Indexed.argtypes = [SA, I, V, V, I, I, I, I, V, I, I, I, I, I, I, I, I]
    for name in ("avg", "avg_tiled", "avg_ignore_padding", "avg_ignore_padding_tiled"):
        getattr(lib, "alpha_Cuda_upool2D_upool2D_" + name).argtypes = [SA, I, V, I, I, I, I, V, I, I, I, I, I, I, I, I]
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        raise AlphaConvError(rc, load().alpha_conv_last_error().decode("utf-8", "replace"))


def last_error():
    return load().alpha_conv_last_error().decode("utf-8", "replace")


def last_algo():
    return load().alpha_conv_last_algo().decode()


def last_plan():
    return load().alpha_conv_last_plan().decode()


def launch_count():
    return int(load().alpha_conv_launch_count())


def set_math_mode(mode):
    """mode: '3xtf32' (default, fp32-faithful) or 'tf32'."""
    m = {"3xtf32": ALPHA_MATH_3XTF32, "tf32": ALPHA_MATH_TF32}.get(mode, mode)
    check(load().alpha_conv_set_math_mode(int(m)))


def set_algo(algo):
    a = {"auto": 0, "tensor": 1, "simt": 2, "winograd": 3}.get(algo, algo)
    check(load().alpha_conv_set_algo(int(a)))


OPS = {"forward": 0, "deltaX": 1, "deltaW": 2, "bias_grad": 3}
_OPTION_WORDS = {"auto": 0, "im2col": 1, "halo": 2, "split": 1}


def set_option(name, value):
    """Sets one tuning switch of the tile planners (alpha_conv_set_option); returns the old value."""
    old = get_option(name)
    check(load().alpha_conv_set_option(name.encode(), int(_OPTION_WORDS.get(value, value))))
    return old


def get_option(name):
    v = C.c_int(0)
    check(load().alpha_conv_get_option(name.encode(), C.byref(v)))
    return v.value


def workspace_bytes(shape, op):
    """Scratch bytes one call of `op` ('forward', 'deltaX', 'deltaW', 'bias_grad') on `shape` needs."""
    n = C.c_size_t(0)
    check(load().alpha_conv_workspace_bytes(C.byref(shape), OPS[op], C.byref(n)))
    return n.value


def set_workspace(stream, ptr, nbytes):
    check(load().alpha_conv_set_workspace(C.c_void_p(stream), C.c_void_p(ptr) if ptr else None, nbytes))


def reserve_workspace(stream, nbytes):
    check(load().alpha_conv_reserve_workspace(C.c_void_p(stream), nbytes))


def release_workspace():
    check(load().alpha_conv_release_workspace())


def workspace_in_use():
    return int(load().alpha_conv_workspace_in_use())


def prepared_weights_bytes(shape, op):
    """Bytes of the weight-side transform `op` ('forward' or 'deltaX') needs for `shape` (0 = none)."""
    n = C.c_size_t(0)
    check(load().alpha_conv_prepared_weights_bytes(C.byref(shape), OPS[op], C.byref(n)))
    return n.value


def weight_cache(enable):
    check(load().alpha_conv_weight_cache(1 if enable else 0))


def weights_updated(W=None):
    """Tells the weight cache that tensor W (a device address; None = every tensor) has new values."""
    check(load().alpha_conv_weights_updated(C.c_void_p(W) if W else None))


def device_status():
    """Synchronises the device and returns its kernel status word (0 = clean)."""
    return int(load().alpha_conv_device_status())
