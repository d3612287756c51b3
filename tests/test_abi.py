"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol the
public headers declare, validates arguments before touching a device, and the JNI entry points
drive a JNIEnv function table the way the specification lays it out."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")


@pytest.fixture(scope="module")
def lib(pkg):
    pkg.submodule("build").build()
    return pkg.submodule("lib").load()


def _declared_symbols():
    names = set()
    for fn in sorted(os.listdir(INCLUDE)):
        text = open(os.path.join(INCLUDE, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(alpha_(?:conv|Cuda|engine|matMul|batchMatMul|pool2D|upool2D)\w*)\s*\(", text))
        names.update(re.findall(r"\b(Java_z_dragon_\w+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    # 29 natives of the three convolution classes + 5 of Cuda_matMul + 5 of Cuda_batchMatMul + 4 of Cuda_pool2D + 6 of Cuda_upool2D
    assert len([n for n in names if n.startswith("Java_")]) == 49
    assert len([n for n in names if n.startswith("alpha_Cuda_")]) == 49
    assert len([n for n in names if n.startswith(("alpha_pool2D", "alpha_upool2D"))]) == 6
    assert len([n for n in names if n.startswith("alpha_matMul")]) == 3
    assert len([n for n in names if n.startswith("alpha_batchMatMul")]) == 3
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_argument_errors_come_before_any_device_work(lib, pkg):
    L = pkg.submodule("lib")
    s = L.AlphaConvShape(4, 8, 8, 6, 8, 3, 3, 8, 8, 1, 1, 1, 1)  # IC = 6 is not a multiple of 4
    rc = lib.alpha_conv3d_forward(C.byref(s), 16, 32, None, 48, None)
    assert rc == -1 and b"multiples of 4" in lib.alpha_conv_last_error()
    s = L.AlphaConvShape(4, 8, 8, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1)
    assert lib.alpha_conv3d_forward(C.byref(s), None, 32, None, 48, None) == -1  # null X
    assert lib.alpha_conv3d_forward(C.byref(s), 20, 32, None, 48, None) == -1  # misaligned X
    s = L.AlphaConvShape(4, 8, 8, 8, 8, 3, 3, 9, 9, 1, 1, 1, 1)  # OH/OW too large for IH/IW
    assert lib.alpha_conv3d_deltaW(C.byref(s), 16, 32, 48, None) == -1
    assert lib.alpha_conv_set_math_mode(7) == -1
    assert lib.alpha_Cuda_dconv3D_deltaW_buf_summary(0, None, None, 3, 64) == -1
    # the bias gradient and the fused-activation forward check their arguments the same way
    assert lib.alpha_conv_bias_grad(None, 16, 8, 32, None) == -1          # null deltaY
    assert lib.alpha_conv_bias_grad(16, 16, 6, 32, None) == -1            # OC not a multiple of 4
    assert lib.alpha_conv_bias_grad(16, 0, 8, 32, None) == -1             # no rows
    assert lib.alpha_conv_bias_grad(20, 16, 8, 32, None) == -1            # misaligned
    s = L.AlphaConvShape(4, 8, 8, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1)
    assert lib.alpha_conv3d_forward_leakyRelu(C.byref(s), None, 32, None, 0.1, 48, None) == -1
    assert lib.alpha_conv3d_forward_leakyRelu(C.byref(s), 16, 32, None, float("nan"), 48, None) == -1


def test_options_and_per_call_settings_need_no_device(lib, pkg):
    """The tuning table is seeded from the environment once and changed by name afterwards; unknown names
    and out-of-range per-call settings are argument errors."""
    L = pkg.submodule("lib")
    old = L.set_option("HALO_PAIR", 3)
    assert L.get_option("ALPHA_HALO_PAIR") == 3       # the environment variable's name is accepted too
    L.set_option("HALO_PAIR", old)
    assert L.get_option("HALO_PAIR") == old
    assert L.set_option("CONV_TILE", "im2col") in (0, 1, 2) and L.get_option("CONV_TILE") == 1
    L.set_option("CONV_TILE", "auto")
    assert lib.alpha_conv_set_option(b"NO_SUCH_SWITCH", 1) == -1 and b"unknown option" in lib.alpha_conv_last_error()
    s = L.AlphaConvShape(4, 8, 8, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1)
    assert lib.alpha_conv3d_forward_ex(C.byref(s), 16, 32, None, 48, 2, -1, None) == -1      # math mode 2 does not exist
    assert lib.alpha_conv3d_deltaX_ex(C.byref(s), 16, 32, 48, -1, 9, None) == -1             # nor algo 9
    assert lib.alpha_conv3d_deltaW_ex(C.byref(s), None, 32, 48, -1, -1, None) == -1          # null X, default settings
    assert lib.alpha_matMul(None, 16, None, 32, 8, 8, 8, None) == -1 and b"null" in lib.alpha_conv_last_error()
    assert lib.alpha_matMulT1(16, 32, 48, 8, 0, 8, None) == -1                               # M = 0
    assert lib.alpha_matMulT2(16, 32, None, 48, 8, 8, 6, None) == -1                         # K = 6: not a multiple of 4
    assert lib.alpha_batchMatMul(16, 32, 48, 2, 8, 8, 8, 4, None) == -1 and b"row pitch" in lib.alpha_conv_last_error()
    assert lib.alpha_batchMatMulT2(16, 32, 48, 0, 8, 8, 8, 8, None) == -1                    # empty batch
    assert lib.alpha_Cuda_matMul_SKbuf_summary(0, None, None, 3, 64) == -1
    n = C.c_size_t(0)
    assert lib.alpha_conv_workspace_bytes(C.byref(s), 17, C.byref(n)) == -1                  # unknown op
    assert lib.alpha_conv_workspace_bytes(None, 0, C.byref(n)) == -1


def test_no_silent_fallback_without_a_gpu(lib, pkg):
    """On a machine without a B200 a well-formed call fails loudly; there is no CPU path."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = pkg.submodule("lib")
    s = L.AlphaConvShape(4, 8, 8, 8, 8, 3, 3, 8, 8, 1, 1, 1, 1)
    rc = lib.alpha_conv3d_forward(C.byref(s), 16, 32, None, 48, None)
    assert rc in (-2, -3)
    assert lib.alpha_conv_bias_grad(16, 16, 8, 32, None) in (-2, -3)
    assert lib.alpha_conv3d_forward_leakyRelu(C.byref(s), 16, 32, None, 0.1, 48, None) in (-2, -3)
    with pytest.raises(L.AlphaConvError):
        L.check(rc)


def test_jni_entry_points_use_the_jnienv_table(lib):
    """A fake JNIEnv with functions at the specification's slots (FindClass 6, ThrowNew 14,
    GetLongArrayRegion 204, ExceptionCheck 228): the shim must fetch the stream array through it and
    turn a failed call into a pending z.dragon.engine.cuda.impl.CudaException."""
    log = {}
    FINDCLASS = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p)
    THROWNEW = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_char_p)
    GETREGION = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64))
    EXCCHECK = C.CFUNCTYPE(C.c_uint8, C.c_void_p)

    def find_class(env, name):
        log["class"] = name
        return 0x1234

    def throw_new(env, cls, msg):
        log["thrown"] = (cls, msg)
        return 0

    def get_region(env, arr, start, n, buf):
        log["region"] = (arr, start, n)
        for i in range(n):
            buf[i] = 0
    cbs = [FINDCLASS(find_class), THROWNEW(throw_new), GETREGION(get_region), EXCCHECK(lambda env: 0)]
    table = (C.c_void_p * 235)()
    for slot, cb in zip((6, 14, 204, 228), cbs):
        table[slot] = C.cast(cb, C.c_void_p)
    env = C.pointer(C.c_void_p(C.addressof(table)))  # JNIEnv*: pointer to {const table*}

    f = lib.Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR
    f.restype = None
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int64,
                  C.c_int, C.c_int, C.c_int64] + [C.c_int] * 9
    # null tensor addresses: the call must fail in the argument check, on any machine
    f(env, None, 0xABCD, 2, 0, 8, 8, 0, 0, 3, 3, 0, 8, 8, 4, 8, 8, 1, 1, 1, 1)
    assert log["region"] == (0xABCD, 0, 2)
    assert log["class"] == b"z/dragon/engine/cuda/impl/CudaException"
    assert log["thrown"][0] == 0x1234 and b"null" in log["thrown"][1]
