"""GPU test of alpha_conv3d_deltaW_noalloc, the deltaW entry point for callers that cannot allocate.

A host that has given all device memory to its own pool (Dragon-Alpha's engine does), or that calls
from code where the CUDA allocator must not be entered, cannot let a native call cudaMalloc.  This
entry point keeps its split-K partial sums in a fixed 32 MiB array inside the library instead.  The
test calls it through the C ABI twice in a row - the second call finds the first call's partials
still in the array - and compares each result with alpha_conv3d_deltaW on the same input; it also
checks that a shape whose partials do not fit is refused with a clear message.

The file name sorts last so that a run that stops at the first failure has already run every other
test; the test does not depend on any of them having run.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _shape(L, N, HW, IC, OC):
    return L.AlphaConvShape(N, HW, HW, IC, OC, 3, 3, HW, HW, 1, 1, 1, 1)


def test_deltaW_noalloc_matches_deltaW_on_two_calls(pkg):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    L = pkg.submodule("lib")
    lib = L.load()
    lib.alpha_conv3d_deltaW_noalloc.argtypes = [C.POINTER(L.AlphaConvShape)] + [C.c_void_p] * 4
    lib.alpha_conv3d_deltaW_noalloc_capacity.restype = C.c_size_t
    assert lib.alpha_conv3d_deltaW_noalloc_capacity() == 32 << 20
    L.set_math_mode("3xtf32")
    L.set_algo("auto")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(5)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # two different layers back to back: the second call runs over the first call's leftovers
    for (N, HW, IC, OC) in [(32, 28, 64, 64), (16, 14, 128, 96)]:
        X = torch.randn((N, HW, HW, IC), device=dev, generator=gen).relu_()
        dY = torch.randn((N, HW, HW, OC), device=dev, generator=gen)
        ref = torch.empty((OC, 3, 3, IC), device=dev)
        got = torch.full((OC, 3, 3, IC), float("nan"), device=dev)
        s = _shape(L, N, HW, IC, OC)
        p = lambda t: C.c_void_p(t.data_ptr())
        L.check(lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(ref), stream))
        assert L.last_algo().startswith("dw")
        L.check(lib.alpha_conv3d_deltaW_noalloc(C.byref(s), p(X), p(dY), p(got), stream))
        assert L.last_algo() == "dw_noalloc"
        assert lib.alpha_conv3d_deltaW_noalloc_status() == 0
        assert L.device_status() == 0
        a, b = got.cpu().numpy(), ref.cpu().numpy()
        assert np.isfinite(a).all()
        # the tolerance of the parity tests (normwise 1e-4); the two entry points may tile and order
        # the pixel sum differently
        assert np.abs(a - b).max() <= 1e-4 * np.abs(b).max()
        # and against the fp64 result, independent of the other entry point
        d64 = torch.einsum("nhwc,nhwo->oc", X.double(), dY.double())  # centre tap only
        centre = torch.from_numpy(a[:, 1, 1, :]).double().to(dev)
        assert float((centre - d64).abs().max()) <= 1e-4 * float(d64.abs().max())


def test_deltaW_noalloc_rejects_what_does_not_fit(pkg):
    import torch
    torch.cuda.set_device(0)
    L = pkg.submodule("lib")
    lib = L.load()
    lib.alpha_conv3d_deltaW_noalloc.argtypes = [C.POINTER(L.AlphaConvShape)] + [C.c_void_p] * 4
    L.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    # 3x3, 256 -> 256 channels on 14x14 images: 16 partials of 589824 floats = 36 MiB > 32 MiB
    N, HW, IC, OC = 64, 14, 256, 256
    X = torch.zeros((N, HW, HW, IC), device=dev)
    dY = torch.zeros((N, HW, HW, OC), device=dev)
    dW = torch.zeros((OC, 3, 3, IC), device=dev)
    s = _shape(L, N, HW, IC, OC)
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = lib.alpha_conv3d_deltaW_noalloc(C.byref(s), p(X), p(dY), p(dW), None)
    assert rc == -5
    assert "fixed scratch" in L.last_error()
    # a channel count the tensor-core kernel does not take is refused as an argument error
    s = _shape(L, 4, 8, 16, 32)
    rc = lib.alpha_conv3d_deltaW_noalloc(C.byref(s), p(X), p(dY), p(dW), None)
    assert rc == -1
