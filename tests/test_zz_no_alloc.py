"""GPU test of alpha_conv3d_deltaW_noalloc, the deltaW entry point for callers that cannot allocate.

A host that has given all device memory to its own pool (Dragon-Alpha's engine does), or that calls
from code where the CUDA allocator must not be entered, cannot let a native call cudaMalloc.  This
entry point keeps its split-K partial sums in a fixed 32 MiB array inside the library instead.  The
test calls it through the C ABI twice in a row - the second call finds the first call's partials
still in the array - and compares each result with alpha_conv3d_deltaW on the same input (to
rounding against its default kernel, bit for bit against the same split-K kernel); it checks that
the free device memory does not move across a call, and that a shape whose partials do not fit is
refused with a clear message.

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
    assert lib.alpha_conv3d_deltaW_noalloc_capacity() == 32 << 20
    L.set_math_mode("3xtf32")
    L.set_algo("auto")
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(5)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # two different layers back to back: the second call runs over the first call's leftovers
    calls = 0
    for (N, HW, IC, OC) in [(32, 28, 64, 64), (16, 14, 128, 96)]:
        X = torch.randn((N, HW, HW, IC), device=dev, generator=gen).relu_()
        dY = torch.randn((N, HW, HW, OC), device=dev, generator=gen)
        ref = torch.empty((OC, 3, 3, IC), device=dev)
        got = torch.full((OC, 3, 3, IC), float("nan"), device=dev)
        s = _shape(L, N, HW, IC, OC)
        p = lambda t: C.c_void_p(t.data_ptr())
        L.check(lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(ref), stream))
        assert L.last_algo().startswith("dw")
        # the same split-K im2col kernel through the allocating entry point: bit-for-bit the same result
        same_kernel = torch.empty((OC, 3, 3, IC), device=dev)
        old = L.set_option("CONV_DW", "split")
        try:
            L.check(lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(same_kernel), stream))
            assert L.last_algo() == "dw"
        finally:
            L.set_option("CONV_DW", old)
        calls += 1
        if calls == 2:
            # the property the entry point exists for: the second call (the first one on this device may
            # load the kernel image) takes no device memory, neither through the CUDA allocator nor torch's
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
            reserved_before = torch.cuda.memory_reserved()
            held_before = L.workspace_in_use()
        L.check(lib.alpha_conv3d_deltaW_noalloc(C.byref(s), p(X), p(dY), p(got), stream))
        assert L.last_algo() == "dw_noalloc"
        if calls == 2:
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.cuda.memory_reserved() == reserved_before
            assert L.workspace_in_use() == held_before
        assert torch.equal(got, same_kernel)
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
