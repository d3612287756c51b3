"""GPU tests of the scratch-memory interface, the weight cache and the per-call settings.

The reference's natives get all scratch from the Java mempool; this library keeps one block per
stream, which a host may size in advance, replace with memory of its own, or release.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw): one shape per scratch user
SHAPES = {
    "s1_pair": (16, 14, 14, 128, 128, 3, 3, 1, 1, 1, 1),       # lo plane / transposed planes / per-CTA partials
    "s2_phases": (8, 16, 16, 64, 64, 3, 3, 2, 2, 1, 1),        # stride phases of deltaX, split-K deltaW
    "stem_ic4": (8, 32, 32, 4, 64, 7, 7, 2, 2, 3, 3),          # patch matrix, col2im
    "tiny_image": (32, 2, 2, 64, 64, 3, 3, 1, 1, 1, 1),        # patch matrix of a stride-1 layer
}


def _tensors(case, dev, seed=3):
    import torch
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    g = torch.Generator(device=dev).manual_seed(seed)
    X = torch.randn((N, IH, IW, IC), device=dev, generator=g)
    W = torch.randn((OC, FH, FW, IC), device=dev, generator=g) * 0.1
    dY = torch.randn((N, OH, OW, OC), device=dev, generator=g)
    return X, W, dY, (OH, OW)


def _run_all(L, lib, case, X, W, dY, OH, OW, stream):
    import torch
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    s = L.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
    p = lambda t: C.c_void_p(t.data_ptr())
    Y = torch.empty((N, OH, OW, OC), device=X.device)
    dX = torch.empty_like(X)
    dW = torch.empty_like(W)
    st = C.c_void_p(stream.cuda_stream)
    with torch.cuda.stream(stream):
        rcs = (lib.alpha_conv3d_forward(C.byref(s), p(X), p(W), None, p(Y), st),
               lib.alpha_conv3d_deltaX(C.byref(s), p(dY), p(W), p(dX), st),
               lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(dW), st))
    stream.synchronize()
    return rcs, (Y, dX, dW), s


@pytest.mark.parametrize("name", list(SHAPES))
def test_caller_owned_workspace_of_the_announced_size(pkg, name):
    """alpha_conv_workspace_bytes is exact: a caller block of that size serves the call (same bits as
    with library-owned scratch), a block 256 bytes short is refused with ALPHA_E_NOSCRATCH, and the
    library allocates nothing for the stream."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    lib = L.load()
    L.set_math_mode("3xtf32")
    case = SHAPES[name]
    X, W, dY, (OH, OW) = _tensors(case, dev)
    own = torch.cuda.Stream()
    rcs, ref, s = _run_all(L, lib, case, X, W, dY, OH, OW, own)
    assert rcs == (0, 0, 0), L.last_error()
    need = {op: L.workspace_bytes(s, op) for op in ("forward", "deltaX", "deltaW")}
    assert all(v % 256 == 0 for v in need.values())
    big = max(need.values())
    ext = torch.cuda.Stream()
    block = torch.empty(max(big, 256), dtype=torch.uint8, device=dev)
    assert block.data_ptr() % 256 == 0
    held = L.workspace_in_use()
    L.set_workspace(ext.cuda_stream, block.data_ptr(), big)
    try:
        rcs, got, _ = _run_all(L, lib, case, X, W, dY, OH, OW, ext)
        assert rcs == (0, 0, 0), L.last_error()
        assert L.workspace_in_use() == held          # nothing was allocated for this stream
        for a, b in zip(got, ref):
            assert torch.equal(a, b)
        if big >= 256:
            L.set_workspace(ext.cuda_stream, block.data_ptr(), big - 256)
            rcs, _, _ = _run_all(L, lib, case, X, W, dY, OH, OW, ext)
            assert -5 in rcs and all(rc in (0, -5) for rc in rcs), rcs
            assert "alpha_conv_workspace_bytes" in L.last_error()
    finally:
        L.set_workspace(ext.cuda_stream, 0, 0)
    assert L.device_status() == 0


def test_growth_inside_a_stream_capture_is_refused_not_synchronised(pkg):
    """A call that would have to grow its stream's block while the stream is being captured returns
    ALPHA_E_CAPTURE (the capture stays valid); after alpha_conv_reserve_workspace the same capture
    succeeds, and a later, larger eager call on the stream leaves the captured graph replayable."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    lib = L.load()
    L.set_math_mode("3xtf32")
    case = SHAPES["s1_pair"]
    X, W, dY, (OH, OW) = _tensors(case, dev)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    s = L.AlphaConvShape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw)
    p = lambda t: C.c_void_p(t.data_ptr())
    ref = torch.empty_like(W)
    L.check(lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(ref), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()

    side = torch.cuda.Stream()      # a fresh stream: no block yet
    dW = torch.zeros_like(W)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        rc = lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(dW), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        captured_stream = torch.cuda.current_stream().cuda_stream
    assert rc == -6 and "alpha_conv_reserve_workspace" in L.last_error(), (rc, L.last_error())
    del g
    L.reserve_workspace(captured_stream, L.workspace_bytes(s, "deltaW"))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        rc = lib.alpha_conv3d_deltaW(C.byref(s), p(X), p(dY), p(dW), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.last_error()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(dW, ref)
    # a larger eager call on the captured stream outgrows the block; the graph keeps its own
    bigcase = (64, 14, 14, 128, 128, 3, 3, 1, 1, 1, 1)
    bX, bW, bdY, _ = _tensors(bigcase, dev, seed=4)
    bs = L.AlphaConvShape(*bigcase[:7], OH, OW, 1, 1, 1, 1)
    if L.workspace_bytes(bs, "deltaW") <= L.workspace_bytes(s, "deltaW"):
        bigcase = (8, 14, 14, 128, 512, 3, 3, 1, 1, 1, 1)
        bX, bW, bdY, _ = _tensors(bigcase, dev, seed=4)
        bs = L.AlphaConvShape(*bigcase[:7], OH, OW, 1, 1, 1, 1)
    bdW = torch.empty_like(bW)
    with torch.cuda.stream(side):
        L.check(lib.alpha_conv3d_deltaW(C.byref(bs), p(bX), p(bdY), p(bdW), C.c_void_p(captured_stream)))
    dW.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(dW, ref)
    assert L.device_status() == 0


def test_weight_cache_skips_the_transforms_until_the_weights_change(pkg):
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    lib = L.load()
    L.set_math_mode("3xtf32")
    for name in ("s1_pair", "s2_phases", "stem_ic4"):
        case = SHAPES[name]
        X, W, dY, (OH, OW) = _tensors(case, dev)
        st = torch.cuda.current_stream()
        _, ref, s = _run_all(L, lib, case, X, W, dY, OH, OW, st)
        n0 = L.launch_count(); _run_all(L, lib, case, X, W, dY, OH, OW, st); plain = L.launch_count() - n0
        L.weight_cache(True)
        try:
            _, first, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st)                # fills the cache
            n0 = L.launch_count(); _, hit, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st); cached = L.launch_count() - n0
            assert cached < plain, (name, plain, cached)
            for a, b, c in zip(ref, first, hit):
                assert torch.equal(a, b) and torch.equal(a, c)
            # an optimizer step: new values at the same address
            W.mul_(1.5)
            L.weights_updated(W.data_ptr())
            n0 = L.launch_count(); _, upd, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st); refill = L.launch_count() - n0
            assert refill == plain
        finally:
            L.weight_cache(False)
            L.weights_updated(None)
        _, want, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st)
        for a, b in zip(upd, want):
            assert torch.equal(a, b)
    assert L.device_status() == 0


def test_two_engines_of_one_process_keep_their_own_math_mode(pkg):
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    E = pkg.submodule("engine")
    L.set_math_mode("3xtf32")
    case = SHAPES["s1_pair"]
    X, W, dY, _ = _tensors(case, dev)
    exact = E.Engine(E.CudaFloat32EngineBase(math="3xtf32"))
    fast = E.Engine(E.CudaFloat32EngineBase(math="tf32"))
    dflt = E.Engine()
    ref = torch.nn.functional.conv2d(X.double().permute(0, 3, 1, 2), W.double().permute(0, 3, 1, 2), padding=1).permute(0, 2, 3, 1)
    ya, yb, yc, ya2 = exact.conv3D(X, W, 1, 1, 1, 1), fast.conv3D(X, W, 1, 1, 1, 1), dflt.conv3D(X, W, 1, 1, 1, 1), exact.conv3D(X, W, 1, 1, 1, 1)
    err = lambda y: float((y.double() - ref).abs().max() / ref.abs().max())
    assert err(ya) <= 1e-4 and torch.equal(ya, yc) and torch.equal(ya, ya2)
    assert 1e-5 < err(yb) <= 5e-3                # plain TF32: visibly coarser, inside its own bound
    assert L.load().alpha_conv_get_math_mode() == 0     # the process default was never touched
    s = L.AlphaConvShape(*case[:7], 14, 14, 1, 1, 1, 1)
    assert L.load().alpha_conv3d_forward_ex(C.byref(s), 16, 32, None, 48, 7, -1, None) == -1


def test_sm_budget_leaves_sms_free_without_changing_the_results(pkg):
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    lib = L.load()
    L.set_math_mode("3xtf32")
    case = (32, 28, 28, 128, 128, 3, 3, 1, 1, 1, 1)
    X, W, dY, (OH, OW) = _tensors(case, dev)
    st = torch.cuda.current_stream()
    _, ref, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st)
    old = L.set_option("SM_BUDGET", 132)
    try:
        _, got, _ = _run_all(L, lib, case, X, W, dY, OH, OW, st)
    finally:
        L.set_option("SM_BUDGET", old)
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1])      # per-tile results do not depend on the grid
    assert float((got[2] - ref[2]).abs().max()) <= 1e-5 * float(ref[2].abs().max())   # deltaW: other partial sums
    assert L.device_status() == 0


def test_prepared_weights_in_caller_memory(pkg):
    """The weight-side transforms computed ahead of the contraction into blocks the caller owns: same bits as
    the plain calls, one launch fewer per contraction, nothing allocated by the library, and a block made for
    another math mode is refused."""
    import torch
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    base = pkg.submodule("engine").CudaFloat32EngineBase()
    L.set_math_mode("3xtf32")
    for name in ("s1_pair", "s2_phases", "stem_ic4", "tiny_image"):
        case = SHAPES[name]
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        X, W, dY, (OH, OW) = _tensors(case, dev, seed=8)
        Y0, dX0 = torch.empty((N, OH, OW, OC), device=dev), torch.empty_like(X)
        n0 = L.launch_count()
        base.conv3D(Y0, OH, OW, X, IH, IW, W, FH, FW, N, IC, OC, sh, sw, ph, pw)
        base.dconv3D_deltaX(dX0, IH, IW, dY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw)
        plain = L.launch_count() - n0
        held = L.workspace_in_use()
        side = torch.cuda.Stream()
        geo = (FH, FW, N, IH, IW, OH, OW, IC, OC, sh, sw, ph, pw)
        with torch.cuda.stream(side):
            pf = base.prepare_weights("forward", W, *geo, stream=side)
            pd = base.prepare_weights("deltaX", W, *geo, stream=side)
        torch.cuda.current_stream().wait_stream(side)
        assert pd is not None and (pf is not None or sh > 1)      # the strided forward kernel splits W tiles itself
        Y1, dX1 = torch.empty_like(Y0), torch.empty_like(dX0)
        n0 = L.launch_count()
        base.conv3D_prepared(Y1, OH, OW, X, IH, IW, W, FH, FW, N, IC, OC, sh, sw, ph, pw, pf)
        base.dconv3D_deltaX_prepared(dX1, IH, IW, dY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw, pd)
        used = L.launch_count() - n0
        torch.cuda.synchronize()
        assert torch.equal(Y0, Y1) and torch.equal(dX0, dX1), name
        assert used == plain - (pf is not None) - (pd is not None), (name, plain, used)
        assert L.workspace_in_use() <= held, name
        # blocks swapped between the operators, or made under another math mode, are refused on the host
        if pf is not None:
            with pytest.raises(L.AlphaConvError):
                base.dconv3D_deltaX_prepared(dX1, IH, IW, dY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw, pf)
        L.set_math_mode("tf32")
        try:
            assert base.prepare_weights("forward", W, *geo) is None       # plain TF32 forward reads W as it is
            with pytest.raises(L.AlphaConvError):
                base.dconv3D_deltaX_prepared(dX1, IH, IW, dY, OH, OW, W, FH, FW, N, IC, OC, sh, sw, ph, pw, pd)
        finally:
            L.set_math_mode("3xtf32")
    assert L.device_status() == 0
