"""GPU parity of the matrix products (the FullConnect path: Engine.matMul / matMulT1 / matMulT2) against the
oracle's double-precision products, the reference's acceptance test on its own kind of inputs
(experiments/test_cuda/Cuda_matMul_test*.java: samePercentAbsolute at 1e-3 >= 0.999 on uniform [0, 1)
matrices), the stored outputs of the reference's CPU loops, and - where they were built - the
reference's own Cuda_matMul kernels rebuilt for sm_100, natives called in the engine's order."""
import ctypes as C
import os

import numpy as np
import pytest

from helpers import TOL, floor_rel, gen, record

pytestmark = pytest.mark.gpu

# (N, M, K) before padding to multiples of 4; the last ones are the FullConnect layers of the reference's
# CIFAR-10 ResNet-18 head (512 -> 128 -> 10 at batch 512) and a square product of its own speed test
DIMS = [(8, 12, 16), (64, 64, 64), (128, 256, 512), (20, 36, 44), (1149, 1149, 1024), (512, 128, 512), (512, 10, 128),
        (4, 4, 4), (256, 1024, 96)]
VARIANTS = ("matMul", "matMulT1", "matMulT2")


def _shapes(variant, N, M, K):
    return {"matMul": ((N, K), (K, M)), "matMulT1": ((K, N), (K, M)), "matMulT2": ((N, K), (M, K))}[variant]


@pytest.fixture(scope="module")
def eng(pkg):
    import torch
    torch.cuda.set_device(0)
    return pkg.submodule("engine").Engine()


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("dims", DIMS)
def test_matmul_against_the_oracle(pkg, eng, oracle_mod, dims, variant, mode):
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    N, M, K = dims
    sa, sb = _shapes(variant, N, M, K)
    rng = np.random.default_rng(N * 7 + M * 3 + K)
    A, B = gen(sa, "u11", rng), gen(sb, "n01", rng)
    dev = torch.device("cuda:0")
    got = getattr(eng, variant)(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)).cpu().numpy()
    assert lib.device_status() == 0 and got.shape == (N, M)
    ref, S = oracle_mod.matmul_f64(A, B, variant, threads=8)
    err = np.abs(got - ref)
    m = dict(norm=float(err.max() / np.abs(ref).max()), comp=float((err / np.maximum(S, 1e-30)).max()), floor_rel=floor_rel(got, ref))
    record(dict(case="%s_%dx%dx%d" % (variant, N, M, K), mode=mode, algo=lib.last_algo(), mm=m))
    assert np.isfinite(got).all() and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= TOL[mode]["comp"], (lib.last_algo(), m)
    lib.set_math_mode("3xtf32")


def test_reference_acceptance_and_golden_vectors(pkg, eng, oracle_mod):
    """The reference's own pass criterion on its own kind of inputs, and the committed outputs of its CPU loops."""
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(77)
    for variant in VARIANTS:
        for (N, M, K) in ((64, 32, 128), (100, 52, 76)):
            sa, sb = _shapes(variant, N, M, K)
            A, B = gen(sa, "u01", rng), gen(sb, "u01", rng)
            got = getattr(eng, variant)(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)).cpu().numpy()
            cpu = O.matmul(A, B, variant)
            same = float((np.abs(got - cpu) < 1e-3).mean())      # Vector.samePercentAbsolute(float[], float[]), threshold 1e-3
            assert same >= 0.999, (variant, N, M, K, same)
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "matmul_golden.npz"))
    for key in sorted({k.rsplit("/", 1)[0] for k in g.files}):
        variant = key.split("/")[1]
        A, B, ref = g[key + "/A"], g[key + "/B"], g[key + "/ref_C"]
        got = getattr(eng, variant)(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)).cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), key
    assert lib.device_status() == 0


def test_matmul_biased_and_engine_modes(pkg, eng, oracle_mod):
    import torch
    lib = pkg.submodule("lib")
    E = pkg.submodule("engine")
    lib.set_math_mode("3xtf32")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    A, B, bias = gen((96, 160), "u11", rng), gen((160, 72), "n01", rng), gen((72,), "u11", rng)
    tA, tB, tb = (torch.from_numpy(a).to(dev) for a in (A, B, bias))
    got = eng.matMul(tA, tB, Bias=tb).cpu().numpy()
    ref, S = oracle_mod.matmul_f64(A, B, "matMul", threads=8)
    ref = ref + bias.astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()
    assert ((np.abs(got - ref)) <= 1e-5 * (S + np.abs(bias)) + 1e-30).all()
    fast = E.Engine(E.CudaFloat32EngineBase(math="tf32"))
    coarse = fast.matMul(tA, tB).cpu().numpy()
    e = np.abs(coarse - (ref - bias)).max() / np.abs(ref).max()
    assert 1e-5 < e <= 5e-3 and lib.load().alpha_conv_get_math_mode() == 0
    assert lib.device_status() == 0


def test_matmul_natives_against_the_rebuilt_reference(pkg, oracle_mod):
    """Both implementations of the five Cuda_matMul natives, driven by the same harness in the engine's
    call order (matMulT1 -> matMulT1SK + SKbuf_summary from K = 512 on), on identical device tensors."""
    import torch
    from oracle import cu32_ref
    from test_gpu_jni import FakeEnv
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    L.set_math_mode("3xtf32")
    env = FakeEnv([])
    ours = cu32_ref.Cu32MatMul(lib=L.load(), env=env)
    theirs = cu32_ref.Cu32MatMul() if cu32_ref.matmul_available() else None
    rng = np.random.default_rng(11)
    for (N, M, K) in ((64, 96, 128), (128, 64, 768), (256, 128, 2048), (52, 20, 36)):
        for variant in VARIANTS:
            sa, sb = _shapes(variant, N, M, K)
            A, B = gen(sa, "u11", rng), gen(sb, "u11", rng)
            tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
            got = getattr(ours, variant)(tA, tB)
            assert env.thrown is None, env.thrown
            ref, S = oracle_mod.matmul_f64(A, B, variant, threads=8)
            err = np.abs(got.cpu().numpy() - ref)
            assert err.max() <= 1e-4 * np.abs(ref).max() and (err <= 1e-5 * S + 1e-30).all(), (variant, N, M, K)
            if theirs is not None:
                want = getattr(theirs, variant)(tA, tB).cpu().numpy()
                assert np.isfinite(want).all(), (variant, N, M, K)
                assert np.abs(want - ref).max() <= 1e-4 * np.abs(ref).max(), ("cu32 vs fp64", variant, N, M, K)
                assert np.abs(got.cpu().numpy() - want).max() <= 1e-4 * np.abs(want).max(), (variant, N, M, K)
    assert {"matMul", "matMulT1", "matMulT1SK", "SKbuf_1summary", "matMulT2"} <= set(ours.called)
    # SKbuf_summary on buffers that hold numbers
    C0 = torch.randn(64 * 96, device=dev)
    buf = torch.randn(3 * 64 * 96, device=dev)
    want = C0.double() + buf.double().view(3, -1).sum(0)
    ours._call("SKbuf_1summary", ("long", ours.streams[0].cuda_stream), buf, C0, 3, 64 * 96)
    torch.cuda.synchronize()
    assert float((C0.double() - want).abs().max()) <= 1e-6 * float(want.abs().max() + 1)
    assert L.device_status() == 0
