"""GPU parity of the batched matrix products (Engine.batchMatMul / batchMatMulT1 / batchMatMulT2, the reference's
Cuda_batchMatMul natives) against the oracle's double-precision products, the reference's CPU loops
(Cuda_batch_matMul/Cuda_batchMatMul/test.cuh:95-140) and - where they were built - the reference's own kernels
rebuilt for sm_100, natives and texture switch as in CudaFloat32EngineBase.java:1256-1318."""
import numpy as np
import pytest

from helpers import TOL, floor_rel, gen, record

pytestmark = pytest.mark.gpu

VARIANTS = ("batchMatMul", "batchMatMulT1", "batchMatMulT2")
# (Batch, N, M, K) before the engine pads last dimensions to multiples of 4
ALIGNED = [(8, 128, 128, 256), (3, 64, 96, 64), (5, 8, 32, 32), (2, 136, 160, 96), (12, 32, 64, 128)]   # tensor-core kernels
RAGGED = [(12, 13, 21, 20), (4, 64, 64, 20), (3, 7, 5, 3), (2, 82, 96, 20), (5, 33, 32, 64), (3, 64, 50, 32)]   # the reference's own test shapes among them
PAD4 = lambda n: (n + 3) & ~3


def _shapes(variant, Bt, N, M, K):
    return {"batchMatMul": ((Bt, N, K), (Bt, K, M)), "batchMatMulT1": ((Bt, K, N), (Bt, K, M)),
            "batchMatMulT2": ((Bt, N, K), (Bt, M, K))}[variant]


def _f64(variant, A, B):
    sub = {"batchMatMul": "bnk,bkm->bnm", "batchMatMulT1": "bkn,bkm->bnm", "batchMatMulT2": "bnk,bmk->bnm"}[variant]
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    return np.einsum(sub, A64, B64), np.einsum(sub, np.abs(A64), np.abs(B64))


def _pad_last(a):
    out = np.zeros(a.shape[:-1] + (PAD4(a.shape[-1]),), np.float32)
    out[..., : a.shape[-1]] = a
    return out


@pytest.fixture(scope="module")
def eng(pkg):
    import torch
    torch.cuda.set_device(0)
    return pkg.submodule("engine").Engine()


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("dims", ALIGNED + RAGGED)
def test_batched_products_against_fp64(pkg, eng, dims, variant, mode):
    import torch
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    try:
        Bt, N, M, K = dims
        sa, sb = _shapes(variant, *dims)
        rng = np.random.default_rng(Bt * 1000 + N * 7 + M * 3 + K)
        A, B = gen(sa, "u11", rng), gen(sb, "n01", rng)
        dev = torch.device("cuda:0")
        got = getattr(eng, variant)(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)).cpu().numpy()
        algo = lib.last_algo()
        assert lib.device_status() == 0 and got.shape == (Bt, N, M)
        ref, S = _f64(variant, A, B)
        err = np.abs(got - ref)
        m = dict(norm=float(err.max() / np.abs(ref).max()), comp=float((err / np.maximum(S, 1e-30)).max()), floor_rel=floor_rel(got, ref))
        record(dict(case="%s_%dx%dx%dx%d" % ((variant,) + dims), mode=mode, algo=algo, mm=m))
        assert np.isfinite(got).all() and m["norm"] <= TOL[mode]["norm"] and m["comp"] <= TOL[mode]["comp"], (algo, m)
        if dims in ALIGNED:
            assert algo.startswith("halo") or algo.startswith("dw_halo"), algo   # the tensor-core kernels, one image per entry
        else:
            assert algo in ("bmm_simt",) or algo.startswith(("halo", "dw_halo")), algo
            if mode == "tf32" and algo == "bmm_simt":
                assert m["norm"] <= TOL["3xtf32"]["norm"]      # the plain fp32 kernel does not lose precision in TF32 mode
    finally:
        lib.set_math_mode("3xtf32")


def test_reference_cpu_loops_and_acceptance(pkg, eng, oracle_mod):
    """On the reference's own kind of inputs (uniform [0, 1), its test shapes): the oracle's float loops, and the
    acceptance rule of its tests (samePercentAbsolute at 1e-3 >= 0.999)."""
    import torch
    O = oracle_mod
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    for variant in VARIANTS:
        for dims in ((12, 13, 21, 20), (15, 82, 96, 20), (4, 64, 64, 256)):
            Bt, N, M, K = dims
            sa, sb = _shapes(variant, *dims)
            A, B = gen(sa, "u01", rng), gen(sb, "u01", rng)
            got = getattr(eng, variant)(torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)).cpu().numpy()
            cpu = O.batch_matmul(_pad_last(A), _pad_last(B), variant, rows=N)[..., :M]
            assert cpu.shape == got.shape
            same = float((np.abs(got - cpu) < 1e-3).mean())
            assert same >= 0.999, (variant, dims, same)


def test_golden_vectors_of_the_reference_loops(pkg, eng):
    """The committed outputs of the reference's own bmm / bmmT1 / bmmT2 loops (tests/golden/bmm_golden.npz), through the
    engine-level entry points with the padded pitches the golden matrices carry."""
    import os
    import torch
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bmm_golden.npz"))
    dev = torch.device("cuda:0")
    base = eng.base
    for key in sorted({k.rsplit("/", 1)[0] for k in g.files}):
        variant = key.split("/")[1]
        A, B, ref, rows = g[key + "/A"], g[key + "/B"], g[key + "/ref_C"], int(g[key + "/rows"])
        tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
        Cm = torch.zeros(ref.shape, device=dev)
        Bt = A.shape[0]
        if variant == "batchMatMul":        # A [Bt, N, AK], B [Bt, BK, M]
            base.batchMatMul(Cm, tA, tB, Bt, A.shape[1], B.shape[2], B.shape[1], A.shape[2])
        elif variant == "batchMatMulT1":    # A [Bt, K, AN], B [Bt, K, M], C [Bt, CN, M]
            base.batchMatMulT1(Cm, tA, tB, Bt, rows, A.shape[2], B.shape[2], A.shape[1])
        else:                               # A [Bt, N, K], B [Bt, BM, K], C [Bt, N, CM]
            base.batchMatMulT2(Cm, tA, tB, Bt, A.shape[1], ref.shape[2], B.shape[1], A.shape[2])
        got = Cm.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max(), key


def test_natives_against_the_rebuilt_reference(pkg):
    """Both implementations of the five Cuda_batchMatMul natives, driven by the same harness with the engine's
    texture switch, on identical device tensors in the engine's memory layout."""
    import torch
    from oracle import cu32_ref
    from test_gpu_jni import FakeEnv
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    L = pkg.submodule("lib")
    L.set_math_mode("3xtf32")
    env = FakeEnv([])
    ours = cu32_ref.Cu32BatchMatMul(lib=L.load(), env=env)
    theirs = cu32_ref.Cu32BatchMatMul() if cu32_ref.batch_matmul_available() else None
    rng = np.random.default_rng(21)
    for dims in ((8, 128, 128, 256), (4, 64, 96, 64), (12, 13, 21, 20), (4, 52, 60, 36), (4, 7, 5, 3)):   # the engine rounds the batch up to 4
        Bt, N, M, K = dims
        for variant in VARIANTS:
            sa, sb = _shapes(variant, *dims)
            A, B = gen(sa, "u11", rng), gen(sb, "u11", rng)
            ref, S = _f64(variant, A, B)
            tA, tB = torch.from_numpy(_pad_last(A)).to(dev), torch.from_numpy(_pad_last(B)).to(dev)
            kw = dict(CN=N) if variant == "batchMatMulT1" else {}
            got = getattr(ours, variant)(tA, tB, **kw).cpu().numpy()
            assert env.thrown is None, env.thrown
            assert np.isfinite(got).all(), (variant, dims)
            if variant == "batchMatMulT2":
                assert (got[..., M:] == 0).all()        # padding columns of C are not touched
            err = np.abs(got[..., :M] - ref)
            assert err.max() <= 1e-4 * np.abs(ref).max() and (err <= 1e-5 * S + 1e-30).all(), (variant, dims)
            if theirs is not None:
                want = getattr(theirs, variant)(tA, tB, **kw).cpu().numpy()
                assert np.isfinite(want).all(), (variant, dims)
                assert np.abs(want[..., :M] - ref).max() <= 1e-4 * np.abs(ref).max(), ("cu32 vs fp64", variant, dims)
                assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max(), (variant, dims)
    assert {"batchMatMul", "batchMatMul_1texture", "batchMatMulT1", "batchMatMulT2", "batchMatMulT2_1texture"} <= set(ours.called)
    assert L.device_status() == 0


def test_argument_errors(pkg):
    import ctypes as C
    import torch
    L = pkg.submodule("lib")
    lib = L.load()
    t = torch.zeros(64, device="cuda:0")
    p = C.c_void_p(t.data_ptr())
    assert lib.alpha_batchMatMul(p, p, p, 0, 4, 4, 4, 4, None) == -1 and b"non-positive" in lib.alpha_conv_last_error()
    assert lib.alpha_batchMatMul(p, p, p, 1, 4, 4, 8, 4, None) == -1 and b"row pitch" in lib.alpha_conv_last_error()
    assert lib.alpha_batchMatMulT1(p, p, p, 1, 8, 4, 4, 4, None) == -1
    assert lib.alpha_batchMatMulT2(p, None, p, 1, 4, 4, 4, 4, None) == -1 and b"null" in lib.alpha_conv_last_error()
