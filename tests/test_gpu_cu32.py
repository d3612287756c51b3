"""GPU parity against the reference's own cu32 kernels rebuilt for sm_100 ("cu32 outputs").

oracle/build_ref_gpu.sh compiles the reference's three CUDA libraries where its checkout exists;
the built libraries travel with the repository snapshot.  Where they are missing the tests skip.
The rebuilt reference kernels are the only oracle of these tests: whatever they write must agree with
the reference's own CPU loop, and ours with them.
Bar: max|ours - cu32| / max|cu32| <= 1e-4 in 3xTF32 mode, 5e-3 in TF32 mode, on identical seeded
inputs, plus the reference's own samePercentRelative thresholds on positive inputs.
"""
import zlib

import numpy as np
import pytest

from helpers import floor_rel, gen, out_hw, record

pytestmark = pytest.mark.gpu

# shapes obey the natives' contract: N, IC, OC multiples of 4, GK >= 8
CASES = {
    "cfg1": (4, 32, 32, 16, 32, 3, 3, 1, 1, 1, 1),
    "s1_64_64": (8, 14, 14, 64, 64, 3, 3, 1, 1, 1, 1),
    "s1_128_256_V2": (64, 7, 7, 128, 256, 3, 3, 1, 1, 1, 1),
    "s2_3x3": (8, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1),
    "s2_4x4_deconv": (8, 16, 16, 32, 64, 4, 4, 2, 2, 1, 1),
    "w1": (8, 14, 14, 64, 96, 1, 1, 1, 1, 0, 0),
    "5x5": (4, 12, 12, 32, 36, 5, 5, 1, 1, 2, 2),
    "small_ic_crossadd": (4, 16, 16, 4, 32, 3, 3, 1, 1, 1, 1),
    "nopad": (4, 10, 10, 32, 32, 3, 3, 1, 1, 0, 0),
}


@pytest.fixture(scope="module")
def ref():
    import torch
    from oracle import cu32_ref
    if not cu32_ref.available():
        pytest.skip("oracle/_ref/libcu32_*.so not built (needs the reference checkout)")
    torch.cuda.set_device(0)
    # outputs start as NaN, so that an element no reference kernel wrote shows as such
    return cu32_ref.Cu32Reference(fill=float("nan"))


def _pixels_the_reference_leaves_unwritten(name, shape):
    """Elements of deltaX the reference's own dispatcher never writes, as a boolean mask, or None.

    Its stride-1 "A" kernels (u88As1W3_oc2pow and relatives, chosen when N % 8 == 0:
    Cuda_dconv3D_deltaX/dconv3D_dX.cuh:171, 414) number the GM = N*IH*IW output pixels with the image
    index innermost, j = (ih*IW + iw)*N + n (get_ih_iw_n, micro.cuh:193-194), while the kernels that
    take the remainder GM % 64 (k84s1_pure ..., dconv3D_dX.cuh:305-323, 467, 470-472) number them
    j = n*IH*IW + ih*IW + iw (get_n_ih_iw, micro.cuh:190-191).  The remainder is handed over as a bare
    j_index, so when GM is not a multiple of the A kernel's 64-pixel tile the two numberings do not
    describe the same pixels: the tail of the A ordering is never computed, and the tail of the
    (n, ih, iw) ordering is computed twice.  For 8 images of 14 x 14 (GM = 1568 = 24*64 + 32) the A
    kernel covers positions p = ih*IW + iw < 192 of every image, the remainder kernel positions
    164..195 of image 7 only: positions 192..195 of images 0..6 keep whatever the buffer held.
    """
    if name != "s1_64_64":
        return None
    N, IH, IW, IC = shape
    gm = N * IH * IW
    covered_a = (gm // 64) * 64
    mask = np.zeros((N, IH * IW, IC), bool)
    for n in range(N):
        for p in range(IH * IW):
            in_a = p * N + n < covered_a
            in_rem = n * IH * IW + p >= covered_a
            mask[n, p] = not (in_a or in_rem)
    return mask.reshape(N, IH, IW, IC)


@pytest.fixture(scope="module")
def eng(pkg):
    return pkg.submodule("engine").Engine()


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
@pytest.mark.parametrize("name", list(CASES))
def test_against_cu32_outputs(pkg, eng, ref, oracle_mod, name, mode):
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode(mode)
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = CASES[name]
    OH, OW = out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
    rng = np.random.default_rng(zlib.crc32(name.encode()) + 7)
    dev = torch.device("cuda:0")
    X, W, dY = (torch.from_numpy(a).to(dev) for a in (gen((N, IH, IW, IC), "u11", rng), gen((OC, FH, FW, IC), "u11", rng),
                                                      gen((N, OH, OW, OC), "n01", rng)))
    got = dict(fwd=eng.conv3D(X, W, sh, sw, ph, pw), dx=eng.dconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw),
               dw=eng.dconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw))
    assert lib.device_status() == 0
    want = dict(fwd=ref.conv3D(X, W, sh, sw, ph, pw))
    k_fwd = ref.last
    want["dx"] = ref.dconv3D_deltaX(dY, W, IH, IW, sh, sw, ph, pw)
    k_dx = ref.last
    want["dw"] = ref.dconv3D_deltaW(X, dY, FH, FW, sh, sw, ph, pw)
    tol = 1e-4 if mode == "3xtf32" else 5e-3
    Xn, Wn, dYn = X.cpu().numpy(), W.cpu().numpy(), dY.cpu().numpy()
    cpu = dict(fwd=O.conv3D_f64(Xn, Wn, sh, sw, ph, pw, threads=8)[0],
               dx=O.deconv3D_deltaX_f64(dYn, Wn, IH, IW, sh, sw, ph, pw, threads=8)[0],
               dw=O.deconv3D_deltaW_f64(Xn, dYn, FH, FW, sh, sw, ph, pw, threads=8)[0])
    errs, cu32_vs_cpu, floor = {}, {}, {}
    for op in ("fwd", "dx", "dw"):
        a, b, c = got[op].double().cpu().numpy(), want[op].double().cpu().numpy(), cpu[op]
        written = ~np.isnan(b)
        expected_holes = _pixels_the_reference_leaves_unwritten(name, (N, IH, IW, IC)) if op == "dx" else None
        if expected_holes is None:
            assert written.all(), (op, "cu32 left %d elements unwritten" % int((~written).sum()))
        else:
            # the reference's dispatcher leaves exactly these elements unwritten (see the helper's note)
            assert np.array_equal(~written, expected_holes), (op, int((~written).sum()), int(expected_holes.sum()))
        # everything cu32 did write must agree with the reference's own CPU loop: no fallback oracle
        cu32_vs_cpu[op] = float(np.abs(b - c)[written].max() / np.abs(c).max())
        assert cu32_vs_cpu[op] <= 1e-4, (op, cu32_vs_cpu)
        errs[op] = float(np.abs(a - b)[written].max() / np.abs(b[written]).max())
        floor[op] = floor_rel(a[written], b[written])
        if not written.all():   # the elements cu32 never wrote: against the CPU loop
            errs[op] = max(errs[op], float(np.abs(a - c)[~written].max() / np.abs(c).max()))
    record(dict(case=name, mode=mode, vs="cu32", ref_kernels=[k_fwd, k_dx, ref.last], cu32_vs_cpu_loop=cu32_vs_cpu,
                floor_rel_vs_cu32=floor, **errs))
    for op in ("fwd", "dx", "dw"):
        assert errs[op] <= tol, (op, errs)


def test_reference_thresholds_against_cu32(pkg, eng, ref, oracle_mod):
    """Positive inputs, the reference's own acceptance test applied between the two GPU results."""
    import torch
    O = oracle_mod
    lib = pkg.submodule("lib")
    lib.set_math_mode("3xtf32")
    N, IH, IW, IC, OC = 8, 16, 16, 64, 64
    rng = np.random.default_rng(99)
    dev = torch.device("cuda:0")
    X, W, dY = (torch.from_numpy(gen(s, "u01", rng)).to(dev) for s in ((N, IH, IW, IC), (OC, 3, 3, IC), (N, IH, IW, OC)))
    assert O.samePercentRelative(ref.conv3D(X, W, 1, 1, 1, 1).cpu().numpy(), eng.conv3D(X, W, 1, 1, 1, 1).cpu().numpy(), 1e-5) >= 0.999
    assert O.samePercentRelative(ref.dconv3D_deltaX(dY, W, IH, IW, 1, 1, 1, 1).cpu().numpy(),
                                 eng.dconv3D_deltaX(dY, W, IH, IW, 1, 1, 1, 1).cpu().numpy(), 1e-4) >= 0.999
    assert O.samePercentRelative(ref.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1).cpu().numpy(),
                                 eng.dconv3D_deltaW(X, dY, 3, 3, 1, 1, 1, 1).cpu().numpy(), 1e-5) == 1.0
