"""Generates tests/golden/conv_golden.npz, matmul_golden.npz, bmm_golden.npz and pool_golden.npz.

Run in a container that has the reference checkout (so that `make -C oracle ref` has built
oracle/_ref/libref_cpu.so).  For each small seeded case the file stores the inputs and
  ref_*   outputs of the reference project's own C++ loops (CONV_3D_NAIVE, deconv3D_deltaX_img2col,
          deconv3D_deltaW_img2col2), compiled unmodified from the checkout;
  java_*  outputs of the C restatement of the Java loops (Tense.conv3D_naive, deconv3d_deltaW_naive),
          which no JVM-less machine can run in the original; they are stored as a regression anchor
          and must stay within fp32 round-off of the ref_* values.
matmul_golden.npz holds, for small seeded matrices, the outputs of the reference's own multiply /
multiplyT1 / multiplyT2 loops (src/cu32_src/Cuda_matMul/Cuda_matMul/test.cuh:59-81); bmm_golden.npz those of bmm / bmmT1 /
bmmT2 (src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/test.cuh:95-140) on matrices in the engine's padded memory layout;
pool_golden.npz those of Pool2D_max_img2col / Pool2D_avg_img2col (src/cu32_src/Cuda_pool2D/Cuda_pool2D/test.cuh:79-157) and
unpool2D_max_img2col_plus / unpooling_avg_img2col_plus (src/cu32_src/Cuda_upool2D/Cuda_upool2D/test.cuh:90-229), on inputs
with many ties.
The GPU box has no reference checkout; the committed files are what travels.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

# name: (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, input distribution)
CASES = {
    "g_3x3_s1_p1": (2, 8, 8, 8, 12, 3, 3, 1, 1, 1, 1, "u11"),
    "g_3x3_s2_p1": (2, 9, 7, 8, 8, 3, 3, 2, 2, 1, 1, "u11"),
    "g_4x4_s2_p1": (2, 8, 8, 4, 8, 4, 4, 2, 2, 1, 1, "n01"),
    "g_5x5_s1_p2": (1, 7, 9, 8, 4, 5, 5, 1, 1, 2, 2, "u01"),
    "g_1x1": (2, 6, 6, 16, 8, 1, 1, 1, 1, 0, 0, "u11"),
    "g_3x3_nopad": (2, 7, 7, 4, 4, 3, 3, 1, 1, 0, 0, "u01"),
    "g_ic32_oc32": (2, 6, 6, 32, 32, 3, 3, 1, 1, 1, 1, "n01"),
}


# name: (N, M, K, input distribution); N, M, K multiples of 4 as the engine pads them
MATMUL_CASES = {
    "m_small": (8, 12, 16, "u11"),
    "m_k32": (16, 8, 32, "n01"),
    "m_ragged": (20, 36, 44, "u01"),
    "m_tall": (64, 4, 8, "u11"),
}


# name: (Batch, N, M, K, input distribution) before the last dimensions are padded to multiples of 4
BMM_CASES = {
    "b_ref_test": (12, 13, 21, 20, "u01"),
    "b_aligned": (3, 8, 16, 32, "n01"),
    "b_tiny": (2, 3, 5, 7, "u11"),
}

# name: (N, IH, IW, IC, FH, FW, sh, sw, ph, pw)
POOL_CASES = {
    "p_3x3_s2_p1": (2, 9, 11, 8, 3, 3, 2, 2, 1, 1),
    "p_2x2_s2": (2, 8, 8, 4, 2, 2, 2, 2, 0, 0),
    "p_2x2_s2_odd": (1, 7, 9, 4, 2, 2, 2, 2, 0, 0),
    "p_3x3_s1x2_p1": (2, 10, 9, 5, 3, 3, 1, 2, 1, 1),
    "p_4x4_s2_p1": (1, 10, 10, 8, 4, 4, 2, 2, 1, 1),
    "p_5x2_s3x1": (2, 12, 6, 4, 5, 2, 3, 1, 2, 1),
}


def pad_last(a):
    out = np.zeros(a.shape[:-1] + ((a.shape[-1] + 3) & ~3,), np.float32)
    out[..., : a.shape[-1]] = a
    return out


def gen(shape, dist, rng):
    if dist == "u11":
        return rng.uniform(-1, 1, shape).astype(np.float32)
    if dist == "u01":
        return rng.uniform(0, 1, shape).astype(np.float32)
    return rng.standard_normal(shape).astype(np.float32)


def main():
    if O.ref_lib() is None:
        raise SystemExit("oracle/_ref/libref_cpu.so is missing: run `make -C oracle ref` first")
    out = {}
    for i, (name, c) in enumerate(CASES.items()):
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw, dist = c
        rng = np.random.Generator(np.random.Philox(1000 + i))
        OH, OW = O.out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
        X = gen((N, IH, IW, IC), dist, rng)
        W = gen((OC, FH, FW, IC), dist, rng)
        dY = gen((N, OH, OW, OC), dist, rng)
        out[name + "/shape"] = np.array(c[:11], np.int32)
        out[name + "/X"], out[name + "/W"], out[name + "/dY"] = X, W, dY
        out[name + "/ref_Y"] = O.ref_CONV_3D_NAIVE(X, W, sh, sw, ph, pw)
        out[name + "/ref_dX"] = O.ref_deconv3D_deltaX_img2col(dY, W, IH, IW, sh, sw, ph, pw)
        out[name + "/ref_dW"] = O.ref_deconv3D_deltaW_img2col2(X, dY, FH, FW, sh, sw, ph, pw)
        out[name + "/java_Y"] = O.conv3D_naive(X, W, sh, sw, ph, pw)
        out[name + "/java_dW"] = O.deconv3d_deltaW_naive(X, dY, FH, FW, sh, sw, ph, pw)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    mm = {}
    for i, (name, (N, M, K, dist)) in enumerate(MATMUL_CASES.items()):
        rng = np.random.Generator(np.random.Philox(2000 + i))
        for variant, (sa, sb) in (("matMul", ((N, K), (K, M))), ("matMulT1", ((K, N), (K, M))), ("matMulT2", ((N, K), (M, K)))):
            A, B = gen(sa, dist, rng), gen(sb, dist, rng)
            mm["%s/%s/A" % (name, variant)], mm["%s/%s/B" % (name, variant)] = A, B
            mm["%s/%s/ref_C" % (name, variant)] = O.ref_matmul(A, B, variant)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "matmul_golden.npz")
    np.savez_compressed(path, **mm)
    print("wrote", path, os.path.getsize(path), "bytes")
    bm = {}
    for i, (name, (Bt, N, M, K, dist)) in enumerate(BMM_CASES.items()):
        rng = np.random.Generator(np.random.Philox(3000 + i))
        for variant, (sa, sb) in (("batchMatMul", ((Bt, N, K), (Bt, K, M))), ("batchMatMulT1", ((Bt, K, N), (Bt, K, M))),
                                  ("batchMatMulT2", ((Bt, N, K), (Bt, M, K)))):
            A, B = pad_last(gen(sa, dist, rng)), pad_last(gen(sb, dist, rng))
            key = "%s/%s" % (name, variant)
            bm[key + "/A"], bm[key + "/B"], bm[key + "/rows"] = A, B, np.int32(N)
            bm[key + "/ref_C"] = O.ref_batch_matmul(A, B, variant, rows=N)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bmm_golden.npz")
    np.savez_compressed(path, **bm)
    print("wrote", path, os.path.getsize(path), "bytes")
    pl = {}
    for i, (name, c) in enumerate(POOL_CASES.items()):
        N, IH, IW, IC, FH, FW, sh, sw, ph, pw = c
        rng = np.random.Generator(np.random.Philox(4000 + i))
        X = (np.round(gen((N, IH, IW, IC), "n01", rng) * 2) / 2).astype(np.float32)    # ties inside every window
        OH, OW = O.pool_out_hw(IH, IW, FH, FW, sh, sw, ph, pw)
        dY = gen((N, OH, OW, IC), "n01", rng)
        win = (FH, FW, sh, sw, ph, pw)
        pl[name + "/shape"] = np.array(c, np.int32)
        pl[name + "/X"], pl[name + "/dY"] = X, dY
        Y = O.ref_pool2D(X, *win, op="max")
        pl[name + "/ref_max"] = Y
        pl[name + "/ref_avg_ip"] = O.ref_pool2D(X, *win, op="avg_ignore_padding")
        pl[name + "/ref_d_max"] = O.ref_upool2D(dY, IH, IW, *win, op="max", Y=Y, X=X)
        pl[name + "/ref_d_avg_ip"] = O.ref_upool2D(dY, IH, IW, *win, op="avg")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pool_golden.npz")
    np.savez_compressed(path, **pl)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
