// Thin C wrapper around the reference project's own C++ CPU convolution loops
// (TEST INFRASTRUCTURE, not product code).
//
// The build recipe (Makefile, target `ref`) cuts three functions out of the reference checkout,
// where they sit behind a disabled include guard, into generated .inc files next to the built
// library:
//   CONV_3D_NAIVE             src/cu32_src/Cuda_conv3D/Cuda_conv3D/test.cuh:80-110
//   deconv3D_deltaX_img2col   src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/test.cuh:89-131
//   deconv3D_deltaW_img2col2  src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/test.cuh:77-121
// and, for the matrix products of the FullConnect path,
//   multiply, multiplyT1, multiplyT2   src/cu32_src/Cuda_matMul/Cuda_matMul/test.cuh:59-81
//   bmm, bmmT1, bmmT2                  src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/test.cuh:95-140
// for the pooling operators,
//   Pool2D_max_img2col, Pool2D_avg_img2col                    src/cu32_src/Cuda_pool2D/Cuda_pool2D/test.cuh:79-157
//   unpooling_avg_img2col_plus, unpool2D_max_img2col_plus     src/cu32_src/Cuda_upool2D/Cuda_upool2D/test.cuh:90-229
// (with FLOAT_MIN of Cuda_pool2D/micro.cuh:40).
// This file only supplies the indexing macros they use (get4d, micro.cuh:93 of each conv library; get,
// Cuda_matMul/micro.cuh:21; get3d, Cuda_batchMatMul/micro.cuh:9) and exports them with C linkage.  No reference source text is stored in this repository.
#include <cstddef>
#include <cmath>

#define get4d(A, w, z, y, x, Sz, Sy, Sx) A[(((w) * (Sz) + (z)) * (Sy) + (y)) * (Sx) + (x)]

#define get(A, i, j, stride) A[(i) * (stride) + (j)]

#define get3d(A, z, y, x, Sy, Sx) A[(((z) * (Sy)) + (y)) * (Sx) + (x)]

#include "conv3D_naive.inc"
#include "deltaX_img2col.inc"
#include "deltaW_img2col2.inc"
#include "matmul.inc"
#include "matmulT1.inc"
#include "matmulT2.inc"
#include "bmm.inc"
#include "bmmT1.inc"
#include "bmmT2.inc"

#define FLOAT_MIN (-3.4028234E38f)
#include "pool_max.inc"
#include "pool_avg.inc"
#include "upool_avg.inc"
#include "upool_max.inc"

extern "C" {

void ref_CONV_3D_NAIVE(float *X, int IH, int IW, float *W, int FH, int FW, float *Y, int OH, int OW,
                       int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    CONV_3D_NAIVE(X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}

void ref_deconv3D_deltaX_img2col(float *deltaY, int OH, int OW, float *W, int FH, int FW,
                                 float *deltaX, int IH, int IW, int N, int IC, int OC, int sh,
                                 int sw, int ph, int pw)
{
    deconv3D_deltaX_img2col(deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}

void ref_deconv3D_deltaW_img2col2(float *X, int IH, int IW, float *deltaY, int OH, int OW,
                                  float *deltaW, int FH, int FW, int N, int IC, int OC, int sh,
                                  int sw, int ph, int pw)
{
    deconv3D_deltaW_img2col2(X, IH, IW, deltaY, OH, OW, deltaW, FH, FW, N, IC, OC, sh, sw, ph, pw);
}

// C must be zero on entry (the loops accumulate into it), as in the reference's own test driver.
void ref_multiply(float *A, float *B, float *C, int N, int M, int K) { multiply(A, B, C, N, M, K); }
void ref_multiplyT1(float *A, float *B, float *C, int N, int M, int K) { multiplyT1(A, B, C, N, M, K); }
void ref_multiplyT2(float *A, float *B, float *C, int N, int M, int K) { multiplyT2(A, B, C, N, M, K); }

// Batched products; C must be zero on entry.  Argument order of the reference's functions.
void ref_bmm(float *A, float *B, float *C, int Batch, int N, int CM, int BK, int AK) { bmm(A, B, C, Batch, N, CM, BK, AK); }
void ref_bmmT1(float *A, float *B, float *C, int Batch, int CN, int AN, int CM, int K) { bmmT1(A, B, C, Batch, CN, AN, CM, K); }
void ref_bmmT2(float *A, float *B, float *C, int Batch, int N, int CM, int BM, int K) { bmmT2(A, B, C, Batch, N, CM, BM, K); }

// Pooling: forward loops write every element of Y, backward loops every element of deltaX.
void ref_Pool2D_max(float *X, int IH, int IW, int FH, int FW, float *Y, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    Pool2D_max_img2col(X, IH, IW, FH, FW, Y, OH, OW, N, IC, sh, sw, ph, pw);
}
void ref_Pool2D_avg(float *X, int IH, int IW, int FH, int FW, float *Y, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    Pool2D_avg_img2col(X, IH, IW, FH, FW, Y, OH, OW, N, IC, sh, sw, ph, pw);
}
void ref_unpool2D_avg(float *deltaY, int OH, int OW, int FH, int FW, float *deltaX, int IH, int IW, int N, int IC, int sh, int sw,
                      int ph, int pw)
{
    unpooling_avg_img2col_plus(deltaY, OH, OW, FH, FW, deltaX, IH, IW, N, IC, sh, sw, ph, pw);
}
void ref_unpool2D_max(float *deltaY, float *Y, int OH, int OW, int FH, int FW, float *deltaX, float *X, int IH, int IW, int N,
                      int IC, int sh, int sw, int ph, int pw)
{
    unpool2D_max_img2col_plus(deltaY, Y, OH, OW, FH, FW, deltaX, X, IH, IW, N, IC, sh, sw, ph, pw);
}

}  // extern "C"
