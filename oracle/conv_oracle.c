/*
 * CPU oracle for the Dragon-Alpha conv hot path (TEST INFRASTRUCTURE, not product code).
 *
 * A plain-C restatement of the reference's CPU convolution loops.  Only the test suite, the
 * smoke check and the benchmark's cpu_baseline / reference arm may link or call this file;
 * the CUDA library never does.
 *
 * Layouts (all fp32, C-contiguous, NHWC):
 *   X[N,IH,IW,IC]  W[OC,FH,FW,IC]  Y[N,OH,OW,OC]   deltaX like X, deltaY like Y, deltaW like W.
 *
 * Every function states the reference loop it follows (path inside the reference project).
 * Java semantics that matter for bit-exactness are kept:
 *   - `double v; v += x*w` with float x, w: the product is rounded to float first, then widened.
 *   - `float v; v += x*w`: float product, float add (no fused multiply-add).
 * Compile with -ffp-contract=off so the compiler cannot fuse the multiply and the add.
 *
 * The *_mt variants split the outermost independent loop over OpenMP threads; each output element
 * is still produced by exactly the same sequence of operations, so results are bit-identical.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define IDX4(w, z, y, x, Sz, Sy, Sx) ((((size_t)(w) * (Sz) + (z)) * (Sy) + (y)) * (Sx) + (x))

int oracle_max_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Forward convolution, double accumulator.
 * Follows src/zutil_src/z/util/math/vector/Tense.java:143-173 (Tense.conv3D_naive):
 * loop order n -> oc -> oh -> ow -> fh -> fw -> ic, `double v += X*W` (float product), cast to
 * float on store (:170).  Taps outside the image are skipped (:168).
 */
void oracle_conv3D_naive(const float *X, int IH, int IW, const float *W, int FH, int FW, float *Y,
                         int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                         int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int n = 0; n < N; n++)
        for (int oc = 0; oc < OC; oc++) {
            for (int oh = 0; oh < OH; oh++) {
                int ih_s = -ph + oh * sh;
                if (ih_s > IH + ph - FH) break;
                for (int ow = 0; ow < OW; ow++) {
                    int iw_s = -pw + ow * sw;
                    if (iw_s > IW + pw - FW) break;
                    double v = 0;
                    for (int fh = 0; fh < FH; fh++)
                        for (int fw = 0; fw < FW; fw++)
                            for (int ic = 0; ic < IC; ic++) {
                                int ih = ih_s + fh, iw = iw_s + fw;
                                if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                                float p = X[IDX4(n, ih, iw, ic, IH, IW, IC)] *
                                          W[IDX4(oc, fh, fw, ic, FH, FW, IC)];
                                v += (double)p;
                            }
                    Y[IDX4(n, oh, ow, oc, OH, OW, OC)] = (float)v;
                }
            }
        }
}

/*
 * Forward convolution, float accumulator.
 * Follows CONV_3D_NAIVE, src/cu32_src/Cuda_conv3D/Cuda_conv3D/test.cuh:80-110: the same taps in the
 * same fh -> fw -> ic order as the Java loop above, but `float v += X*W`.  Exists so that the
 * restatement can be pinned bit-for-bit against the reference's own compiled C++ loop.
 */
void oracle_conv3D_naive_f32(const float *X, int IH, int IW, const float *W, int FH, int FW,
                             float *Y, int OH, int OW, int N, int IC, int OC, int sh, int sw,
                             int ph, int pw, int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int oc = 0; oc < OC; oc++)
        for (int n = 0; n < N; n++) {
            int oh = 0;
            for (int ih_s = -ph; ih_s <= (IH + ph - FH); ih_s += sh, oh++) {
                int ow = 0;
                for (int iw_s = -pw; iw_s <= (IW + pw - FW); iw_s += sw, ow++) {
                    float v = 0;
                    for (int fh = 0; fh < FH; fh++)
                        for (int fw = 0; fw < FW; fw++)
                            for (int ic = 0; ic < IC; ic++) {
                                int ih = ih_s + fh, iw = iw_s + fw;
                                if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                                float p = X[IDX4(n, ih, iw, ic, IH, IW, IC)] *
                                          W[IDX4(oc, fh, fw, ic, FH, FW, IC)];
                                v = v + p;
                            }
                    Y[IDX4(n, oh, ow, oc, OH, OW, OC)] = v;
                }
            }
        }
}

/*
 * Forward convolution in full double precision (double products, double accumulator); used only
 * for error analysis.  Follows Tense.conv3D_naive_double, Tense.java:175-205, with the float
 * inputs widened first.  Also returns S[n,oh,ow,oc] = sum |x|*|w| when S != NULL: the
 * denominator of the componentwise forward-error bound.
 */
void oracle_conv3D_f64(const float *X, int IH, int IW, const float *W, int FH, int FW, double *Y,
                       double *S, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph,
                       int pw, int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int n = 0; n < N; n++)
        for (int oc = 0; oc < OC; oc++)
            for (int oh = 0; oh < OH; oh++)
                for (int ow = 0; ow < OW; ow++) {
                    double v = 0, s = 0;
                    for (int fh = 0; fh < FH; fh++)
                        for (int fw = 0; fw < FW; fw++) {
                            int ih = oh * sh - ph + fh, iw = ow * sw - pw + fw;
                            if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                            const float *x = X + IDX4(n, ih, iw, 0, IH, IW, IC);
                            const float *w = W + IDX4(oc, fh, fw, 0, FH, FW, IC);
                            for (int ic = 0; ic < IC; ic++) {
                                double p = (double)x[ic] * (double)w[ic];
                                v += p;
                                s += fabs(p);
                            }
                        }
                    Y[IDX4(n, oh, ow, oc, OH, OW, OC)] = v;
                    if (S) S[IDX4(n, oh, ow, oc, OH, OW, OC)] = s;
                }
}

/*
 * Row-broadcast bias add, Y[n,oh,ow,oc] += bias[oc], float add.
 * Follows the bias stage of CudaFloat32EngineBase.conv3D_biased
 * (src/alpha_src/z/dragon/engine/cuda/CudaFloat32EngineBase.java:1548-1557), which runs
 * linear_dual2D_row with alpha = beta = 1, gamma = 0
 * (src/cu32_src/Cuda_function/Cuda_function/type1_linear_dual2D_row.cuh:35-62).
 */
void oracle_add_bias_row(float *Y, const float *bias, size_t rows, int OC)
{
    for (size_t r = 0; r < rows; r++)
        for (int oc = 0; oc < OC; oc++) Y[r * OC + oc] = Y[r * OC + oc] + bias[oc];
}

/*
 * Input gradient / transposed convolution, float accumulator.
 * Follows Tense.deconv3D_deltaX_img2col, Tense.java:334-375 (the same loop exists in C++ at
 * src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/test.cuh:89-131):
 * for ic, for j=(n,ih,iw), for k=(oc,fh,fw): positions of the zero-stuffed, outer-padded deltaY
 * that fall between real samples are skipped; W is read rotated by 180 degrees.
 */
void oracle_deconv3D_deltaX_img2col(const float *deltaY, int OH, int OW, const float *W, int FH,
                                    int FW, float *deltaX, int IH, int IW, int N, int IC, int OC,
                                    int sh, int sw, int ph, int pw, int threads)
{
    (void)threads;
    const int GM = N * IH * IW, GK = OC * FH * FW;
    const int OHp = OH + (OH - 1) * (sh - 1), OWp = OW + (OW - 1) * (sw - 1);
    const int oph = FH - ph - 1, opw = FW - pw - 1;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int j = 0; j < GM; j++) {
        int n = j / (IH * IW), j_res = j % (IH * IW);
        int ih = j_res / IW, iw = j_res % IW;
        for (int ic = 0; ic < IC; ic++) {
            float v = 0;
            for (int k = 0; k < GK; k++) {
                int oc = k / (FH * FW), k_res = k % (FH * FW);
                int fh = k_res / FW, fw = k_res % FW;
                int oh = ih - oph + fh, ow = iw - opw + fw;
                if (oh < 0 || ow < 0 || oh >= OHp || ow >= OWp) continue;
                if (oh % sh != 0 || ow % sw != 0) continue;
                float p = deltaY[IDX4(n, oh / sh, ow / sw, oc, OH, OW, OC)] *
                          W[IDX4(oc, FH - 1 - fh, FW - 1 - fw, ic, FH, FW, IC)];
                v = v + p;
            }
            deltaX[IDX4(n, ih, iw, ic, IH, IW, IC)] = v;
        }
    }
}

/*
 * Input gradient in scatter form, float accumulation into deltaX (caller zeroes deltaX).
 * Follows Tense.deconv3D_deltaX_crossAdd, Tense.java:441-469: loop order oc -> n -> oh -> ow ->
 * fh -> fw -> ic, `deltaX[n][ih][iw][ic] += w*dy`.  Single-threaded: the order of the adds is
 * part of the result.
 */
void oracle_deconv3D_deltaX_crossAdd(const float *deltaY, int OH, int OW, const float *W, int FH,
                                     int FW, float *deltaX, int IH, int IW, int N, int IC, int OC,
                                     int sh, int sw, int ph, int pw)
{
    for (int oc = 0; oc < OC; oc++)
        for (int n = 0; n < N; n++)
            for (int oh = 0; oh < OH; oh++)
                for (int ow = 0; ow < OW; ow++) {
                    float dy = deltaY[IDX4(n, oh, ow, oc, OH, OW, OC)];
                    for (int fh = 0; fh < FH; fh++)
                        for (int fw = 0; fw < FW; fw++) {
                            int ih = oh * sh - ph + fh, iw = ow * sw - pw + fw;
                            if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                            for (int ic = 0; ic < IC; ic++) {
                                float w = W[IDX4(oc, fh, fw, ic, FH, FW, IC)];
                                float p = w * dy;
                                float *d = deltaX + IDX4(n, ih, iw, ic, IH, IW, IC);
                                *d = *d + p;
                            }
                        }
                }
}

/* Input gradient in double precision with S = sum |dy|*|w| (error analysis only). */
void oracle_deconv3D_deltaX_f64(const float *deltaY, int OH, int OW, const float *W, int FH, int FW,
                                double *deltaX, double *S, int IH, int IW, int N, int IC, int OC,
                                int sh, int sw, int ph, int pw, int threads)
{
    (void)threads;
    const int GM = N * IH * IW;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int j = 0; j < GM; j++) {
        int n = j / (IH * IW), j_res = j % (IH * IW);
        int ih = j_res / IW, iw = j_res % IW;
        for (int ic = 0; ic < IC; ic++) {
            double v = 0, s = 0;
            for (int fh = 0; fh < FH; fh++) {
                int t = ih + ph - fh;
                if (t < 0 || t % sh != 0 || t / sh >= OH) continue;
                for (int fw = 0; fw < FW; fw++) {
                    int u = iw + pw - fw;
                    if (u < 0 || u % sw != 0 || u / sw >= OW) continue;
                    for (int oc = 0; oc < OC; oc++) {
                        double p = (double)deltaY[IDX4(n, t / sh, u / sw, oc, OH, OW, OC)] *
                                   (double)W[IDX4(oc, fh, fw, ic, FH, FW, IC)];
                        v += p;
                        s += fabs(p);
                    }
                }
            }
            deltaX[IDX4(n, ih, iw, ic, IH, IW, IC)] = v;
            if (S) S[IDX4(n, ih, iw, ic, IH, IW, IC)] = s;
        }
    }
}

/*
 * Weight gradient, float accumulator.
 * Follows Tense.deconv3D_deltaW_img2col2, Tense.java:1364-1401 (C++ twin:
 * src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/test.cuh:77-121):
 * for oc, for j=(ic,fh,fw), for k=(n,oh,ow): float `v += X*deltaY`.
 */
void oracle_deconv3D_deltaW_img2col2(const float *X, int IH, int IW, const float *deltaY, int OH,
                                     int OW, float *deltaW, int FH, int FW, int N, int IC, int OC,
                                     int sh, int sw, int ph, int pw, int threads)
{
    (void)threads;
    const int GM = IC * FH * FW, GK = N * OH * OW;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int oc = 0; oc < OC; oc++)
        for (int j = 0; j < GM; j++) {
            int ic = j / (FH * FW), j_res = j % (FH * FW);
            int fh = j_res / FW, fw = j_res % FW;
            float v = 0;
            for (int k = 0; k < GK; k++) {
                int n = k / (OH * OW), k_res = k % (OH * OW);
                int oh = k_res / OW, ow = k_res % OW;
                int ih = fh - ph + oh * sh, iw = fw - pw + ow * sw;
                if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                float p = X[IDX4(n, ih, iw, ic, IH, IW, IC)] *
                          deltaY[IDX4(n, oh, ow, oc, OH, OW, OC)];
                v = v + p;
            }
            deltaW[IDX4(oc, fh, fw, ic, FH, FW, IC)] = v;
        }
}

/*
 * Weight gradient, double accumulator.
 * Follows Tense.deconv3d_deltaW_naive, Tense.java:1277-1319, which swaps the N and channel axes of
 * X and of the zero-stuffed deltaY and runs Tense.conv3D_naive over them.  Unrolled, that is: for
 * each (ic, oc, fh, fw) a double accumulator over oh -> ow -> n (the conv's fh', fw', ic' loops),
 * float products; the zero-stuffed positions contribute an exact +0 and are skipped here.
 */
void oracle_deconv3d_deltaW_naive(const float *X, int IH, int IW, const float *deltaY, int OH,
                                  int OW, float *deltaW, int FH, int FW, int N, int IC, int OC,
                                  int sh, int sw, int ph, int pw, int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int ic = 0; ic < IC; ic++)
        for (int oc = 0; oc < OC; oc++)
            for (int fh = 0; fh < FH; fh++)
                for (int fw = 0; fw < FW; fw++) {
                    double v = 0;
                    for (int oh = 0; oh < OH; oh++) {
                        int ih = fh - ph + oh * sh;
                        if (ih < 0 || ih >= IH) continue;
                        for (int ow = 0; ow < OW; ow++) {
                            int iw = fw - pw + ow * sw;
                            if (iw < 0 || iw >= IW) continue;
                            for (int n = 0; n < N; n++) {
                                float p = X[IDX4(n, ih, iw, ic, IH, IW, IC)] *
                                          deltaY[IDX4(n, oh, ow, oc, OH, OW, OC)];
                                v += (double)p;
                            }
                        }
                    }
                    deltaW[IDX4(oc, fh, fw, ic, FH, FW, IC)] = (float)v;
                }
}

/* Weight gradient in double precision with S = sum |x|*|dy| (error analysis only). */
void oracle_deconv3D_deltaW_f64(const float *X, int IH, int IW, const float *deltaY, int OH, int OW,
                                double *deltaW, double *S, int FH, int FW, int N, int IC, int OC,
                                int sh, int sw, int ph, int pw, int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int oc = 0; oc < OC; oc++)
        for (int fh = 0; fh < FH; fh++)
            for (int fw = 0; fw < FW; fw++)
                for (int ic = 0; ic < IC; ic++) {
                    double v = 0, s = 0;
                    for (int n = 0; n < N; n++)
                        for (int oh = 0; oh < OH; oh++) {
                            int ih = fh - ph + oh * sh;
                            if (ih < 0 || ih >= IH) continue;
                            for (int ow = 0; ow < OW; ow++) {
                                int iw = fw - pw + ow * sw;
                                if (iw < 0 || iw >= IW) continue;
                                double p = (double)X[IDX4(n, ih, iw, ic, IH, IW, IC)] *
                                           (double)deltaY[IDX4(n, oh, ow, oc, OH, OW, OC)];
                                v += p;
                                s += fabs(p);
                            }
                        }
                    deltaW[IDX4(oc, fh, fw, ic, FH, FW, IC)] = v;
                    if (S) S[IDX4(oc, fh, fw, ic, FH, FW, IC)] = s;
                }
}

/*
 * Fraction of elements that agree, the reference's acceptance metric.
 * Follows Vector.samePercentRelative, src/zutil_src/z/util/math/vector/Vector.java:4109-4125:
 * equal values count; otherwise |(a-b+MIN)/(a+b+MIN)| < threshold with MIN = Float.MIN_VALUE,
 * evaluated in float; two NaNs count as equal.
 */
float oracle_samePercentRelative(const float *A, const float *B, size_t length, float threshold)
{
    const float MINV = 1.4e-45f; /* Float.MIN_VALUE */
    size_t sum = 0;
    for (size_t i = 0; i < length; i++) {
        if (A[i] == B[i]) { sum++; continue; }
        float div = fabsf((A[i] - B[i] + MINV) / (A[i] + B[i] + MINV));
        if (div < threshold) { sum++; continue; }
        if (isnan(A[i]) && isnan(B[i])) { sum++; continue; }
    }
    return (float)sum / (float)length;
}

/*
 * Matrix products of the FullConnect path (the "next" contraction after the convolutions).
 * Follow the CPU loops of the reference's own tests, experiments/test_cuda/Cuda_matMul_test.java:28-36
 * (multiply), Cuda_matMul_test_T1.java:27-35 (multiplyT1), Cuda_matMul_test_T2.java:27-35 (multiplyT2),
 * and the same loops in src/cu32_src/Cuda_matMul/Cuda_matMul/test.cuh:59-81: loop order k -> i -> j,
 * `float C[i][j] += A * B` (float product, float add), C zero at the start.
 *   variant 0: C[N,M] = A[N,K]   * B[K,M]
 *   variant 1: C[N,M] = A[K,N]^T * B[K,M]
 *   variant 2: C[N,M] = A[N,K]   * B[M,K]^T
 */
void oracle_matmul(const float *A, const float *B, float *C, int N, int M, int K, int variant)
{
    memset(C, 0, sizeof(float) * (size_t)N * M);
    for (int k = 0; k < K; k++)
        for (int i = 0; i < N; i++) {
            const float a = variant == 1 ? A[(size_t)k * N + i] : A[(size_t)i * K + k];
            for (int j = 0; j < M; j++) {
                const float b = variant == 2 ? B[(size_t)j * K + k] : B[(size_t)k * M + j];
                C[(size_t)i * M + j] += a * b;
            }
        }
}

/* The same products in double, with S[i][j] = sum_k |a||b| (the scale of the forward error bound). */
void oracle_matmul_f64(const float *A, const float *B, double *C, double *S, int N, int M, int K, int variant,
                       int threads)
{
    (void)threads;
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int i = 0; i < N; i++)
        for (int j = 0; j < M; j++) {
            double v = 0, sa = 0;
            for (int k = 0; k < K; k++) {
                const double a = variant == 1 ? A[(size_t)k * N + i] : A[(size_t)i * K + k];
                const double b = variant == 2 ? B[(size_t)j * K + k] : B[(size_t)k * M + j];
                v += a * b;
                sa += fabs(a * b);
            }
            C[(size_t)i * M + j] = v;
            S[(size_t)i * M + j] = sa;
        }
}

/* Batched matrix products with the engine's padded row pitches (TEST INFRASTRUCTURE).  Follows the reference's CPU
 * loops bmm / bmmT1 / bmmT2 (src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/test.cuh:95-140): k outermost, float
 * multiply then float add into C, which is zeroed first.
 *   variant 0: C[b][N][M]       = A[b][N][AK](:, 0:K) * B[b][K][M]          (p = AK)
 *   variant 1: C[b][N][M]       = (A[b][K][AN](:, 0:N))^T * B[b][K][M]      (p = AN)
 *   variant 2: C[b][N][CM](:, 0:M) = A[b][N][K] * B[b][M][K]^T              (p = CM)
 * The f64 form also returns S = sum_k |a||b| (the scale of the forward error bound); padding columns of C
 * (variant 2) are set to zero in both.
 */
static inline size_t bmm_a(int v, int b, int i, int k, int N, int K, int p)
{
    return v == 1 ? ((size_t)b * K + k) * p + i : (v == 0 ? ((size_t)b * N + i) * p + k : ((size_t)b * N + i) * K + k);
}
static inline size_t bmm_b(int v, int b, int k, int j, int M, int K)
{
    return v == 2 ? ((size_t)b * M + j) * K + k : ((size_t)b * K + k) * M + j;
}
void oracle_bmm(const float *A, const float *B, float *C, int Batch, int N, int M, int K, int p, int variant)
{
    const int cm = variant == 2 ? p : M;
    memset(C, 0, sizeof(float) * (size_t)Batch * N * cm);
    for (int b = 0; b < Batch; b++)
        for (int k = 0; k < K; k++)
            for (int i = 0; i < N; i++) {
                const float a = A[bmm_a(variant, b, i, k, N, K, p)];
                for (int j = 0; j < M; j++)
                    C[((size_t)b * N + i) * cm + j] += a * B[bmm_b(variant, b, k, j, M, K)];
            }
}
void oracle_bmm_f64(const float *A, const float *B, double *C, double *S, int Batch, int N, int M, int K, int p,
                    int variant, int threads)
{
    const int cm = variant == 2 ? p : M;
    (void)threads;
    memset(C, 0, sizeof(double) * (size_t)Batch * N * cm);
    memset(S, 0, sizeof(double) * (size_t)Batch * N * cm);
#if defined(_OPENMP)
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
    for (int b = 0; b < Batch; b++)
        for (int i = 0; i < N; i++)
            for (int j = 0; j < M; j++) {
                double v = 0, sa = 0;
                for (int k = 0; k < K; k++) {
                    const double a = A[bmm_a(variant, b, i, k, N, K, p)], w = B[bmm_b(variant, b, k, j, M, K)];
                    v += a * w;
                    sa += fabs(a * w);
                }
                C[((size_t)b * N + i) * cm + j] = v;
                S[((size_t)b * N + i) * cm + j] = sa;
            }
}

/* ---- 2D pooling (TEST INFRASTRUCTURE) ---------------------------------------------------------------------------
 * Forward: the reference's CPU loops Pool2D_max_img2col / Pool2D_avg_img2col
 * (src/cu32_src/Cuda_pool2D/Cuda_pool2D/test.cuh:79-157; the average there divides by the number of window positions
 * inside the image = the ignore_padding variant); op 2 divides by FH * FW as pool2D_avg_kernel.cuh does, op 1 also
 * writes the index of pool2D_max_indexed_kernel.cuh:41-96 (offset into X of the winning element; among equal maxima
 * the last one in (fh, fw) order; 0 + image offset for a window without positions).
 *   op 0 max, 1 max + index, 2 avg, 3 avg ignoring padding.  X[N][IH][IW][IC], Y[N][OH][OW][IC].
 */
#define ORACLE_FLOAT_MIN (-3.4028234E38f)   /* Cuda_pool2D/micro.cuh:40 */
void oracle_pool2D(const float *X, float *Y, int *Index, int N, int IH, int IW, int IC, int FH, int FW, int OH, int OW,
                   int sh, int sw, int ph, int pw, int op)
{
    for (int n = 0; n < N; n++)
        for (int oh = 0; oh < OH; oh++)
            for (int ow = 0; ow < OW; ow++)
                for (int ic = 0; ic < IC; ic++) {
                    float v = op <= 1 ? ORACLE_FLOAT_MIN : 0.f;
                    int count = 0;
                    long long idx = 0;
                    for (int fh = 0; fh < FH; fh++)
                        for (int fw = 0; fw < FW; fw++) {
                            const int ih = oh * sh - ph + fh, iw = ow * sw - pw + fw;
                            if (ih < 0 || iw < 0 || ih >= IH || iw >= IW) continue;
                            const long long off = ((long long)ih * IW + iw) * IC + ic;
                            const float x = X[(long long)n * IH * IW * IC + off];
                            if (op <= 1) {
                                if (!(x < v)) idx = off;
                                if (v < x) v = x;
                            } else {
                                v += x;
                                count++;
                            }
                        }
                    if (op == 2) v = v / (float)(FH * FW);
                    if (op == 3) v = v / (float)count;
                    const long long yo = (((long long)n * OH + oh) * OW + ow) * IC + ic;
                    Y[yo] = v;
                    if (op == 1) Index[yo] = (int)(idx + (long long)n * IH * IW * IC);
                }
}

/* Backward: the reference's CPU loops unpool2D_max_img2col_plus / unpooling_avg_img2col_plus
 * (src/cu32_src/Cuda_upool2D/Cuda_upool2D/test.cuh:90-229): every input element sums, in ascending (oh, ow) order,
 * over the output windows that contain it.
 *   op 0 max:      deltaY where !(Y > X)                         (needs X, Y)
 *   op 1 indexed:  deltaY where Index == offset of the element   (upool2d_max_indexed_kernel.cuh:44-100)
 *   op 2 avg:      sum of alpha * deltaY, alpha = 1 / (FH * FW)  (upool2D_avg_kernel.cuh:84-94)
 *   op 3 avg ip:   sum of deltaY / (positions of that window inside the image)
 */
void oracle_upool2D(const float *deltaY, const float *Y, const float *X, const int *Index, float *deltaX, int N, int IH,
                    int IW, int IC, int FH, int FW, int OH, int OW, int sh, int sw, int ph, int pw, int op)
{
    for (int n = 0; n < N; n++)
        for (int ih = 0; ih < IH; ih++)
            for (int iw = 0; iw < IW; iw++)
                for (int ic = 0; ic < IC; ic++) {
                    const long long xo = (((long long)n * IH + ih) * IW + iw) * IC + ic;
                    const float alpha = 1.0f / (float)(FH * FW);
                    float v = 0.f;
                    for (int oh = 0; oh < OH; oh++) {
                        const int fh = ih - (oh * sh - ph);
                        if (fh < 0 || fh >= FH) continue;
                        for (int ow = 0; ow < OW; ow++) {
                            const int fw = iw - (ow * sw - pw);
                            if (fw < 0 || fw >= FW) continue;
                            const long long yo = (((long long)n * OH + oh) * OW + ow) * IC + ic;
                            if (op == 0) {
                                if (Y[yo] > X[xo]) continue;
                                v += deltaY[yo];
                            } else if (op == 1) {
                                if (Index[yo] == (int)xo) v += deltaY[yo];
                            } else if (op == 2) {
                                v += alpha * deltaY[yo];
                            } else {
                                int h0 = oh * sh - ph, h1 = h0 + FH, w0 = ow * sw - pw, w1 = w0 + FW;
                                if (h0 < 0) h0 = 0;
                                if (h1 > IH) h1 = IH;
                                if (w0 < 0) w0 = 0;
                                if (w1 > IW) w1 = IW;
                                v += deltaY[yo] / (float)((h1 - h0) * (w1 - w0));
                            }
                        }
                    }
                    deltaX[xo] = v;
                }
}
