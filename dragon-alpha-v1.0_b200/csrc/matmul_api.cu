// Matrix products of the FullConnect path behind the reference's Cuda_matMul natives, on the kernels of
// the convolution path: a matrix product is a 1x1 convolution over a "batch" of rows.
//   C = A * B^T  (matMulT2)  forward:  Y[row][oc] = sum_ic X[row][ic] * W[oc][ic]
//   C = A * B    (matMul)    deltaX:   dX[row][ic] = sum_oc dY[row][oc] * W[oc][ic]
//   C = A^T * B  (matMulT1)  deltaW:   dW[oc][ic] = sum_row dY[row][oc] * X[row][ic]
// so each form runs the tensor-core kernel (and every fallback) of the contraction it maps to.
// The batched products behind Cuda_batchMatMul run the same kernels with one image, and one set of weights, per
// batch entry; shapes those kernels do not take (reduction lengths that are not a multiple of 32, padded row
// pitches) run a plain fp32 kernel.
#include "../../include/alpha_conv_b200.h"
#include "host_common.h"

namespace alpha {
int launch_buf_summary(cudaStream_t stream, const float* buf, float* deltaW, int part, size_t sizeW);
void set_caller_scratch(void* ptr, size_t bytes);
int launch_bmm_tensor(int form, const float* A, const float* B, float* C, int Batch, int N, int M, int K, cudaStream_t stream);
}
using namespace alpha;

namespace {

// C[i][j] += bias[j]: the row-bias stage of matMul_biased (the reference runs linear_dual2D_row after
// the product, CudaFloat32EngineBase.java:1156-1165).
__global__ void add_bias_rows_kernel(float4* __restrict__ C, const float* __restrict__ bias, size_t n4, int cols4)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 c = C[i];
        const float4 b = *reinterpret_cast<const float4*>(bias + 4 * (i % cols4));
        c.x += b.x; c.y += b.y; c.z += b.z; c.w += b.w;
        C[i] = c;
    }
}

// `rows` matrix rows as the pixels of a 1x1 convolution: images of 1 x 4 pixels when the row count
// allows it (the engine pads every dimension to a multiple of 4), single pixels otherwise.  The
// kernels flatten 1x1 problems over all pixels anyway; the image shape only matters to their fallbacks.
AlphaConvShape rows_as_pixels(long long rows, int IC, int OC)
{
    AlphaConvShape s{};
    const int w = rows % 4 == 0 ? 4 : 1;
    s.N = static_cast<int>(rows / w);
    s.IH = s.OH = 1; s.IW = s.OW = w;
    s.IC = IC; s.OC = OC; s.FH = s.FW = 1; s.sh = s.sw = 1; s.ph = s.pw = 0;
    return s;
}

// C[b][i][j] = sum over k < K of a(b, i, k) * b(b, k, j) for i < N, j < M, every matrix with its own strides
// (element (i, k) of A[b] at A[b * a_b + i * a_i + k * a_k], and so on): the three batched forms with any row
// pitch.  Tiles of 64 x 64 outputs per CTA, 4 x 4 per thread, 16 reduction steps staged in shared memory at a
// time; k in ascending order, fp32 FMA - the arithmetic of the reference's kernels
// (Cuda_batch_matMul/Cuda_batchMatMul/batchMatMul_kernel.cuh), results do not depend on the launch.
struct BmmStrides { long long a_b, b_b, c_b; int a_i, a_k, b_k, b_j, c_i; };
__global__ void __launch_bounds__(256) bmm_simt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       float* __restrict__ C, int N, int M, int K, BmmStrides st)
{
    __shared__ float As[16][64 + 4], Bs[16][64 + 4];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    const float* a = A + static_cast<size_t>(blockIdx.z) * st.a_b;
    const float* b = B + static_cast<size_t>(blockIdx.z) * st.b_b;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = t + 256 * r;
            // consecutive threads walk the contiguous dimension of each matrix
            const int ai = st.a_k == 1 ? e >> 4 : e & 63, ak = st.a_k == 1 ? e & 15 : e >> 6;
            const int bj = st.b_j == 1 ? e & 63 : e >> 4, bk = st.b_j == 1 ? e >> 6 : e & 15;
            As[ak][ai] = (i0 + ai < N && k0 + ak < K) ? a[static_cast<size_t>(i0 + ai) * st.a_i + static_cast<size_t>(k0 + ak) * st.a_k] : 0.f;
            Bs[bk][bj] = (j0 + bj < M && k0 + bk < K) ? b[static_cast<size_t>(j0 + bj) * st.b_j + static_cast<size_t>(k0 + bk) * st.b_k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int y = 0; y < 4; ++y)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[y][x] = fmaf(ar[y], br[x], acc[y][x]);
        }
        __syncthreads();
    }
    float* c = C + static_cast<size_t>(blockIdx.z) * st.c_b;
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = i0 + ty * 4 + y, j = j0 + tx * 4 + x;
            if (i < N && j < M) c[static_cast<size_t>(i) * st.c_i + j] = acc[y][x];
        }
}

int launch_bmm_simt(const float* A, const float* B, float* C, int Batch, int N, int M, int K, const BmmStrides& st,
                    alpha_stream_t stream)
{
    for (int b0 = 0; b0 < Batch; b0 += 65535) {   // gridDim.z limit
        const int nb = Batch - b0 < 65535 ? Batch - b0 : 65535;
        dim3 grid((M + 63) / 64, (N + 63) / 64, nb);
        bmm_simt_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(A + b0 * st.a_b, B + b0 * st.b_b, C + b0 * st.c_b, N, M, K, st);
    }
    note_launch("bmm_simt");
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "bmm_simt_kernel launch failed: %s", cudaGetErrorString(e));
    return ALPHA_OK;
}

int check_batch(const char* what, const void* A, const void* B, const void* C, int Batch, int d0, int d1, int d2, int d3)
{
    if (!A || !B || !C) return fail(ALPHA_E_ARG, "%s: null matrix pointer", what);
    if (Batch <= 0 || d0 <= 0 || d1 <= 0 || d2 <= 0 || d3 <= 0)
        return fail(ALPHA_E_ARG, "%s: non-positive dimension (Batch=%d, %d %d %d %d)", what, Batch, d0, d1, d2, d3);
    return ALPHA_OK;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_dims(const char* what, const void* A, const void* B, const void* C, int N, int M, int K)
{
    if (!A || !B || !C) return fail(ALPHA_E_ARG, "%s: null matrix pointer", what);
    if (N <= 0 || M <= 0 || K <= 0) return fail(ALPHA_E_ARG, "%s: non-positive dimension (N=%d M=%d K=%d)", what, N, M, K);
    return ALPHA_OK;
}

inline alpha_stream_t first_stream(const int64_t* streams, int length)
{
    return (streams && length > 0) ? reinterpret_cast<alpha_stream_t>(static_cast<intptr_t>(streams[0])) : nullptr;
}

}  // namespace

extern "C" {

int alpha_matMul(const float* A, const float* B, const float* bias, float* C, int N, int M, int K, alpha_stream_t stream)
{
    int rc = check_dims("matMul", A, B, C, N, M, K);
    if (rc) return rc;
    if (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) return fail(ALPHA_E_ARG, "matMul: bias must be 16-byte aligned");
    // B[K][M] is W[OC = K][IC = M]; A[N][K] is deltaY; C[N][M] is deltaX
    AlphaConvShape s = rows_as_pixels(N, M, K);
    rc = alpha_conv3d_deltaX(&s, A, B, C, stream);
    if (rc || !bias) return rc;
    const size_t n4 = static_cast<size_t>(N) * M / 4;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    add_bias_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<float4*>(C), bias, n4, M / 4);
    note_launch("matmul_bias");
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "add_bias_rows_kernel launch failed: %s", cudaGetErrorString(e));
    return ALPHA_OK;
}

int alpha_matMulT1(const float* A, const float* B, float* C, int N, int M, int K, alpha_stream_t stream)
{
    int rc = check_dims("matMulT1", A, B, C, N, M, K);
    if (rc) return rc;
    // A[K][N] is deltaY[row][OC = N]; B[K][M] is X[row][IC = M]; C[N][M] is deltaW[OC][IC]
    AlphaConvShape s = rows_as_pixels(K, M, N);
    return alpha_conv3d_deltaW(&s, B, A, C, stream);
}

int alpha_matMulT2(const float* A, const float* B, const float* bias, float* C, int N, int M, int K, alpha_stream_t stream)
{
    int rc = check_dims("matMulT2", A, B, C, N, M, K);
    if (rc) return rc;
    // A[N][K] is X[row][IC = K]; B[M][K] is W[OC = M][IC = K]; C[N][M] is Y; the bias is fused into the epilogue
    AlphaConvShape s = rows_as_pixels(N, K, M);
    return alpha_conv3d_forward(&s, A, B, bias, C, stream);
}

// ---- batched products (src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/test.cuh:95-140 states the three forms) ----

// C[b][N][M] = A[b][N][AK] (first BK columns) * B[b][BK][M]
int alpha_batchMatMul(const float* A, const float* B, float* C, int Batch, int N, int M, int BK, int AK, alpha_stream_t stream)
{
    int rc = check_batch("batchMatMul", A, B, C, Batch, N, M, BK, AK);
    if (rc) return rc;
    if (AK < BK) return fail(ALPHA_E_ARG, "batchMatMul: row pitch of A (AK=%d) below the reduction length (BK=%d)", AK, BK);
    if (AK == BK && aligned16(A) && aligned16(B) && aligned16(C)) {
        rc = launch_bmm_tensor(0, A, B, C, Batch, N, M, BK, static_cast<cudaStream_t>(stream));
        if (rc != 1) return rc;
    }
    const BmmStrides st{(long long)N * AK, (long long)BK * M, (long long)N * M, AK, 1, M, 1, M};
    return launch_bmm_simt(A, B, C, Batch, N, M, BK, st, stream);
}

// C[b][CN][M] = A[b][K][AN]^T (first CN columns) * B[b][K][M]
int alpha_batchMatMulT1(const float* A, const float* B, float* C, int Batch, int CN, int AN, int M, int K, alpha_stream_t stream)
{
    int rc = check_batch("batchMatMulT1", A, B, C, Batch, CN, AN, M, K);
    if (rc) return rc;
    if (AN < CN) return fail(ALPHA_E_ARG, "batchMatMulT1: row pitch of A (AN=%d) below the rows of C (CN=%d)", AN, CN);
    if (AN == CN && aligned16(A) && aligned16(B) && aligned16(C)) {
        rc = launch_bmm_tensor(1, A, B, C, Batch, CN, M, K, static_cast<cudaStream_t>(stream));
        if (rc != 1) return rc;
    }
    const BmmStrides st{(long long)K * AN, (long long)K * M, (long long)CN * M, 1, AN, M, 1, M};
    return launch_bmm_simt(A, B, C, Batch, CN, M, K, st, stream);
}

// C[b][N][CM] (first BM columns) = A[b][N][K] * B[b][BM][K]^T
int alpha_batchMatMulT2(const float* A, const float* B, float* C, int Batch, int N, int CM, int BM, int K, alpha_stream_t stream)
{
    int rc = check_batch("batchMatMulT2", A, B, C, Batch, N, CM, BM, K);
    if (rc) return rc;
    if (CM < BM) return fail(ALPHA_E_ARG, "batchMatMulT2: row pitch of C (CM=%d) below its columns (BM=%d)", CM, BM);
    if (CM == BM && aligned16(A) && aligned16(B) && aligned16(C)) {
        rc = launch_bmm_tensor(2, A, B, C, Batch, N, BM, K, static_cast<cudaStream_t>(stream));
        if (rc != 1) return rc;
    }
    const BmmStrides st{(long long)N * K, (long long)BM * K, (long long)N * CM, K, 1, 1, K, CM};
    return launch_bmm_simt(A, B, C, Batch, N, BM, K, st, stream);
}

// ---- Cuda_batchMatMul natives (src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/A.cu:17-135) -------------
int alpha_Cuda_batchMatMul_batchMatMul(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N, int M, int BK, int AK)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_batchMatMul(A, B, C, Batch, N, M, BK, AK, first_stream(streams, length));
}
int alpha_Cuda_batchMatMul_batchMatMul_texture(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N, int M, int BK, int AK)
{
    return alpha_Cuda_batchMatMul_batchMatMul(streams, length, A, B, C, Batch, N, M, BK, AK);
}
int alpha_Cuda_batchMatMul_batchMatMulT1(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int CN, int AN, int M, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_batchMatMulT1(A, B, C, Batch, CN, AN, M, K, first_stream(streams, length));
}
int alpha_Cuda_batchMatMul_batchMatMulT2(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N, int CM, int BM, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_batchMatMulT2(A, B, C, Batch, N, CM, BM, K, first_stream(streams, length));
}
int alpha_Cuda_batchMatMul_batchMatMulT2_texture(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N, int CM, int BM, int K)
{
    return alpha_Cuda_batchMatMul_batchMatMulT2(streams, length, A, B, C, Batch, N, CM, BM, K);
}

// ---- Cuda_matMul natives (src/cu32_src/Cuda_matMul/Cuda_matMul/A.cu:18-120) --------------------------

int alpha_Cuda_matMul_matMul(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_matMul(A, B, nullptr, C, N, M, K, first_stream(streams, length));
}
int alpha_Cuda_matMul_matMulT1(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_matMulT1(A, B, C, N, M, K, first_stream(streams, length));
}
// Split-K entry: the complete product goes to C, the caller's (GridZ - 1) * N * M floats of Cbuf serve as
// scratch and are left zero, so that the SKbuf_summary the engine runs next (C += sum of buffers) adds zeros.
int alpha_Cuda_matMul_matMulT1SK(const int64_t* streams, int length, int GridZ, float* A, float* B, float* C, float* Cbuf,
                                 int N, int M, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    if (GridZ > 1 && !Cbuf) return fail(ALPHA_E_ARG, "GridZ=%d but Cbuf is null", GridZ);
    const size_t bytes = GridZ > 1 ? static_cast<size_t>(GridZ - 1) * N * M * sizeof(float) : 0;
    if (bytes && (reinterpret_cast<uintptr_t>(Cbuf) & 255) == 0) set_caller_scratch(Cbuf, bytes);
    const int rc = alpha_matMulT1(A, B, C, N, M, K, first_stream(streams, length));
    set_caller_scratch(nullptr, 0);
    if (rc) return rc;
    if (bytes) {
        cudaError_t e = cudaMemsetAsync(Cbuf, 0, bytes, static_cast<cudaStream_t>(first_stream(streams, length)));
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemsetAsync(Cbuf): %s", cudaGetErrorString(e));
    }
    return ALPHA_OK;
}
int alpha_Cuda_matMul_matMulT2(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    return alpha_matMulT2(A, B, nullptr, C, N, M, K, first_stream(streams, length));
}
int alpha_Cuda_matMul_SKbuf_summary(int64_t stream, float* Cbuf, float* C, int part, int sizeC)
{
    if (part < 0 || sizeC <= 0 || (sizeC & 3) || !C || (part > 0 && !Cbuf))
        return fail(ALPHA_E_ARG, "bad SKbuf_summary arguments (part=%d sizeC=%d)", part, sizeC);
    if (part == 0) return ALPHA_OK;
    return launch_buf_summary(reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream)), Cbuf, C, part, static_cast<size_t>(sizeC));
}

// ---- CudaFloat32EngineBase operator methods (CudaFloat32EngineBase.java:1129-1245) -------------------

int alpha_engine_matMul(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream)
{
    return alpha_matMul(A, B, nullptr, C, N, M, K, stream);
}
int alpha_engine_matMul_biased(float* C, const float* A, const float* B, int N, int M, int K, const float* Bias, alpha_stream_t stream)
{
    if (!Bias) return fail(ALPHA_E_ARG, "matMul_biased needs a bias vector");
    return alpha_matMul(A, B, Bias, C, N, M, K, stream);
}
int alpha_engine_matMulT1(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream)
{
    return alpha_matMulT1(A, B, C, N, M, K, stream);
}
int alpha_engine_matMulT2(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream)
{
    return alpha_matMulT2(A, B, nullptr, C, N, M, K, stream);
}

// CudaFloat32EngineBase.java:1256-1318
int alpha_engine_batchMatMul(float* C, const float* A, const float* B, int Batch, int N, int M, int BK, int AK, alpha_stream_t stream)
{
    return alpha_batchMatMul(A, B, C, Batch, N, M, BK, AK, stream);
}
int alpha_engine_batchMatMulT1(float* C, const float* A, const float* B, int Batch, int CN, int AN, int M, int K, alpha_stream_t stream)
{
    return alpha_batchMatMulT1(A, B, C, Batch, CN, AN, M, K, stream);
}
int alpha_engine_batchMatMulT2(float* C, const float* A, const float* B, int Batch, int N, int CM, int BM, int K, alpha_stream_t stream)
{
    return alpha_batchMatMulT2(A, B, C, Batch, N, CM, BM, K, stream);
}

}  // extern "C"
