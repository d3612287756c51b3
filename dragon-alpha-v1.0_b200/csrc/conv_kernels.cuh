// Device kernels of the conv hot path for sm_100a.
//
//   conv_igemm_kernel   forward conv and stride-1 deltaX as an implicit GEMM:
//                       D[128 pixels][BN channels] += im2col(act)[128][K] * Wt[BN][K]
//                       A tiles come from an im2col-mode TMA of the NHWC activation tensor, B tiles
//                       from a tiled TMA of W[OC,FH,FW,IC]; tcgen05.mma kind::tf32 accumulates in
//                       tensor memory; 3xTF32 splits each staged tile into hi/lo planes.
//   conv_dw_kernel      deltaW as a split-K GEMM whose K axis is the pixel axis; both operands are
//                       MN-major (channels contiguous), several accumulators per CTA.
//   dw_reduce_kernel    fixed-order (deterministic) compensated sum of the split-K partials.
//   *_simt kernels      plain fp32 kernels for shapes the tensor path does not take (channel counts
//                       that are not a multiple of 8, strided deltaX); they keep the library
//                       complete on the GPU, there is no CPU path.
#pragma once
#include "sm100_ptx.cuh"
#include "fast_div.cuh"

namespace alpha {

constexpr int kBM = 128;           // GEMM M tile = tensor-memory lanes
constexpr int kIgemmThreads = 192;  // warp 0: TMA, warp 1: MMA, warps 2-5: split + epilogue

enum KernelStatus : int {
    kStatusOk = 0,
    kStatusProducerTimeout = 1,
    kStatusMmaTimeout = 2,
    kStatusSplitTimeout = 3,
    kStatusEpilogueTimeout = 4,
};

// The reference's LeakyReLU, x * ((x > 0) + k * (x < 0)) (Cuda_function/type4_leakyRelu2D.cuh:32);
// k = 0 is ReLU.  Applied after the bias in the forward epilogues when a plan asks for it.
__device__ __forceinline__ float leaky_relu(float x, float k) { return x > 0.f ? x : k * x; }
__device__ __forceinline__ void leaky_relu4(float4& v, float k)
{
    v.x = leaky_relu(v.x, k); v.y = leaky_relu(v.y, k); v.z = leaky_relu(v.z, k); v.w = leaky_relu(v.w, k);
}

struct IgemmParams {
    float* out;         // [M_total][ldo]
    const float* bias;  // [Ncols] or nullptr
    int act_on;         // 1: LeakyReLU with slope act_k after the bias
    float act_k;
    int* status;        // device status word, 0 = ok
    int M_total;        // output pixels
    int Ncols;          // output channels
    int ldo;            // row stride of out in floats
    int OHo, OWo;       // output spatial extent (pixel -> coordinates)
    int sh, sw, ph, pw; // base pixel coordinate = (q*sw - pw, p*sh - ph)
    int FH, FW;
    int kchunks;        // channel chunks per filter tap
    int KC;             // reduction channels per chunk: 32, 16 or 8
    int BN;             // N tile, multiple of 16 (of 32 when b_mn)
    int stages;
    int mode3x;         // 1: 3xTF32 split, 0: plain TF32
    int b_mn;           // 1: B operand is MN-major (deltaX reads W[oc][tap][ic] in place)
    int flip;           // 1: B uses the 180-degree rotated tap
    uint32_t tmem_cols;
    uint32_t idesc;
    uint32_t a_bytes;   // bytes of one A plane per stage
    uint32_t b_bytes;   // bytes of one B plane per stage (rounded up to 1024)
    uint32_t b_tx;      // bytes the B loads of one stage deliver
    uint32_t swz;       // descriptor layout type of the K-major operands
};

__device__ __forceinline__ void report(int* status, int code)
{
    if (status) atomicCAS(status, 0, code);
}

// Round to TF32 (10 explicit mantissa bits), nearest with ties away from zero: add half a TF32 ulp
// to the magnitude and clear the 13 low bits.  Two full-rate integer instructions; the dedicated
// conversion instruction (cvt.rna.tf32.f32) runs at a fraction of that rate and made the operand
// split the slowest stage of the 3xTF32 kernels.
__device__ __forceinline__ uint32_t to_tf32_rna(float x)
{
    return (__float_as_uint(x) + 0x1000u) & 0xFFFFE000u;
}

// hi = tf32(x), lo = tf32(x - hi): x = hi + lo up to 2^-22 |x|.
__device__ __forceinline__ void split_tf32(float4& hi, float4& lo)
{
    float4 x = hi;
    hi.x = __uint_as_float(to_tf32_rna(x.x));
    hi.y = __uint_as_float(to_tf32_rna(x.y));
    hi.z = __uint_as_float(to_tf32_rna(x.z));
    hi.w = __uint_as_float(to_tf32_rna(x.w));
    lo.x = __uint_as_float(to_tf32_rna(x.x - hi.x));
    lo.y = __uint_as_float(to_tf32_rna(x.y - hi.y));
    lo.z = __uint_as_float(to_tf32_rna(x.z - hi.z));
    lo.w = __uint_as_float(to_tf32_rna(x.w - hi.w));
}

// Rewrites one staged plane in place as its hi part and fills the lo plane; 128 threads.
__device__ __forceinline__ void split_plane(uint8_t* hi_plane, uint8_t* lo_plane, uint32_t bytes,
                                            int tid128)
{
    float4* h = reinterpret_cast<float4*>(hi_plane);
    float4* l = reinterpret_cast<float4*>(lo_plane);
    const uint32_t nvec = bytes >> 4;
    for (uint32_t v = tid128; v < nvec; v += 128) {
        float4 a = h[v], b;
        split_tf32(a, b);
        h[v] = a;
        l[v] = b;
    }
}

// Same, four vectors per thread in flight so that the shared-memory latencies overlap.
__device__ __forceinline__ void split_plane_x4(uint8_t* hi_plane, uint8_t* lo_plane, uint32_t bytes, int tid, int nthreads)
{
    float4* h = reinterpret_cast<float4*>(hi_plane);
    float4* l = reinterpret_cast<float4*>(lo_plane);
    const uint32_t nvec = bytes >> 4, n = nthreads;
    uint32_t v = tid;
    for (; v + 3 * n < nvec; v += 4 * n) {
        float4 a0 = h[v], a1 = h[v + n], a2 = h[v + 2 * n], a3 = h[v + 3 * n], b0, b1, b2, b3;
        split_tf32(a0, b0); split_tf32(a1, b1); split_tf32(a2, b2); split_tf32(a3, b3);
        h[v] = a0; h[v + n] = a1; h[v + 2 * n] = a2; h[v + 3 * n] = a3;
        l[v] = b0; l[v + n] = b1; l[v + 2 * n] = b2; l[v + 3 * n] = b3;
    }
    for (; v < nvec; v += n) {
        float4 a = h[v], b;
        split_tf32(a, b);
        h[v] = a;
        l[v] = b;
    }
}

// tcgen05.mma kind::tf32 reads only the upper 19 bits of each fp32 operand word, so a staged fp32
// plane already acts as hi = x with the low 13 mantissa bits cleared, and only lo = tf32(x - hi)
// has to be written: one shared-memory store per vector instead of two.
__device__ __forceinline__ float tf32_lo_of_trunc(float x)
{
    const float hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    return __uint_as_float(to_tf32_rna(x - hi));
}

__device__ __forceinline__ float4 tf32_lo_of_trunc(const float4& x)
{
    return make_float4(tf32_lo_of_trunc(x.x), tf32_lo_of_trunc(x.y), tf32_lo_of_trunc(x.z), tf32_lo_of_trunc(x.w));
}

// Fills the lo plane of a staged plane that stays as it is; four vectors per thread in flight.
__device__ __forceinline__ void split_plane_lo_x4(const uint8_t* plane, uint8_t* lo_plane, uint32_t bytes, int tid, int nthreads)
{
    const float4* h = reinterpret_cast<const float4*>(plane);
    float4* l = reinterpret_cast<float4*>(lo_plane);
    const uint32_t nvec = bytes >> 4, n = nthreads;
    uint32_t v = tid;
    for (; v + 3 * n < nvec; v += 4 * n) {
        const float4 a0 = h[v], a1 = h[v + n], a2 = h[v + 2 * n], a3 = h[v + 3 * n];
        l[v] = tf32_lo_of_trunc(a0); l[v + n] = tf32_lo_of_trunc(a1);
        l[v + 2 * n] = tf32_lo_of_trunc(a2); l[v + 3 * n] = tf32_lo_of_trunc(a3);
    }
    for (; v < nvec; v += n) l[v] = tf32_lo_of_trunc(h[v]);
}

// Patch matrix of a convolution for channel counts the tensor kernels cannot stage directly:
// A[m][k] with m = (n, oh, ow), k = (fh * FW + fw) * IC + ic < K, zero for K <= k < Kp and outside
// the image.  One thread per four consecutive k (IC is a multiple of 4, so they share a pixel).
struct PatchShape {
    int N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw, K, Kp;
};

__global__ void __launch_bounds__(256) patch_matrix_kernel(const float* __restrict__ X, float* __restrict__ A, const PatchShape s)
{
    const int k4n = s.Kp >> 2;
    const size_t total = static_cast<size_t>(s.N) * s.OH * s.OW * k4n;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t m = i / k4n;
        const int k = static_cast<int>(i - m * k4n) << 2;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < s.K) {
            const int tap = k / s.IC, ic = k - tap * s.IC;
            const int fh = tap / s.FW, fw = tap - fh * s.FW;
            const int ow = static_cast<int>(m % s.OW);
            const size_t t = m / s.OW;
            const int oh = static_cast<int>(t % s.OH);
            const size_t n = t / s.OH;
            const int ih = oh * s.sh - s.ph + fh, iw = ow * s.sw - s.pw + fw;
            if (ih >= 0 && ih < s.IH && iw >= 0 && iw < s.IW)
                v = __ldg(reinterpret_cast<const float4*>(X + ((n * s.IH + ih) * s.IW + iw) * s.IC + ic));
        }
        reinterpret_cast<float4*>(A)[i] = v;
    }
}

// The same for matrices and tensors of fewer than 2^31 elements: 32-bit indices, divisions as multiplications
// (the kernel is a gather of 16-byte pieces; five divisions per piece, three of them 64-bit, cost more than the loads).
struct PatchDivs {
    FastDiv by_k4n, by_IC, by_FW, by_OW, by_OH;
};
__global__ void __launch_bounds__(256) patch_matrix32_kernel(const float* __restrict__ X, float* __restrict__ A, const PatchShape s,
                                                             const PatchDivs dv)
{
    const unsigned k4n = static_cast<unsigned>(s.Kp) >> 2;
    const unsigned total = static_cast<unsigned>(s.N) * s.OH * s.OW * k4n;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        unsigned m, k4;
        dv.by_k4n.divmod(i, m, k4);
        const unsigned k = k4 << 2;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < static_cast<unsigned>(s.K)) {
            unsigned tap, ic, fh, fw, t, ow, n, oh;
            dv.by_IC.divmod(k, tap, ic);
            dv.by_FW.divmod(tap, fh, fw);
            dv.by_OW.divmod(m, t, ow);
            dv.by_OH.divmod(t, n, oh);
            const int ih = static_cast<int>(oh) * s.sh - s.ph + static_cast<int>(fh), iw = static_cast<int>(ow) * s.sw - s.pw + static_cast<int>(fw);
            if (ih >= 0 && ih < s.IH && iw >= 0 && iw < s.IW)
                v = __ldg(reinterpret_cast<const float4*>(X + static_cast<size_t>((n * s.IH + ih) * s.IW + iw) * s.IC + ic));
        }
        reinterpret_cast<float4*>(A)[i] = v;
    }
}

// dst[r][0..K) = src[r][0..K) of a matrix with row pitch Kp (drops the zero padding columns).
__global__ void __launch_bounds__(256) unpad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int K, int Kp)
{
    const int k4n = K >> 2;
    const size_t total = static_cast<size_t>(rows) * k4n;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / k4n;
        const int k = static_cast<int>(i - r * k4n) << 2;
        reinterpret_cast<float4*>(dst)[i] = *reinterpret_cast<const float4*>(src + r * Kp + k);
    }
}

// dst[n][sh*a + py][sw*b + px][:] = src[(n*A + a)*B + b][:]: one stride phase of deltaX, computed
// densely, placed on its pixels.  dst already points at pixel (py, px) of image 0.
__global__ void __launch_bounds__(256) scatter_phase_kernel(const float* __restrict__ src, float* __restrict__ dst, int N, int A,
                                                            int B, int C, int sh, int sw, int IH, int IW)
{
    const int c4n = C >> 2;
    const size_t total = static_cast<size_t>(N) * A * B * c4n;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t m = i / c4n;
        const int c = static_cast<int>(i - m * c4n) << 2;
        const int b = static_cast<int>(m % B);
        const size_t t = m / B;
        const int a = static_cast<int>(t % A);
        const size_t n = t / A;
        *reinterpret_cast<float4*>(dst + ((n * IH + static_cast<size_t>(a) * sh) * IW + static_cast<size_t>(b) * sw) * C + c) =
            reinterpret_cast<const float4*>(src)[i];
    }
}

// col2im of a deltaX with few input channels: P[(n, oh, ow)][ic * taps + fh * FW + fw] holds the
// contribution of output pixel (oh, ow) to input pixel (oh*sh - ph + fh, ow*sw - pw + fw); every
// input pixel gathers its (at most ceil(FH/sh) * ceil(FW/sw)) contributions in a fixed order.
// One thread per four input channels.
__global__ void __launch_bounds__(256) col2im_gather_kernel(const float* __restrict__ P, float* __restrict__ dX, const PatchShape s)
{
    const int c4n = s.IC >> 2, taps = s.FH * s.FW, ldp = s.IC * taps;
    const size_t total = static_cast<size_t>(s.N) * s.IH * s.IW * c4n;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c0 = static_cast<int>(i % c4n) << 2;
        size_t t = i / c4n;
        const int iw = static_cast<int>(t % s.IW); t /= s.IW;
        const int ih = static_cast<int>(t % s.IH);
        const size_t n = t / s.IH;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int fh = (ih + s.ph) % s.sh; fh < s.FH; fh += s.sh) {
            const int oh = (ih + s.ph - fh) / s.sh;
            if (ih + s.ph - fh < 0 || oh >= s.OH) continue;
            for (int fw = (iw + s.pw) % s.sw; fw < s.FW; fw += s.sw) {
                const int ow = (iw + s.pw - fw) / s.sw;
                if (iw + s.pw - fw < 0 || ow >= s.OW) continue;
                const float* row = P + ((n * s.OH + oh) * s.OW + ow) * ldp + fh * s.FW + fw;
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[q] += __ldg(row + (c0 + q) * taps);
            }
        }
        *reinterpret_cast<float4*>(dX + i * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
}

// The same gather for any channel count, with P laid out tap-major: P[pixel][tap][ic], so that the
// threads of a warp read neighbouring channels.  One thread per four input channels.
__global__ void __launch_bounds__(256) col2im_gather_tapmajor_kernel(const float* __restrict__ P, float* __restrict__ dX, const PatchShape s)
{
    const int c4n = s.IC >> 2, taps = s.FH * s.FW;
    const size_t ldp = static_cast<size_t>(s.IC) * taps;
    const size_t total = static_cast<size_t>(s.N) * s.IH * s.IW * c4n;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c0 = static_cast<int>(i % c4n) << 2;
        size_t t = i / c4n;
        const int iw = static_cast<int>(t % s.IW); t /= s.IW;
        const int ih = static_cast<int>(t % s.IH);
        const size_t n = t / s.IH;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int fh = (ih + s.ph) % s.sh; fh < s.FH; fh += s.sh) {
            const int oh = (ih + s.ph - fh) / s.sh;
            if (ih + s.ph - fh < 0 || oh >= s.OH) continue;
            for (int fw = (iw + s.pw) % s.sw; fw < s.FW; fw += s.sw) {
                const int ow = (iw + s.pw - fw) / s.sw;
                if (iw + s.pw - fw < 0 || ow >= s.OW) continue;
                const float4 v = __ldg(reinterpret_cast<const float4*>(
                    P + ((n * s.OH + oh) * s.OW + ow) * ldp + static_cast<size_t>(fh * s.FW + fw) * s.IC + c0));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        *reinterpret_cast<float4*>(dX + i * 4) = acc;
    }
}

// The same gather for tensors of fewer than 2^31 elements, the common case: 32-bit index arithmetic with the
// divisions by tensor extents as multiplications, and no division inside the tap loops (the output row of the
// k-th tap of a phase is floor((ih + ph) / sh) - k).  The 64-bit kernel above spent more time on its divisions
// than on its loads (2.2 TB/s on a 1x1 stride-2 deltaX).
struct GatherDivs {
    FastDiv by_c4n, by_IW, by_IH, by_sh, by_sw;
};
__global__ void __launch_bounds__(256) col2im_gather_tapmajor32_kernel(const float* __restrict__ P, float* __restrict__ dX, const PatchShape s,
                                                                         const GatherDivs dv)
{
    const unsigned c4n = static_cast<unsigned>(s.IC) >> 2;
    const unsigned ldp = static_cast<unsigned>(s.IC) * s.FH * s.FW;
    const unsigned total = static_cast<unsigned>(s.N) * s.IH * s.IW * c4n;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        unsigned t, c4, iw, ih, n;
        dv.by_c4n.divmod(i, t, c4);
        dv.by_IW.divmod(t, t, iw);
        dv.by_IH.divmod(t, n, ih);
        unsigned qh, fh0, qw, fw0;
        dv.by_sh.divmod(ih + s.ph, qh, fh0);
        dv.by_sw.divmod(iw + s.pw, qw, fw0);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int oh = static_cast<int>(qh);
        for (int fh = static_cast<int>(fh0); fh < s.FH && oh >= 0; fh += s.sh, --oh) {
            if (oh >= s.OH) continue;
            const float* prow = P + static_cast<size_t>((n * s.OH + oh) * s.OW) * ldp + (c4 << 2);
            int ow = static_cast<int>(qw);
            for (int fw = static_cast<int>(fw0); fw < s.FW && ow >= 0; fw += s.sw, --ow) {
                if (ow >= s.OW) continue;
                const float4 v = __ldg(reinterpret_cast<const float4*>(prow + static_cast<size_t>(ow) * ldp + (fh * s.FW + fw) * s.IC));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        *reinterpret_cast<float4*>(dX + static_cast<size_t>(i) * 4) = acc;
    }
}

// The channel-major gather (image planes, P[pixel][ic][tap]) with 32-bit indices and divisions as multiplications.
__global__ void __launch_bounds__(256) col2im_gather32_kernel(const float* __restrict__ P, float* __restrict__ dX, const PatchShape s,
                                                              const GatherDivs dv)
{
    const unsigned c4n = static_cast<unsigned>(s.IC) >> 2;
    const unsigned taps = static_cast<unsigned>(s.FH) * s.FW, ldp = static_cast<unsigned>(s.IC) * taps;
    const unsigned total = static_cast<unsigned>(s.N) * s.IH * s.IW * c4n;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        unsigned t, c4, iw, ih, n;
        dv.by_c4n.divmod(i, t, c4);
        dv.by_IW.divmod(t, t, iw);
        dv.by_IH.divmod(t, n, ih);
        unsigned qh, fh0, qw, fw0;
        dv.by_sh.divmod(ih + s.ph, qh, fh0);
        dv.by_sw.divmod(iw + s.pw, qw, fw0);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int oh = static_cast<int>(qh);
        for (int fh = static_cast<int>(fh0); fh < s.FH && oh >= 0; fh += s.sh, --oh) {
            if (oh >= s.OH) continue;
            const float* prow = P + static_cast<size_t>((n * s.OH + oh) * s.OW) * ldp + (c4 << 2) * taps;
            int ow = static_cast<int>(qw);
            for (int fw = static_cast<int>(fw0); fw < s.FW && ow >= 0; fw += s.sw, --ow) {
                if (ow >= s.OW) continue;
                const float* row = prow + static_cast<size_t>(ow) * ldp + fh * s.FW + fw;
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[q] += __ldg(row + q * taps);
            }
        }
        *reinterpret_cast<float4*>(dX + static_cast<size_t>(i) * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
}

// hi/lo planes of a whole tensor in global memory (weights are split once per call, not per tile).
__global__ void split_tensor_kernel(const float4* __restrict__ src, float4* __restrict__ hi, float4* __restrict__ lo, size_t n4)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 a = src[i], b;
        split_tf32(a, b);
        hi[i] = a;
        lo[i] = b;
    }
}

// out = sum of `splits` partial results of n4 float4 each (+ bias per column, + LeakyReLU): the tail of a
// split-K forward / deltaX launch.  Partials are added in index order, so the result does not depend
// on how the CTAs were scheduled.
__global__ void splitk_reduce_kernel(const float4* __restrict__ part, size_t n4, int splits, const float* __restrict__ bias,
                                     int ncols4, int act_on, float act_k, float4* __restrict__ out)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 a = part[i];
        for (int s = 1; s < splits; ++s) {
            const float4 b = part[static_cast<size_t>(s) * n4 + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (bias) {
            const float4 b = *reinterpret_cast<const float4*>(bias + 4 * (i % ncols4));
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (act_on) leaky_relu4(a, act_k);
        out[i] = a;
    }
}

// lo plane of a tensor whose fp32 words serve as the hi plane where they lie (the tensor core reads
// only the upper 19 bits of an operand word): lo = tf32(x - trunc19(x)).
__global__ void split_lo_kernel(const float4* __restrict__ src, float4* __restrict__ lo, size_t n4)
{
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float4 a = src[i];
        lo[i] = make_float4(tf32_lo_of_trunc(a.x), tf32_lo_of_trunc(a.y), tf32_lo_of_trunc(a.z), tf32_lo_of_trunc(a.w));
    }
}

// Source filter taps of a transposed weight tensor: output tap t reads W[.][src[t]][.].
struct TapMap {
    int n;
    int src[64];
};

// Wt[ic][t][oc] = W[oc][map.src[t]][ic]: the weights of deltaX seen as a forward convolution over
// deltaY (channels swapped; the tap list rotates the filter by 180 degrees and, for strided
// convolutions, picks the sub-filter of one output phase), written as hi (and, when `split`, lo) TF32
// planes.  32 x 32 tiles through shared memory; grid (ceil(IC/32), ceil(OC/32), map.n).
__global__ void __launch_bounds__(256)
    transpose_weights_kernel(const float* __restrict__ W, float* __restrict__ hi, float* __restrict__ lo, int OC,
                             int IC, int taps, const TapMap map, int split, int tap_major = 0)
{
    __shared__ float tile[32][33];
    const int t = blockIdx.z, tap = map.src[t], ic0 = blockIdx.x * 32, oc0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int oc = oc0 + r, ic = ic0 + tx;
        tile[r][tx] = (oc < OC && ic < IC) ? W[(static_cast<size_t>(oc) * taps + tap) * IC + ic] : 0.f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int ic = ic0 + r, oc = oc0 + tx;
        if (ic < IC && oc < OC) {
            const float x = tile[tx][r];
            // rows of Wt ordered (ic, tap), or (tap, ic) when tap_major
            const size_t o = tap_major ? (static_cast<size_t>(t) * IC + ic) * OC + oc
                                       : (static_cast<size_t>(ic) * map.n + t) * OC + oc;
            if (split) {
                const float h = __uint_as_float(to_tf32_rna(x));
                hi[o] = h;
                lo[o] = __uint_as_float(to_tf32_rna(x - h));
            } else {
                hi[o] = x;
            }
        }
    }
}

__global__ void __launch_bounds__(kIgemmThreads)
    conv_igemm_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const IgemmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.x, tile_n = blockIdx.y;
    const int S = p.stages;
    const uint32_t planes = p.mode3x ? 2u : 1u;
    const uint32_t stage_bytes = (p.a_bytes + p.b_bytes) * planes;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S) * stage_bytes);
    uint64_t* full = bars;
    uint64_t* split_done = bars + S;
    uint64_t* empty = bars + 2 * S;
    uint64_t* accum = bars + 3 * S;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 3 * S + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&split_done[s], 128);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int num_it = p.FH * p.FW * p.kchunks;
    const int m0 = tile_m * kBM;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            const int hw = p.OHo * p.OWo;
            const int n_img = m0 / hw;
            const int rem = m0 - n_img * hw;
            const int pr = rem / p.OWo, qc = rem - pr * p.OWo;
            const int w0 = qc * p.sw - p.pw, h0 = pr * p.sh - p.ph;
            const int taps = p.FH * p.FW;
            const uint32_t smem_a = smem_u32(smem), full_a = smem_u32(full), empty_a = smem_u32(empty);
            RingPos rp;
            bool ok = true;
            int tap = 0;
            for (int fh = 0; fh < p.FH && ok; ++fh)
                for (int fw = 0; fw < p.FW && ok; ++fw, ++tap)
                    for (int kc = 0; kc < p.kchunks; ++kc) {
                        if (!mbar_wait_a(empty_a + 8 * rp.idx, rp.phase ^ 1)) { report(p.status, kStatusProducerTimeout); ok = false; break; }
                        const uint32_t a_dst = smem_a + rp.idx * stage_bytes;
                        const uint32_t b_dst = a_dst + p.a_bytes * planes;
                        const uint32_t bar = full_a + 8 * rp.idx;
                        mbar_arrive_expect_tx_a(bar, p.a_bytes + p.b_tx);
                        tma_load_im2col_4d_a(a_dst, &tmA, bar, kc * p.KC, w0, h0, n_img,
                                             static_cast<uint16_t>(fw), static_cast<uint16_t>(fh));
                        if (!p.b_mn) {
                            tma_load_3d_a(b_dst, &tmB, bar, kc * p.KC, tap, tile_n * p.BN);
                        } else {
                            const int tapw = p.flip ? (taps - 1 - tap) : tap;
                            for (int j = 0; j < p.BN / 32; ++j)
                                tma_load_3d_a(b_dst + j * (p.KC * 128), &tmB, bar, tile_n * p.BN + j * 32, tapw, kc * p.KC);
                        }
                        rp.advance(S);
                    }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            const uint32_t sbo_k = 8 * p.KC * 4;  // 8 rows of KC floats
            const uint32_t a_dhi = smem_desc_hi(sbo_k, p.swz);
            const uint32_t b_dhi = p.b_mn ? smem_desc_hi(512, kSwizzle128B_Base32B) : smem_desc_hi(sbo_k, p.swz);
            const uint32_t b_lbo = p.b_mn ? p.KC * 128u : 16u;
            const uint32_t b_kstep = p.b_mn ? 64u : 2u;
            const uint32_t a_lo_off = p.a_bytes >> 4, b_lo_off = p.b_bytes >> 4;
            const uint32_t wait_a = smem_u32(p.mode3x ? split_done : full), empty_a = smem_u32(empty);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem) + p.a_bytes * planes, b_lbo);
            const uint32_t stage16 = stage_bytes >> 4;
            const int ksteps = p.KC / 8;
            RingPos rp;
            uint32_t acc = 0u;
            for (int it = 0; it < num_it; ++it) {
                if (!mbar_wait_a(wait_a + 8 * rp.idx, rp.phase)) { report(p.status, kStatusMmaTimeout); break; }
                tc_fence_after_sync();
                const uint32_t al = a_lo0 + rp.idx * stage16, bl = b_lo0 + rp.idx * stage16;
                // the math-mode test stays outside the K steps: a branch between two MMAs costs the
                // issuing thread about as much as an MMA
                if (p.mode3x) {
                    for (int kk = 0; kk < ksteps; ++kk, acc = 1u) {
                        const uint32_t a_k = al + kk * 2, b_k = bl + kk * b_kstep;
                        mma_tf32_ss2(tmem_base, a_k + a_lo_off, a_dhi, b_k, b_dhi, p.idesc, acc);
                        mma_tf32_ss2(tmem_base, a_k, a_dhi, b_k + b_lo_off, b_dhi, p.idesc, 1u);
                        mma_tf32_ss2(tmem_base, a_k, a_dhi, b_k, b_dhi, p.idesc, 1u);
                    }
                } else {
                    for (int kk = 0; kk < ksteps; ++kk, acc = 1u)
                        mma_tf32_ss2(tmem_base, al + kk * 2, a_dhi, bl + kk * b_kstep, b_dhi, p.idesc, acc);
                }
                mma_commit_a(empty_a + 8 * rp.idx);
                rp.advance(S);
            }
            mma_commit(accum);
        }
        __syncwarp();
    } else {
        // ---- operand split (3xTF32) and epilogue: warps 2..5 ----
        const int tid128 = threadIdx.x - 64;
        bool ok = true;
        if (p.mode3x) {
            const uint32_t full_a = smem_u32(full), done_a = smem_u32(split_done);
            RingPos rp;
            for (int it = 0; it < num_it; ++it) {
                if (!mbar_wait_a(full_a + 8 * rp.idx, rp.phase)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                uint8_t* a_hi = smem + static_cast<size_t>(rp.idx) * stage_bytes;
                uint8_t* b_hi = a_hi + p.a_bytes * 2;
                split_plane_x4(a_hi, a_hi + p.a_bytes, p.a_bytes, tid128, 128);
                split_plane_x4(b_hi, b_hi + p.b_bytes, p.b_tx, tid128, 128);
                fence_proxy_async_smem();
                mbar_arrive_a(done_a + 8 * rp.idx);
                rp.advance(S);
            }
        }
        if (ok && !mbar_wait(accum, 0)) { report(p.status, kStatusEpilogueTimeout); ok = false; }
        tc_fence_after_sync();
        if (ok) {
            const int quad = warp & 3;
            const int row = quad * 32 + lane;
            const long long m = static_cast<long long>(m0) + row;
            float* orow = p.out + m * p.ldo;
            const int n0 = tile_n * p.BN;
            for (int c = 0; c < p.BN; c += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c, r);
                tmem_ld_wait();
                if (m < p.M_total) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int col = n0 + c + j;
                        if (c + j < p.BN && col < p.Ncols) {
                            float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                   __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                            if (p.bias) {
                                const float4 b = *reinterpret_cast<const float4*>(p.bias + col);
                                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                            }
                            if (p.act_on) leaky_relu4(v, p.act_k);
                            *reinterpret_cast<float4*>(orow + col) = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

// ---------------------------------------------------------------------------------------------
// deltaW
// ---------------------------------------------------------------------------------------------

struct DwParams {
    float* out;           // deltaW, or the partial buffer when splits > 1
    size_t split_stride;  // floats between the partials of two splits
    int* status;
    int Npix;             // N*OH*OW, the reduction extent
    int OHo, OWo, sh, sw, ph, pw, FH, FW;
    int IC, OC;
    int icb;              // 32-channel blocks per tap = IC/32
    int MB;               // M blocks = taps * icb; 4 blocks make one 128-row M tile
    int G;                // M tiles (accumulators) per CTA
    int BN;               // N tile over OC, multiple of 32
    int KP;               // pixels per reduction chunk (multiple of 8)
    int chunks_per_split, total_chunks;
    int stages, mode3x;
    uint32_t tmem_cols, idesc;
};

__global__ void __launch_bounds__(kIgemmThreads)
    conv_dw_kernel(const __grid_constant__ CUtensorMap tmX,
                   const __grid_constant__ CUtensorMap tmDY, const DwParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = blockIdx.x, tile_n = blockIdx.y, split = blockIdx.z;
    const int S = p.stages;
    const uint32_t planes = p.mode3x ? 2u : 1u;
    const uint32_t blk_bytes = p.KP * 128;           // one 32-channel block of KP pixels
    const uint32_t a_bytes = 4 * blk_bytes;          // 128 rows of (tap, ic)
    const uint32_t b_bytes = (p.BN / 32) * blk_bytes;
    const uint32_t stage_bytes = (a_bytes + b_bytes) * planes;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S) * stage_bytes);
    uint64_t* full = bars;
    uint64_t* split_done = bars + S;
    uint64_t* empty = bars + 2 * S;
    uint64_t* accum = bars + 3 * S;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 3 * S + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&split_done[s], 128);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        fence_barrier_init();
        prefetch_tmap(&tmX);
        prefetch_tmap(&tmDY);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int MT = (p.MB + 3) / 4;                       // M tiles in total
    const int g_count = min(p.G, MT - group * p.G);      // M tiles of this CTA
    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(c_begin + p.chunks_per_split, p.total_chunks);
    const int n_chunks = max(c_end - c_begin, 0);
    const int num_it = n_chunks * g_count;

    if (warp == 0) {
        if (lane == 0) {
            const int hw = p.OHo * p.OWo;
            for (int it = 0; it < num_it; ++it) {
                const int s = it % S;
                const uint32_t par = (it / S) & 1;
                if (!mbar_wait(&empty[s], par ^ 1)) { report(p.status, kStatusProducerTimeout); break; }
                const int ci = it / g_count, g = it - ci * g_count;
                const int pix0 = (c_begin + ci) * p.KP;
                const int n_img = pix0 / hw;
                const int rem = pix0 - n_img * hw;
                const int pr = rem / p.OWo, qc = rem - pr * p.OWo;
                const int w0 = qc * p.sw - p.pw, h0 = pr * p.sh - p.ph;
                uint8_t* a_dst = smem + static_cast<size_t>(s) * stage_bytes;
                uint8_t* b_dst = a_dst + a_bytes * planes;
                const int mb0 = (group * p.G + g) * 4;
                const int nblk = min(4, p.MB - mb0);
                mbar_arrive_expect_tx(&full[s], (nblk + p.BN / 32) * blk_bytes);
                for (int b = 0; b < nblk; ++b) {
                    const int mb = mb0 + b;
                    const int tap = mb / p.icb, ic0 = (mb - tap * p.icb) * 32;
                    const int fh = tap / p.FW, fw = tap - fh * p.FW;
                    tma_load_im2col_4d(a_dst + b * blk_bytes, &tmX, &full[s], ic0, w0, h0, n_img,
                                       static_cast<uint16_t>(fw), static_cast<uint16_t>(fh));
                }
                for (int j = 0; j < p.BN / 32; ++j)
                    tma_load_2d(b_dst + j * blk_bytes, &tmDY, &full[s], tile_n * p.BN + j * 32, pix0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t dhi = smem_desc_hi(512, kSwizzle128B_Base32B);
            // ring and group positions as counters, barriers and tiles as 32-bit addresses: the issuing
            // thread does no division, pointer conversion or mode branch between two MMAs
            const uint32_t wait_a = smem_u32(p.mode3x ? split_done : full), empty_a = smem_u32(empty);
            const uint32_t smem_a = smem_u32(smem);
            const uint32_t a_lo_off = a_bytes >> 4, b_lo_off = b_bytes >> 4;
            const int ksteps = p.KP / 8;
            RingPos rp;
            int g = 0;            // accumulator of this iteration
            uint32_t first = 0u;  // 0 during the first pass over the accumulators
            for (int it = 0; it < num_it; ++it) {
                if (!mbar_wait_a(wait_a + 8 * rp.idx, rp.phase)) {
                    report(p.status, kStatusMmaTimeout);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + g * p.BN;
                const uint32_t a_addr = smem_a + rp.idx * stage_bytes;
                const uint32_t al = smem_desc_lo(a_addr, blk_bytes);
                const uint32_t bl = smem_desc_lo(a_addr + a_bytes * planes, blk_bytes);
                if (p.mode3x) {
                    for (int kk = 0; kk < ksteps; ++kk) {
                        const uint32_t acc = kk ? 1u : first;
                        const uint32_t a_k = al + kk * 64, b_k = bl + kk * 64;  // 1024 B per K=8 step
                        mma_tf32_ss2(d, a_k + a_lo_off, dhi, b_k, dhi, p.idesc, acc);
                        mma_tf32_ss2(d, a_k, dhi, b_k + b_lo_off, dhi, p.idesc, 1u);
                        mma_tf32_ss2(d, a_k, dhi, b_k, dhi, p.idesc, 1u);
                    }
                } else {
                    for (int kk = 0; kk < ksteps; ++kk)
                        mma_tf32_ss2(d, al + kk * 64, dhi, bl + kk * 64, dhi, p.idesc, kk ? 1u : first);
                }
                mma_commit_a(empty_a + 8 * rp.idx);
                rp.advance(S);
                if (++g == g_count) { g = 0; first = 1u; }
            }
            mma_commit(accum);
        }
        __syncwarp();
    } else {
        const int tid128 = threadIdx.x - 64;
        bool ok = true;
        if (p.mode3x) {
            for (int it = 0; it < num_it; ++it) {
                const int s = it % S;
                const uint32_t par = (it / S) & 1;
                if (!mbar_wait(&full[s], par)) { report(p.status, kStatusSplitTimeout); ok = false; break; }
                uint8_t* a_hi = smem + static_cast<size_t>(s) * stage_bytes;
                uint8_t* b_hi = a_hi + a_bytes * 2;
                split_plane(a_hi, a_hi + a_bytes, a_bytes, tid128);
                split_plane(b_hi, b_hi + b_bytes, b_bytes, tid128);
                fence_proxy_async_smem();
                mbar_arrive(&split_done[s]);
            }
        }
        if (ok && !mbar_wait(accum, 0)) { report(p.status, kStatusEpilogueTimeout); ok = false; }
        tc_fence_after_sync();
        if (ok) {
            const int quad = warp & 3;
            const int taps = p.FH * p.FW;
            float* obase = p.out + static_cast<size_t>(split) * p.split_stride;
            for (int g = 0; g < g_count; ++g) {
                const int mb = (group * p.G + g) * 4 + quad;
                const int tap = mb / p.icb;
                const int ic = (mb - tap * p.icb) * 32 + lane;
                const bool row_ok = (mb < p.MB) && (ic < p.IC);
                for (int c = 0; c < p.BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + g * p.BN + c, r);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int oc = tile_n * p.BN + c + j;
                            if (oc < p.OC) {
                                const float v = (n_chunks > 0) ? __uint_as_float(r[j]) : 0.f;
                                obase[(static_cast<size_t>(oc) * taps + tap) * p.IC + ic] = v;
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

// out[i] = sum over splits of part[s][i] with Kahan compensation (the reference sums its split-K buffers the
// same way: Cuda_dconv3D_deltaW/dconv3d_dW_GemmSK_bufSum.cuh:41-63).  When `accumulate` is set, out[i] itself is
// the first term (deltaW += sum of buffers).  LANES threads share one output vector: lane l adds the partials
// l, l + LANES, ... in that order, then the lanes' sums and compensations are added in lane order - a fixed
// order, so the result does not depend on scheduling.  The loop is bound by load latency (few threads, one
// dependent chain each), which is why many partials are spread over lanes.
template <int LANES>
__global__ void dw_reduce_kernel(const float* __restrict__ part, size_t split_stride, int splits,
                                 float* __restrict__ out, size_t n4, int accumulate)
{
    const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t i = t / LANES;
    const int lane = static_cast<int>(t % LANES);
    const bool live = i < n4;
    float4 s = (live && accumulate && lane == 0) ? reinterpret_cast<const float4*>(out)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
    auto add = [&](const float4& v) {
        float y, u;
        y = v.x - c.x; u = s.x + y; c.x = (u - s.x) - y; s.x = u;
        y = v.y - c.y; u = s.y + y; c.y = (u - s.y) - y; s.y = u;
        y = v.z - c.z; u = s.z + y; c.z = (u - s.z) - y; s.z = u;
        y = v.w - c.w; u = s.w + y; c.w = (u - s.w) - y; s.w = u;
    };
    if (live) {
        // eight loads in flight, then the compensated additions in order
        int k = lane;
        for (; k + 7 * LANES < splits; k += 8 * LANES) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldg(reinterpret_cast<const float4*>(part + (k + j * LANES) * split_stride) + i);
#pragma unroll
            for (int j = 0; j < 8; ++j) add(v[j]);
        }
        for (; k < splits; k += LANES) add(__ldg(reinterpret_cast<const float4*>(part + k * split_stride) + i));
    }
    if (LANES > 1) {
        // lane 0 adds the other lanes' sums, then takes off their compensations (what each lane's sum overshot)
        const unsigned mask = 0xffffffffu;
        const int base = (threadIdx.x & 31) - lane;
#pragma unroll
        for (int l = 1; l < LANES; ++l) {
            float4 so, co;
            so.x = __shfl_sync(mask, s.x, base + l); so.y = __shfl_sync(mask, s.y, base + l);
            so.z = __shfl_sync(mask, s.z, base + l); so.w = __shfl_sync(mask, s.w, base + l);
            co.x = __shfl_sync(mask, c.x, base + l); co.y = __shfl_sync(mask, c.y, base + l);
            co.z = __shfl_sync(mask, c.z, base + l); co.w = __shfl_sync(mask, c.w, base + l);
            if (lane == 0) {
                add(so);
                add(make_float4(-co.x, -co.y, -co.z, -co.w));
            }
        }
    }
    if (live && lane == 0) reinterpret_cast<float4*>(out)[i] = s;
}

// Launch helper: one lane per output vector for a handful of partials, four when there are many
// (lanes: 0 = choose, 1 or 4 = forced).
inline void launch_dw_reduce(const float* part, size_t split_stride, int splits, float* out, size_t n4, int accumulate,
                             cudaStream_t stream, int lanes = 0)
{
    if (lanes == 4 || (lanes == 0 && splits >= 32)) {
        const size_t threads = n4 * 4;
        dw_reduce_kernel<4><<<static_cast<unsigned>((threads + 127) / 128), 128, 0, stream>>>(part, split_stride, splits, out, n4, accumulate);
    } else {
        dw_reduce_kernel<1><<<static_cast<unsigned>((n4 + 63) / 64), 64, 0, stream>>>(part, split_stride, splits, out, n4, accumulate);
    }
}

// Column sums of a row-major matrix x[rows][cols4 * 4] (the bias gradient: deltaY summed over batch
// and pixels, Engine.field_sum(deltaY, OC) in nn/unit/simple/Conv3D.java:160).  HBM-bound: every
// byte is read once, 8 independent 16-byte loads in flight per thread.  CTA (bx, by) owns the rows
// [rows*bx/Gx, rows*(bx+1)/Gx) of the CT float4 columns starting at by*CT; thread (rl, ct) of
// RL x CT adds rows rl, rl+RL, ... of its column; the RL row lanes are then added in lane order and
// the CTA writes its piece of partial row bx.  A second launch sums the partial rows the same way,
// so the result does not depend on timing.
constexpr int kFieldSumThreads = 256;
__global__ void __launch_bounds__(kFieldSumThreads)
    field_sum_partial_kernel(const float4* __restrict__ x, long long rows, int cols4, int CT, int RL,
                             float4* __restrict__ partials)
{
    __shared__ float4 red[kFieldSumThreads];
    const int tid = threadIdx.x;
    const int rl = tid / CT, ct = tid - rl * CT;
    const int c = blockIdx.y * CT + ct;
    const bool on = rl < RL && c < cols4;
    const long long r0 = rows * blockIdx.x / gridDim.x, r1 = rows * (blockIdx.x + 1) / gridDim.x;
    auto add4 = [](float4& a, const float4& v) { a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; };
    float4 acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) {
        const float4* col = x + c;
        long long r = r0 + rl;
        for (; r + 7LL * RL < r1; r += 8LL * RL) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __ldg(col + (r + static_cast<long long>(k) * RL) * cols4);
#pragma unroll
            for (int k = 0; k < 8; ++k) add4(acc[k], v[k]);
        }
        for (; r < r1; r += RL) add4(acc[0], __ldg(col + r * cols4));
        add4(acc[0], acc[1]); add4(acc[2], acc[3]); add4(acc[4], acc[5]); add4(acc[6], acc[7]);
        add4(acc[0], acc[2]); add4(acc[4], acc[6]); add4(acc[0], acc[4]);
    }
    red[tid] = acc[0];
    __syncthreads();
    if (rl == 0 && c < cols4) {
        float4 sum = red[ct];
        for (int l = 1; l < RL; ++l) add4(sum, red[l * CT + ct]);
        partials[static_cast<size_t>(blockIdx.x) * cols4 + c] = sum;
    }
}

// ---------------------------------------------------------------------------------------------
// plain fp32 kernels for the shapes the tensor path leaves out
// ---------------------------------------------------------------------------------------------

struct ConvShape {
    int N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw;
};

// One thread per output element (n, oh, ow, oc); taps in fh -> fw -> ic order.
__global__ void conv_fwd_simt(const float* __restrict__ X, const float* __restrict__ W,
                              const float* __restrict__ bias, float* __restrict__ Y, ConvShape s, int act_on,
                              float act_k)
{
    const size_t total = static_cast<size_t>(s.N) * s.OH * s.OW * s.OC;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int oc = static_cast<int>(i % s.OC);
        size_t t = i / s.OC;
        const int ow = static_cast<int>(t % s.OW); t /= s.OW;
        const int oh = static_cast<int>(t % s.OH);
        const int n = static_cast<int>(t / s.OH);
        float v = 0.f;
        for (int fh = 0; fh < s.FH; ++fh) {
            const int ih = oh * s.sh - s.ph + fh;
            if (ih < 0 || ih >= s.IH) continue;
            for (int fw = 0; fw < s.FW; ++fw) {
                const int iw = ow * s.sw - s.pw + fw;
                if (iw < 0 || iw >= s.IW) continue;
                const float* x = X + ((static_cast<size_t>(n) * s.IH + ih) * s.IW + iw) * s.IC;
                const float* w = W + ((static_cast<size_t>(oc) * s.FH + fh) * s.FW + fw) * s.IC;
                for (int ic = 0; ic < s.IC; ++ic) v = fmaf(x[ic], w[ic], v);
            }
        }
        if (bias) v += bias[oc];
        if (act_on) v = leaky_relu(v, act_k);
        Y[i] = v;
    }
}

// One thread per (n, ih, iw, ic); gathers the taps whose stride phase matches, no atomics.
__global__ void conv_dx_simt(const float* __restrict__ dY, const float* __restrict__ W,
                             float* __restrict__ dX, ConvShape s)
{
    const size_t total = static_cast<size_t>(s.N) * s.IH * s.IW * s.IC;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int ic = static_cast<int>(i % s.IC);
        size_t t = i / s.IC;
        const int iw = static_cast<int>(t % s.IW); t /= s.IW;
        const int ih = static_cast<int>(t % s.IH);
        const int n = static_cast<int>(t / s.IH);
        float v = 0.f;
        for (int fh = 0; fh < s.FH; ++fh) {
            const int a = ih + s.ph - fh;
            if (a < 0 || a % s.sh != 0) continue;
            const int oh = a / s.sh;
            if (oh >= s.OH) continue;
            for (int fw = 0; fw < s.FW; ++fw) {
                const int b = iw + s.pw - fw;
                if (b < 0 || b % s.sw != 0) continue;
                const int ow = b / s.sw;
                if (ow >= s.OW) continue;
                const float* dy = dY + ((static_cast<size_t>(n) * s.OH + oh) * s.OW + ow) * s.OC;
                const float* w = W + (static_cast<size_t>(fh) * s.FW + fw) * s.IC + ic;
                const size_t wstride = static_cast<size_t>(s.FH) * s.FW * s.IC;
                for (int oc = 0; oc < s.OC; ++oc) v = fmaf(dy[oc], w[oc * wstride], v);
            }
        }
        dX[i] = v;
    }
}

// One block per deltaW element (oc, fh, fw, ic): 128 threads stride over the pixels, then a
// fixed-shape tree sum in shared memory (deterministic).
__global__ void __launch_bounds__(128)
    conv_dw_simt(const float* __restrict__ X, const float* __restrict__ dY, float* __restrict__ dW,
                 ConvShape s)
{
    __shared__ float red[128];
    const size_t e = blockIdx.x;
    const int ic = static_cast<int>(e % s.IC);
    size_t t = e / s.IC;
    const int fw = static_cast<int>(t % s.FW); t /= s.FW;
    const int fh = static_cast<int>(t % s.FH);
    const int oc = static_cast<int>(t / s.FH);
    const int npix = s.N * s.OH * s.OW;
    float v = 0.f;
    for (int k = threadIdx.x; k < npix; k += 128) {
        const int n = k / (s.OH * s.OW);
        const int r = k - n * s.OH * s.OW;
        const int oh = r / s.OW, ow = r - oh * s.OW;
        const int ih = oh * s.sh - s.ph + fh, iw = ow * s.sw - s.pw + fw;
        if (ih < 0 || iw < 0 || ih >= s.IH || iw >= s.IW) continue;
        v = fmaf(X[((static_cast<size_t>(n) * s.IH + ih) * s.IW + iw) * s.IC + ic],
                 dY[static_cast<size_t>(k) * s.OC + oc], v);
    }
    red[threadIdx.x] = v;
    __syncthreads();
    for (int o = 64; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) dW[e] = red[0];
}

}  // namespace alpha
