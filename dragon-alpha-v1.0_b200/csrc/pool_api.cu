// 2D pooling on NHWC fp32 tensors: the operators that sit between the convolutions of a network
// (the reference's Cuda_pool2D and Cuda_upool2D libraries).  All of them move every input byte once
// and do a handful of flops per byte, so they are bound by HBM: one thread owns four channels of one
// output element (one 16-byte load per window position, consecutive threads on consecutive channels,
// so a warp reads 512 contiguous bytes per position), the grid is a multiple of the SM count, and the
// backward kernels GATHER (one thread per input element sums over the output windows that cover it,
// in ascending (oh, ow) order) - no atomics, no zero fill, results independent of the launch.
//
//   forward   max          Y = max over the valid window positions            pool2D_max_kernel.cuh:44-76
//             max_indexed  + Index = flat offset into X of the winning element pool2D_max_indexed_kernel.cuh:41-96
//             avg          Y = (sum over valid positions) / (FH * FW)          pool2D_avg_kernel.cuh
//             avg_ip       Y = (sum over valid positions) / (number of them)   pool2D_avg_ip_kernel.cuh
//   backward  max          dX = sum over covering windows of (X >= Y) * dY     upool2D_max_kernel.cuh:52-100
//             max_indexed  dX = sum over covering windows of (Index == me) * dY upool2d_max_indexed_kernel.cuh:44-100
//             avg / avg_ip dX = sum over covering windows of dY * (1 / (FH * FW))  or  dY / (valid positions of that window)
// (file names under src/cu32_src/Cuda_pool2D/Cuda_pool2D and src/cu32_src/Cuda_upool2D/Cuda_upool2D).
#include "../../include/alpha_conv_b200.h"
#include "host_common.h"
#include "fast_div.cuh"

using namespace alpha;

namespace {

constexpr float kFloatMin = -3.4028234e38f;   // the reference's FLOAT_MIN (Cuda_pool2D/micro.cuh:40)

using alpha::FastDiv;
using alpha::fast_div;

struct PoolDims {
    int N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw;
    FastDiv by_cqu, by_IW, by_IH, by_OW, by_OH, by_sh, by_sw;   // by_cqu: channel groups per thread step, IC / (V * U)
};

template <int V> struct Vec;
template <> struct Vec<4> { using F = float4; using I = int4; };
template <> struct Vec<1> { using F = float; using I = int; };

__device__ __forceinline__ float4 splat4(float v) { return make_float4(v, v, v, v); }
template <int V> __device__ __forceinline__ typename Vec<V>::F splat(float v);
template <> __device__ __forceinline__ float4 splat<4>(float v) { return splat4(v); }
template <> __device__ __forceinline__ float splat<1>(float v) { return v; }

// element-wise helpers on float / float4
__device__ __forceinline__ void vmax(float& a, float x) { a = fmaxf(a, x); }
__device__ __forceinline__ void vmax(float4& a, const float4& x) { a.x = fmaxf(a.x, x.x); a.y = fmaxf(a.y, x.y); a.z = fmaxf(a.z, x.z); a.w = fmaxf(a.w, x.w); }
__device__ __forceinline__ void vadd(float& a, float x) { a += x; }
__device__ __forceinline__ void vadd(float4& a, const float4& x) { a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w; }
__device__ __forceinline__ void vfma(float& a, float s, float x) { a = fmaf(s, x, a); }
__device__ __forceinline__ void vfma(float4& a, float s, const float4& x) { a.x = fmaf(s, x.x, a.x); a.y = fmaf(s, x.y, a.y); a.z = fmaf(s, x.z, a.z); a.w = fmaf(s, x.w, a.w); }
__device__ __forceinline__ float vdiv(float a, float d) { return a / d; }
__device__ __forceinline__ float4 vdiv(const float4& a, float d) { return make_float4(a.x / d, a.y / d, a.z / d, a.w / d); }
// the index follows the maximum: it moves to `off` unless x < v (so the last of several equal maxima wins)
__device__ __forceinline__ void vidx(int& idx, float x, float v, int off) { idx = x < v ? idx : off; }
__device__ __forceinline__ void vidx(int4& idx, const float4& x, const float4& v, int off)
{
    idx.x = x.x < v.x ? idx.x : off; idx.y = x.y < v.y ? idx.y : off + 1;
    idx.z = x.z < v.z ? idx.z : off + 2; idx.w = x.w < v.w ? idx.w : off + 3;
}
__device__ __forceinline__ void iadd(int& i, int s) { i += s; }
__device__ __forceinline__ void iadd(int4& i, int s) { i.x += s; i.y += s; i.z += s; i.w += s; }
__device__ __forceinline__ void vsel_ge(float& a, float x, float y, float dy) { a += (x >= y) * dy; }
__device__ __forceinline__ void vsel_ge(float4& a, const float4& x, const float4& y, const float4& dy)
{
    a.x += (x.x >= y.x) * dy.x; a.y += (x.y >= y.y) * dy.y; a.z += (x.z >= y.z) * dy.z; a.w += (x.w >= y.w) * dy.w;
}
__device__ __forceinline__ void vsel_eq(float& a, int idx, int off, float dy) { a += (idx == off) * dy; }
__device__ __forceinline__ void vsel_eq(float4& a, const int4& idx, int off, const float4& dy)
{
    a.x += (idx.x == off) * dy.x; a.y += (idx.y == off + 1) * dy.y; a.z += (idx.z == off + 2) * dy.z; a.w += (idx.w == off + 3) * dy.w;
}

enum FwdOp { kMax = 0, kMaxIndexed = 1, kAvg = 2, kAvgIp = 3 };

// V = 4 (16-byte accesses) or 1; U = channel groups per thread: a thread owns the groups g, g + cq / U, ... of one
// element (cq = IC / V groups per element), so that the index arithmetic of the element - the larger part of the
// instructions of these kernels - is shared by U loads per window position, while consecutive threads still touch
// consecutive groups (a warp reads 32 / (cq / U) elements x cq / U x 16 contiguous bytes per instruction).
template <int V, int U, int OP>
__global__ void __launch_bounds__(256) pool_fwd_kernel(const float* __restrict__ X, float* __restrict__ Y,
                                                       int* __restrict__ Index, PoolDims d)
{
    using F = typename Vec<V>::F;
    using I = typename Vec<V>::I;
    // element counts fit 31 bits (checked on the host), so the index arithmetic is 32-bit: 64-bit divisions per
    // element cost more than the memory traffic of these kernels
    const unsigned cqu = static_cast<unsigned>(d.IC / (V * U));   // groups per thread step
    const unsigned total = static_cast<unsigned>(d.N) * d.OH * d.OW * cqu;
    const FastDiv by_cq = d.by_cqu;
    const int cstep = static_cast<int>(cqu) * V;                  // channels between two groups of one thread
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        unsigned pix, cc, uow, uoh, un;
        by_cq.divmod(e, pix, cc);
        const unsigned opix = pix;
        d.by_OW.divmod(pix, pix, uow);
        d.by_OH.divmod(pix, un, uoh);
        const int c = static_cast<int>(cc) * V, ow = static_cast<int>(uow), oh = static_cast<int>(uoh), n = static_cast<int>(un);
        const int ih0 = oh * d.sh - d.ph, iw0 = ow * d.sw - d.pw;
        const size_t img = static_cast<size_t>(n) * d.IH * d.IW * d.IC;
        const float* x = X + img;
        F v[U];
        I idx[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { v[u] = splat<V>(OP <= kMaxIndexed ? kFloatMin : 0.f); idx[u] = I{}; }
        int count = 0;
        for (int fh = 0; fh < d.FH; ++fh) {
            const int ih = ih0 + fh;
            if (ih < 0 || ih >= d.IH) continue;
            for (int fw = 0; fw < d.FW; ++fw) {
                const int iw = iw0 + fw;
                if (iw < 0 || iw >= d.IW) continue;
                const int off = (ih * d.IW + iw) * d.IC + c;
                F xv[U];
#pragma unroll
                for (int u = 0; u < U; ++u) xv[u] = *reinterpret_cast<const F*>(x + off + u * cstep);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (OP <= kMaxIndexed) {
                        if (OP == kMaxIndexed) vidx(idx[u], xv[u], v[u], off + u * cstep);
                        vmax(v[u], xv[u]);
                    } else {
                        vadd(v[u], xv[u]);
                    }
                }
                ++count;
            }
        }
        const size_t yoff = static_cast<size_t>(opix) * d.IC + c;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (OP == kAvg) v[u] = vdiv(v[u], static_cast<float>(d.FH * d.FW));
            if (OP == kAvgIp) v[u] = vdiv(v[u], static_cast<float>(count));
            *reinterpret_cast<F*>(Y + yoff + u * cstep) = v[u];
            if (OP == kMaxIndexed) {
                iadd(idx[u], static_cast<int>(img));
                *reinterpret_cast<I*>(Index + yoff + u * cstep) = idx[u];
            }
        }
    }
}

enum BwdOp { kBwdMax = 0, kBwdMaxIndexed = 1, kBwdAvg = 2, kBwdAvgIp = 3 };

template <int V, int U, int OP>
__global__ void __launch_bounds__(256) pool_bwd_kernel(const float* __restrict__ dY, const float* __restrict__ Y,
                                                       const float* __restrict__ X, const int* __restrict__ Index,
                                                       float* __restrict__ dX, PoolDims d)
{
    using F = typename Vec<V>::F;
    using I = typename Vec<V>::I;
    const unsigned cqu = static_cast<unsigned>(d.IC / (V * U));
    const unsigned total = static_cast<unsigned>(d.N) * d.IH * d.IW * cqu;
    const FastDiv by_cq = d.by_cqu;
    const int cstep = static_cast<int>(cqu) * V;
    const float alpha = 1.0f / static_cast<float>(d.FH * d.FW);
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        unsigned pix, cc, uiw, uih, un;
        by_cq.divmod(e, pix, cc);
        const unsigned ipix = pix;
        d.by_IW.divmod(pix, pix, uiw);
        d.by_IH.divmod(pix, un, uih);
        const int c = static_cast<int>(cc) * V, iw = static_cast<int>(uiw), ih = static_cast<int>(uih), n = static_cast<int>(un);
        // output windows that contain (ih, iw): oh * sh - ph <= ih < oh * sh - ph + FH
        int t = ih + d.ph - d.FH + 1;
        const int oh_lo = t <= 0 ? 0 : static_cast<int>(d.by_sh.div(static_cast<unsigned>(t + d.sh - 1)));
        int oh_hi = static_cast<int>(d.by_sh.div(static_cast<unsigned>(ih + d.ph)));
        if (oh_hi > d.OH - 1) oh_hi = d.OH - 1;
        t = iw + d.pw - d.FW + 1;
        const int ow_lo = t <= 0 ? 0 : static_cast<int>(d.by_sw.div(static_cast<unsigned>(t + d.sw - 1)));
        int ow_hi = static_cast<int>(d.by_sw.div(static_cast<unsigned>(iw + d.pw)));
        if (ow_hi > d.OW - 1) ow_hi = d.OW - 1;
        const size_t xoff = static_cast<size_t>(ipix) * d.IC + c;
        const size_t yimg = static_cast<size_t>(n) * d.OH * d.OW * d.IC;
        F xv[U], v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            v[u] = splat<V>(0.f);
            xv[u] = OP == kBwdMax ? *reinterpret_cast<const F*>(X + xoff + u * cstep) : splat<V>(0.f);
        }
        for (int oh = oh_lo; oh <= oh_hi; ++oh)
            for (int ow = ow_lo; ow <= ow_hi; ++ow) {
                const size_t yo = yimg + static_cast<size_t>((oh * d.OW + ow) * d.IC + c);
                float scale = alpha;
                if (OP == kBwdAvgIp) {
                    // positions of this window that lie inside the image
                    int h0 = oh * d.sh - d.ph, h1 = h0 + d.FH, w0 = ow * d.sw - d.pw, w1 = w0 + d.FW;
                    if (h0 < 0) h0 = 0;
                    if (h1 > d.IH) h1 = d.IH;
                    if (w0 < 0) w0 = 0;
                    if (w1 > d.IW) w1 = d.IW;
                    scale = static_cast<float>((h1 - h0) * (w1 - w0));
                }
                F dy[U];
#pragma unroll
                for (int u = 0; u < U; ++u) dy[u] = *reinterpret_cast<const F*>(dY + yo + u * cstep);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (OP == kBwdMax) {
                        vsel_ge(v[u], xv[u], *reinterpret_cast<const F*>(Y + yo + u * cstep), dy[u]);
                    } else if (OP == kBwdMaxIndexed) {
                        vsel_eq(v[u], *reinterpret_cast<const I*>(Index + yo + u * cstep), static_cast<int>(xoff) + u * cstep, dy[u]);
                    } else if (OP == kBwdAvg) {
                        vfma(v[u], scale, dy[u]);   // v += alpha * deltaY per window, as upool2D_avg_kernel.cuh:84-94 does
                    } else {
                        vadd(v[u], vdiv(dy[u], scale));
                    }
                }
            }
#pragma unroll
        for (int u = 0; u < U; ++u) *reinterpret_cast<F*>(dX + xoff + u * cstep) = v[u];
    }
}

int check_pool(const char* what, const AlphaPoolShape* s, const void* a, const void* b)
{
    if (!s || !a || !b) return fail(ALPHA_E_ARG, "%s: null pointer", what);
    if (s->N <= 0 || s->IH <= 0 || s->IW <= 0 || s->IC <= 0 || s->FH <= 0 || s->FW <= 0 || s->sh <= 0 || s->sw <= 0 ||
        s->ph < 0 || s->pw < 0)
        return fail(ALPHA_E_ARG, "%s: bad shape (N=%d IH=%d IW=%d IC=%d F=%dx%d s=%dx%d p=%dx%d)", what, s->N, s->IH, s->IW, s->IC,
                    s->FH, s->FW, s->sh, s->sw, s->ph, s->pw);
    if (s->ph >= s->FH || s->pw >= s->FW) return fail(ALPHA_E_ARG, "%s: padding must be smaller than the window", what);
    const int OH = (s->IH + 2 * s->ph - s->FH) / s->sh + 1, OW = (s->IW + 2 * s->pw - s->FW) / s->sw + 1;
    if (s->IH + 2 * s->ph < s->FH || s->IW + 2 * s->pw < s->FW || s->OH != OH || s->OW != OW)
        return fail(ALPHA_E_ARG, "%s: OH x OW = %d x %d does not follow from the input size (expected %d x %d)", what, s->OH, s->OW, OH, OW);
    if (static_cast<long long>(s->N) * s->IH * s->IW * s->IC > 2147483647LL || static_cast<long long>(s->N) * OH * OW * s->IC > 2147483647LL)
        return fail(ALPHA_E_ARG, "%s: more than 2^31 - 1 elements in a tensor (the index tensor and the kernels' index arithmetic are 32-bit)", what);
    return ALPHA_OK;
}

PoolDims dims_of(const AlphaPoolShape* s, int V, int U)
{
    PoolDims d{s->N, s->IH, s->IW, s->IC, s->FH, s->FW, s->OH, s->OW, s->sh, s->sw, s->ph, s->pw, {}, {}, {}, {}, {}, {}, {}};
    d.by_cqu = fast_div(s->IC / (V * U));
    d.by_IW = fast_div(s->IW); d.by_IH = fast_div(s->IH);
    d.by_OW = fast_div(s->OW); d.by_OH = fast_div(s->OH);
    d.by_sh = fast_div(s->sh); d.by_sw = fast_div(s->sw);
    return d;
}

int sm_count()
{
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        sms[dev] = v;
    }
    return sms[dev];
}

unsigned grid_for(long long threads)
{
    const long long blocks = (threads + 255) / 256, cap = static_cast<long long>(sm_count()) * 16;
    return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

bool vec4_ok(const AlphaPoolShape* s, const void* a, const void* b, const void* c = nullptr, const void* d = nullptr)
{
    auto al = [](const void* p) { return !p || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return s->IC % 4 == 0 && al(a) && al(b) && al(c) && al(d);
}

int finish(const char* kernel, const char* algo)
{
    note_launch(algo);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "%s launch failed: %s", kernel, cudaGetErrorString(e));
    return ALPHA_OK;
}

template <int OP>
int run_fwd(const char* what, const AlphaPoolShape* s, const float* X, float* Y, int* Index, alpha_stream_t stream_)
{
    int rc = check_pool(what, s, X, Y);
    if (rc) return rc;
    if (OP == kMaxIndexed && !Index) return fail(ALPHA_E_ARG, "%s: null index tensor", what);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const long long outs = static_cast<long long>(s->N) * s->OH * s->OW * s->IC;
    if (vec4_ok(s, X, Y, Index) && s->IC % 16 == 0)
        pool_fwd_kernel<4, 4, OP><<<grid_for(outs / 16), 256, 0, stream>>>(X, Y, Index, dims_of(s, 4, 4));
    else if (vec4_ok(s, X, Y, Index))
        pool_fwd_kernel<4, 1, OP><<<grid_for(outs / 4), 256, 0, stream>>>(X, Y, Index, dims_of(s, 4, 1));
    else
        pool_fwd_kernel<1, 1, OP><<<grid_for(outs), 256, 0, stream>>>(X, Y, Index, dims_of(s, 1, 1));
    return finish("pool_fwd_kernel", "pool_fwd");
}

template <int OP>
int run_bwd(const char* what, const AlphaPoolShape* s, const float* dY, const float* Y, const float* X, const int* Index,
            float* dX, alpha_stream_t stream_)
{
    int rc = check_pool(what, s, dY, dX);
    if (rc) return rc;
    if (OP == kBwdMax && (!Y || !X)) return fail(ALPHA_E_ARG, "%s: needs X and Y of the forward pass", what);
    if (OP == kBwdMaxIndexed && !Index) return fail(ALPHA_E_ARG, "%s: null index tensor", what);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const long long ins = static_cast<long long>(s->N) * s->IH * s->IW * s->IC;
    const bool v4 = vec4_ok(s, dY, dX, Y, X) && (reinterpret_cast<uintptr_t>(Index) & 15) == 0;
    if (v4 && s->IC % 16 == 0)
        pool_bwd_kernel<4, 4, OP><<<grid_for(ins / 16), 256, 0, stream>>>(dY, Y, X, Index, dX, dims_of(s, 4, 4));
    else if (v4)
        pool_bwd_kernel<4, 1, OP><<<grid_for(ins / 4), 256, 0, stream>>>(dY, Y, X, Index, dX, dims_of(s, 4, 1));
    else
        pool_bwd_kernel<1, 1, OP><<<grid_for(ins), 256, 0, stream>>>(dY, Y, X, Index, dX, dims_of(s, 1, 1));
    return finish("pool_bwd_kernel", "pool_bwd");
}

inline alpha_stream_t first_stream(const int64_t* streams, int length)
{
    return (streams && length > 0) ? reinterpret_cast<alpha_stream_t>(static_cast<intptr_t>(streams[0])) : nullptr;
}

AlphaPoolShape shape_of(int N, int IH, int IW, int IC, int FH, int FW, int OH, int OW, int sh, int sw, int ph, int pw)
{
    return AlphaPoolShape{N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw};
}

}  // namespace

extern "C" {

int alpha_pool2D_max(const AlphaPoolShape* s, const float* X, float* Y, alpha_stream_t stream)
{
    return run_fwd<kMax>("pool2D_max", s, X, Y, nullptr, stream);
}
int alpha_pool2D_max_indexed(const AlphaPoolShape* s, const float* X, float* Y, int* Index, alpha_stream_t stream)
{
    return run_fwd<kMaxIndexed>("pool2D_max_indexed", s, X, Y, Index, stream);
}
int alpha_pool2D_avg(const AlphaPoolShape* s, const float* X, float* Y, int ignore_padding, alpha_stream_t stream)
{
    return ignore_padding ? run_fwd<kAvgIp>("pool2D_avg_ignore_padding", s, X, Y, nullptr, stream)
                          : run_fwd<kAvg>("pool2D_avg", s, X, Y, nullptr, stream);
}
int alpha_upool2D_max(const AlphaPoolShape* s, const float* deltaY, const float* Y, const float* X, float* deltaX,
                      alpha_stream_t stream)
{
    return run_bwd<kBwdMax>("upool2D_max", s, deltaY, Y, X, nullptr, deltaX, stream);
}
int alpha_upool2D_max_indexed(const AlphaPoolShape* s, const float* deltaY, const int* Index, float* deltaX, alpha_stream_t stream)
{
    return run_bwd<kBwdMaxIndexed>("upool2D_max_indexed", s, deltaY, nullptr, nullptr, Index, deltaX, stream);
}
int alpha_upool2D_avg(const AlphaPoolShape* s, const float* deltaY, float* deltaX, int ignore_padding, alpha_stream_t stream)
{
    return ignore_padding ? run_bwd<kBwdAvgIp>("upool2D_avg_ignore_padding", s, deltaY, nullptr, nullptr, nullptr, deltaX, stream)
                          : run_bwd<kBwdAvg>("upool2D_avg", s, deltaY, nullptr, nullptr, nullptr, deltaX, stream);
}

// ---- Cuda_pool2D natives (src/cu32_src/Cuda_pool2D/Cuda_pool2D/A.cu) ---------------------------------------
#define STREAMS_OK if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array")

int alpha_Cuda_pool2D_pool2D_max(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y, int OH,
                                 int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_pool2D_max(&s, X, Y, first_stream(streams, length));
}
int alpha_Cuda_pool2D_pool2D_max_indexed(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y,
                                         int* Index, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_pool2D_max_indexed(&s, X, Y, Index, first_stream(streams, length));
}
int alpha_Cuda_pool2D_pool2D_avg(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y, int OH,
                                 int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_pool2D_avg(&s, X, Y, 0, first_stream(streams, length));
}
int alpha_Cuda_pool2D_pool2D_avg_ignore_padding(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW,
                                                float* Y, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_pool2D_avg(&s, X, Y, 1, first_stream(streams, length));
}

// ---- Cuda_upool2D natives (src/cu32_src/Cuda_upool2D/Cuda_upool2D/A.cu:9-145) ------------------------------
int alpha_Cuda_upool2D_upool2D_max(const int64_t* streams, int length, float* deltaY, float* Y, int OH, int OW, int FH, int FW,
                                   float* deltaX, float* X, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_upool2D_max(&s, deltaY, Y, X, deltaX, first_stream(streams, length));
}
int alpha_Cuda_upool2D_upool2D_max_Indexed(const int64_t* streams, int length, float* deltaY, int* Index, int OH, int OW, int FH,
                                           int FW, float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_upool2D_max_indexed(&s, deltaY, Index, deltaX, first_stream(streams, length));
}
int alpha_Cuda_upool2D_upool2D_avg(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW, float* deltaX,
                                   int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_upool2D_avg(&s, deltaY, deltaX, 0, first_stream(streams, length));
}
int alpha_Cuda_upool2D_upool2D_avg_tiled(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW,
                                         float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw)
{
    return alpha_Cuda_upool2D_upool2D_avg(streams, length, deltaY, OH, OW, FH, FW, deltaX, IH, IW, N, IC, sh, sw, ph, pw);
}
int alpha_Cuda_upool2D_upool2D_avg_ignore_padding(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW,
                                                  float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw)
{
    STREAMS_OK;
    const AlphaPoolShape s = shape_of(N, IH, IW, IC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_upool2D_avg(&s, deltaY, deltaX, 1, first_stream(streams, length));
}
int alpha_Cuda_upool2D_upool2D_avg_ignore_padding_tiled(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH,
                                                        int FW, float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph,
                                                        int pw)
{
    return alpha_Cuda_upool2D_upool2D_avg_ignore_padding(streams, length, deltaY, OH, OW, FH, FW, deltaX, IH, IW, N, IC, sh, sw, ph, pw);
}

}  // extern "C"
