// Winograd F(2,3) along the image width for 3x3 stride-1 forward convolution, the 1-D form the
// reference sketches in src/cu32_src/Cuda_conv3D/Cuda_conv3D/WinoGrad_X5.cuh:26-150 and micro.cuh:382-430:
//   d -> (d0 - d2, d1 + d2, d2 - d1, d1 - d3),  g -> (g0, (g0+g1+g2)/2, (g0-g1+g2)/2, g2),
//   y0 = m0 + m1 + m2,  y1 = m1 - m2 - m3   with  m_k = sum over (fh, ic) of d'_k * g'_k.
// Each of the four element-wise products m_k is a 3x1 convolution over the transformed input and
// runs on the tensor-core forward kernel; the three transforms below are memory-bound passes.
// Six multiply-adds per pair of outputs instead of nine.
#pragma once
#include <cuda_runtime.h>

namespace alpha {

// U[k][oc][fh][ic], k = 0..3, from W[oc][fh][3][ic]; one thread per (oc, fh, ic4).
__global__ void wino_filter_kernel(const float* __restrict__ W, float* __restrict__ U, int OC, int IC)
{
    const size_t n4 = static_cast<size_t>(OC) * 3 * (IC / 4);
    const size_t plane = static_cast<size_t>(OC) * 3 * IC;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c4 = static_cast<int>(i % (IC / 4));
        const size_t row = i / (IC / 4);  // oc*3 + fh
        const float4* g = reinterpret_cast<const float4*>(W + row * 3 * IC) + c4;
        const float4 g0 = g[0], g1 = g[IC / 4], g2 = g[2 * (IC / 4)];
        float4 u1, u2;
        u1.x = 0.5f * (g0.x + g1.x + g2.x); u2.x = 0.5f * (g0.x - g1.x + g2.x);
        u1.y = 0.5f * (g0.y + g1.y + g2.y); u2.y = 0.5f * (g0.y - g1.y + g2.y);
        u1.z = 0.5f * (g0.z + g1.z + g2.z); u2.z = 0.5f * (g0.z - g1.z + g2.z);
        u1.w = 0.5f * (g0.w + g1.w + g2.w); u2.w = 0.5f * (g0.w - g1.w + g2.w);
        float4* o = reinterpret_cast<float4*>(U + row * IC) + c4;
        o[0] = g0;
        o[plane / 4] = u1;
        o[2 * (plane / 4)] = u2;
        o[3 * (plane / 4)] = g2;
    }
}

// V[k][n][ih][j][ic], j = 0..OWp-1 (output column pairs), from X[n][ih][iw][ic] with left padding pw.
__global__ void wino_input_kernel(const float* __restrict__ X, float* __restrict__ V, int N, int IH, int IW, int IC,
                                  int OWp, int pw)
{
    const int C4 = IC / 4;
    const size_t total = static_cast<size_t>(N) * IH * OWp * C4;
    const size_t plane4 = total;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c4 = static_cast<int>(i % C4);
        size_t t = i / C4;
        const int j = static_cast<int>(t % OWp);
        t /= OWp;  // n*IH + ih
        const float4* xrow = reinterpret_cast<const float4*>(X + t * IW * IC) + c4;
        const int iw0 = 2 * j - pw;
        float4 d[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int iw = iw0 + k;
            d[k] = (iw >= 0 && iw < IW) ? xrow[static_cast<size_t>(iw) * C4] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float4 v0, v1, v2, v3;
        v0.x = d[0].x - d[2].x; v1.x = d[1].x + d[2].x; v2.x = d[2].x - d[1].x; v3.x = d[1].x - d[3].x;
        v0.y = d[0].y - d[2].y; v1.y = d[1].y + d[2].y; v2.y = d[2].y - d[1].y; v3.y = d[1].y - d[3].y;
        v0.z = d[0].z - d[2].z; v1.z = d[1].z + d[2].z; v2.z = d[2].z - d[1].z; v3.z = d[1].z - d[3].z;
        v0.w = d[0].w - d[2].w; v1.w = d[1].w + d[2].w; v2.w = d[2].w - d[1].w; v3.w = d[1].w - d[3].w;
        float4* o = reinterpret_cast<float4*>(V) + i;
        o[0] = v0;
        o[plane4] = v1;
        o[2 * plane4] = v2;
        o[3 * plane4] = v3;
    }
}

// Y[n][oh][2j + {0,1}][oc] from M[k][n][oh][j][oc] (+ bias).
__global__ void wino_output_kernel(const float* __restrict__ M, const float* __restrict__ bias, float* __restrict__ Y,
                                   int N, int OH, int OW, int OC, int OWp)
{
    const int C4 = OC / 4;
    const size_t total = static_cast<size_t>(N) * OH * OWp * C4;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int c4 = static_cast<int>(i % C4);
        size_t t = i / C4;
        const int j = static_cast<int>(t % OWp);
        t /= OWp;  // n*OH + oh
        const float4* m = reinterpret_cast<const float4*>(M) + i;
        const float4 m0 = m[0], m1 = m[total], m2 = m[2 * total], m3 = m[3 * total];
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias) b = reinterpret_cast<const float4*>(bias)[c4];
        float4 y0, y1;
        y0.x = m0.x + m1.x + m2.x + b.x; y1.x = m1.x - m2.x - m3.x + b.x;
        y0.y = m0.y + m1.y + m2.y + b.y; y1.y = m1.y - m2.y - m3.y + b.y;
        y0.z = m0.z + m1.z + m2.z + b.z; y1.z = m1.z - m2.z - m3.z + b.z;
        y0.w = m0.w + m1.w + m2.w + b.w; y1.w = m1.w - m2.w - m3.w + b.w;
        float4* yrow = reinterpret_cast<float4*>(Y + t * OW * OC) + c4;
        yrow[static_cast<size_t>(2 * j) * C4] = y0;
        if (2 * j + 1 < OW) yrow[static_cast<size_t>(2 * j + 1) * C4] = y1;
    }
}

}  // namespace alpha
