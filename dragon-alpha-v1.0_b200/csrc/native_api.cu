// Layers 2 and 3 of the C ABI: one function per native of the reference's JNI classes
// (Cuda_conv3D, Cuda_dconv3D_deltaX, Cuda_dconv3D_deltaW) and the four operator methods of
// CudaFloat32EngineBase that sit on this path.  Every variant of one operator (texture / V2 /
// remode / W1 / no-padding ...) computes the same function, so each forwards to the one layer-1
// call for that operator; the variant only chose among SIMT kernels in the reference.
#include "../../include/alpha_conv_b200.h"
#include "host_common.h"

namespace alpha {
int launch_buf_summary(cudaStream_t stream, const float* buf, float* deltaW, int part, size_t sizeW);
int launch_split_lo(cudaStream_t stream, const float* W, float* lo, size_t n);
void set_prepared_lo(const float* W, const float* lo);
void set_caller_scratch(void* ptr, size_t bytes);
}
using namespace alpha;

static inline alpha_stream_t first_stream(const int64_t* streams, int length)
{
    return (streams && length > 0) ? reinterpret_cast<alpha_stream_t>(static_cast<intptr_t>(streams[0]))
                                   : nullptr;
}

static inline AlphaConvShape shape(int N, int IH, int IW, int IC, int OC, int FH, int FW, int OH,
                                   int OW, int sh, int sw, int ph, int pw)
{
    AlphaConvShape s{N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw};
    return s;
}

static int fwd(const int64_t* streams, int length, float* X, int IH, int IW, float* W, int FH, int FW,
               float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_forward(&s, X, W, nullptr, Y, first_stream(streams, length));
}

static int dx(const int64_t* streams, int length, float* dY, int OH, int OW, float* W, int FH, int FW,
              float* dX, int IH, int IW, int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_deltaX(&s, dY, W, dX, first_stream(streams, length));
}

static int dw(const int64_t* streams, int length, float* X, int IH, int IW, float* dY, int OH, int OW,
              float* dW, int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    if (!streams || length < 1) return fail(ALPHA_E_ARG, "empty stream array");
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_deltaW(&s, X, dY, dW, first_stream(streams, length));
}

// Forward through a native that carries CW: kernel_remode has left the lo plane of W there, so the
// 3xTF32 kernels take W as the hi plane and CW as the lo plane and the call needs no scratch of its own.
static int fwd_cw(const int64_t* streams, int length, float* X, int IH, int IW, float* W, float* CW, int FH, int FW,
                  float* Y, int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    if (CW && (reinterpret_cast<uintptr_t>(CW) & 15) == 0) set_prepared_lo(W, CW);
    const int rc = fwd(streams, length, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
    set_prepared_lo(nullptr, nullptr);
    return rc;
}

// deltaW through a split-K entry: full gradient into deltaW, zeros into the caller's buffers.  The
// buffers serve as this call's scratch (per-CTA partial sums) as far as they reach.
static int dw_sk(const int64_t* streams, int length, int GridZ, float* X, int IH, int IW, float* dY,
                 int OH, int OW, float* dW, float* dW_buf, int FH, int FW, int N, int IC, int OC,
                 int sh, int sw, int ph, int pw)
{
    if (GridZ > 1 && !dW_buf) return fail(ALPHA_E_ARG, "GridZ=%d but deltaW_buf is null", GridZ);
    const size_t buf_bytes = GridZ > 1 ? static_cast<size_t>(GridZ - 1) * OC * FH * FW * IC * sizeof(float) : 0;
    if (buf_bytes && (reinterpret_cast<uintptr_t>(dW_buf) & 255) == 0) set_caller_scratch(dW_buf, buf_bytes);
    int rc = dw(streams, length, X, IH, IW, dY, OH, OW, dW, FH, FW, N, IC, OC, sh, sw, ph, pw);
    set_caller_scratch(nullptr, 0);
    if (rc) return rc;
    if (GridZ > 1) {
        const size_t bytes = buf_bytes;
        cudaError_t e = cudaMemsetAsync(dW_buf, 0, bytes, (cudaStream_t)first_stream(streams, length));
        if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemsetAsync(deltaW_buf): %s", cudaGetErrorString(e));
    }
    return ALPHA_OK;
}

static int copy_w(int64_t stream, const float* W, float* CW, int FH, int FW, int OC, int IC)
{
    if (!W || !CW) return fail(ALPHA_E_ARG, "null W or CW");
    const size_t bytes = static_cast<size_t>(OC) * FH * FW * IC * sizeof(float);
    cudaError_t e = cudaMemcpyAsync(CW, W, bytes, cudaMemcpyDeviceToDevice,
                                    reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream)));
    if (e != cudaSuccess) return fail(ALPHA_E_CUDA, "cudaMemcpyAsync(W -> CW): %s", cudaGetErrorString(e));
    return ALPHA_OK;
}

extern "C" {

// ---- Cuda_conv3D ----------------------------------------------------------------------------------

int alpha_Cuda_conv3D_conv3D(const int64_t* streams, int length, float* X, int IH, int IW, float* W,
                             int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC, int sh,
                             int sw, int ph, int pw)
{
    return fwd(streams, length, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3D_texture(const int64_t* streams, int length, float* X, int IH, int IW,
                                     float* W, int FH, int FW, float* Y, int OH, int OW, int N,
                                     int IC, int OC, int sh, int sw, int ph, int pw)
{
    return fwd(streams, length, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3DV2(int, const int64_t* streams, int length, float* X, int IH, int IW,
                               float* W, int FH, int FW, float* Y, int OH, int OW, int N, int IC,
                               int OC, int sh, int sw, int ph, int pw)
{
    return fwd(streams, length, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3D_np(const int64_t* streams, int length, float* X, int IH, int IW,
                                float* W, int FH, int FW, float* Y, int OH, int OW, int N, int IC,
                                int OC, int sh, int sw)
{
    return fwd(streams, length, X, IH, IW, W, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, 0, 0);
}
int alpha_Cuda_conv3D_conv3D_W1(const int64_t* streams, int length, float* X, int IH, int IW,
                                float* W, float* Y, int N, int IC, int OC)
{
    return fwd(streams, length, X, IH, IW, W, 1, 1, Y, IH, IW, N, IC, OC, 1, 1, 0, 0);
}
// The reference transposes W into CW[FH,FW,IC,OC] here.  The tensor path reads W in place through its
// own tensor map; what it needs prepared is the lo plane of the 3xTF32 split, lo = tf32(W - trunc19(W)),
// and CW (OC*FH*FW*IC floats, private between this native and the conv3D_GemmR* consumers) holds it.
int alpha_Cuda_conv3D_kernel_remode(int64_t stream, float* W, float* CW, int FH, int FW, int OC, int IC)
{
    if (!W || !CW || FH <= 0 || FW <= 0 || OC <= 0 || IC <= 0) return fail(ALPHA_E_ARG, "bad kernel_remode arguments");
    if ((IC & 3) || ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(CW)) & 15))
        return fail(ALPHA_E_ARG, "kernel_remode: IC must be a multiple of 4 and W, CW 16-byte aligned");
    return launch_split_lo(reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream)), W, CW,
                           static_cast<size_t>(OC) * FH * FW * IC);
}
int alpha_Cuda_conv3D_conv3D_GemmR(const int64_t* streams, int length, float* X, int IH, int IW,
                                   float* W, float* CW, int FH, int FW, float* Y, int OH, int OW, int N,
                                   int IC, int OC, int sh, int sw, int ph, int pw)
{
    return fwd_cw(streams, length, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3D_GemmR_texture(const int64_t* streams, int length, float* X, int IH,
                                           int IW, float* W, float* CW, int FH, int FW, float* Y,
                                           int OH, int OW, int N, int IC, int OC, int sh, int sw,
                                           int ph, int pw)
{
    return fwd_cw(streams, length, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3D_GemmV2R(int, const int64_t* streams, int length, float* X, int IH,
                                     int IW, float* W, float* CW, int FH, int FW, float* Y, int OH,
                                     int OW, int N, int IC, int OC, int sh, int sw, int ph, int pw)
{
    return fwd_cw(streams, length, X, IH, IW, W, CW, FH, FW, Y, OH, OW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_conv3D_conv3D_GemmR_W1(const int64_t* streams, int length, float* X, int IH, int IW,
                                      float* W, float* CW, float* Y, int N, int IC, int OC)
{
    return fwd_cw(streams, length, X, IH, IW, W, CW, 1, 1, Y, IH, IW, N, IC, OC, 1, 1, 0, 0);
}

// ---- Cuda_dconv3D_deltaX ------------------------------------------------------------------------

int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1(const int64_t* streams, int length, float* deltaY,
                                                int OH, int OW, float* W, int FH, int FW,
                                                float* deltaX, int IH, int IW, int N, int IC, int OC,
                                                int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, 1, 1, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1_texture(const int64_t* streams, int length,
                                                        float* deltaY, int OH, int OW, float* W,
                                                        int FH, int FW, float* deltaX, int IH,
                                                        int IW, int N, int IC, int OC, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, 1, 1, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_V2_s1(int, const int64_t* streams, int length,
                                                   float* deltaY, int OH, int OW, float* W, int FH,
                                                   int FW, float* deltaX, int IH, int IW, int N,
                                                   int IC, int OC, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, 1, 1, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_W1(const int64_t* streams, int length, float* deltaY,
                                                float* W, float* deltaX, int IH, int IW, int N,
                                                int IC, int OC)
{
    return dx(streams, length, deltaY, IH, IW, W, 1, 1, deltaX, IH, IW, N, IC, OC, 1, 1, 0, 0);
}
int alpha_Cuda_dconv3D_deltaX_ks_remode(int64_t stream, float* W, int FH, int FW, float* CW, int CFH,
                                        int CFW, int OC, int IC, int sh, int sw)
{
    if (static_cast<long long>(CFH) * CFW * sh * sw < static_cast<long long>(FH) * FW)
        return fail(ALPHA_E_ARG, "CW (CFH=%d CFW=%d sh=%d sw=%d) is smaller than W (FH=%d FW=%d)", CFH, CFW, sh, sw, FH, FW);
    return copy_w(stream, W, CW, FH, FW, OC, IC);
}
int alpha_Cuda_dconv3D_deltaX_ks_remodev2(int64_t stream, float* W, int FH, int FW, float* CW,
                                          int CFH, int CFW, int OC, int IC, int sh, int sw)
{
    return alpha_Cuda_dconv3D_deltaX_ks_remode(stream, W, FH, FW, CW, CFH, CFW, OC, IC, sh, sw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_kernelSplit(const int64_t* streams, int length,
                                                         float* deltaY, int OH, int OW, float* CW,
                                                         int FH, int FW, float* deltaX, int IH,
                                                         int IW, int N, int IC, int OC, int sh,
                                                         int sw, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR(const int64_t* streams, int length,
                                                    float* deltaY, int OH, int OW, float* CW, int FH,
                                                    int FW, float* deltaX, int IH, int IW, int N,
                                                    int IC, int OC, int sh, int sw, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR_texture(const int64_t* streams, int length,
                                                            float* deltaY, int OH, int OW, float* CW,
                                                            int FH, int FW, float* deltaX, int IH,
                                                            int IW, int N, int IC, int OC, int sh,
                                                            int sw, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R(const int64_t* streams, int length,
                                                     float* deltaY, int OH, int OW, float* CW,
                                                     int FH, int FW, float* deltaX, int IH, int IW,
                                                     int N, int IC, int OC, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, 2, 2, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R_texture(const int64_t* streams, int length,
                                                             float* deltaY, int OH, int OW,
                                                             float* CW, int FH, int FW,
                                                             float* deltaX, int IH, int IW, int N,
                                                             int IC, int OC, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, 2, 2, ph, pw);
}
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksV2_Ims2R(int, const int64_t* streams, int length,
                                                        float* deltaY, int OH, int OW, float* CW,
                                                        int FH, int FW, float* deltaX, int IH,
                                                        int IW, int N, int IC, int OC, int ph, int pw)
{
    return dx(streams, length, deltaY, OH, OW, CW, FH, FW, deltaX, IH, IW, N, IC, OC, 2, 2, ph, pw);
}
// The reference zeroes deltaX, synchronises the stream and scatters with global atomics
// (Cuda_dconv3D_deltaX/A.cu:314-316); the gather kernels here need neither and are deterministic.
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_crossAdd(const int64_t* streams, int length,
                                                      float* deltaY, int OH, int OW, float* W,
                                                      int FH, int FW, float* deltaX, int IH, int IW,
                                                      int N, int IC, int OC, int sh, int sw, int ph,
                                                      int pw)
{
    return dx(streams, length, deltaY, OH, OW, W, FH, FW, deltaX, IH, IW, N, IC, OC, sh, sw, ph, pw);
}

// ---- Cuda_dconv3D_deltaW ------------------------------------------------------------------------

int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW(const int64_t* streams, int length, float* X, int IH,
                                             int IW, float* deltaY, int OH, int OW, float* deltaW,
                                             int FH, int FW, int N, int IC, int OC, int sh, int sw,
                                             int ph, int pw)
{
    return dw(streams, length, X, IH, IW, deltaY, OH, OW, deltaW, FH, FW, N, IC, OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_W1(const int64_t* streams, int length, float* X, int IH,
                                                int IW, float* deltaY, float* deltaW, int N, int IC,
                                                int OC)
{
    return dw(streams, length, X, IH, IW, deltaY, IH, IW, deltaW, 1, 1, N, IC, OC, 1, 1, 0, 0);
}
int alpha_Cuda_dconv3D_deltaW_buf_summary(int64_t stream, float* deltaW_buf, float* deltaW, int part,
                                          int sizeW)
{
    if (part < 0 || sizeW <= 0 || (sizeW & 3) || !deltaW || (part > 0 && !deltaW_buf))
        return fail(ALPHA_E_ARG, "bad buf_summary arguments (part=%d sizeW=%d)", part, sizeW);
    if (part == 0) return ALPHA_OK;
    return launch_buf_summary(reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(stream)), deltaW_buf,
                              deltaW, part, static_cast<size_t>(sizeW));
}
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK(const int64_t* streams, int length, int GridZ,
                                                    float* X, int IH, int IW, float* deltaY, int OH,
                                                    int OW, float* deltaW, float* deltaW_buf, int FH,
                                                    int FW, int N, int IC, int OC, int sh, int sw,
                                                    int ph, int pw)
{
    return dw_sk(streams, length, GridZ, X, IH, IW, deltaY, OH, OW, deltaW, deltaW_buf, FH, FW, N, IC,
                 OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmV2SK(const int64_t* streams, int length, int GridZ,
                                                      float* X, int IH, int IW, float* deltaY,
                                                      int OH, int OW, float* deltaW,
                                                      float* deltaW_buf, int FH, int FW, int N,
                                                      int IC, int OC, int sh, int sw, int ph, int pw)
{
    return dw_sk(streams, length, GridZ, X, IH, IW, deltaY, OH, OW, deltaW, deltaW_buf, FH, FW, N, IC,
                 OC, sh, sw, ph, pw);
}
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK_W1(const int64_t* streams, int length, int GridZ,
                                                       float* X, int IH, int IW, float* deltaY,
                                                       float* deltaW, float* deltaW_buf, int N,
                                                       int IC, int OC)
{
    return dw_sk(streams, length, GridZ, X, IH, IW, deltaY, IH, IW, deltaW, deltaW_buf, 1, 1, N, IC,
                 OC, 1, 1, 0, 0);
}

// ---- CudaFloat32EngineBase operator methods ---------------------------------------------------------

int alpha_engine_conv3D(float* Y, int OH, int OW, const float* X, int IH, int IW, const float* W,
                        int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                        alpha_stream_t stream)
{
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_forward(&s, X, W, nullptr, Y, stream);
}
int alpha_engine_conv3D_biased(float* Y, int OH, int OW, const float* X, int IH, int IW,
                               const float* W, int FH, int FW, const float* Bias, int N, int IC,
                               int OC, int sh, int sw, int ph, int pw, alpha_stream_t stream)
{
    if (!Bias) return fail(ALPHA_E_ARG, "conv3D_biased needs a bias vector");
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_forward(&s, X, W, Bias, Y, stream);
}
int alpha_engine_dconv3D_deltaW(float* deltaW, int FH, int FW, const float* X, int IH, int IW,
                                const float* deltaY, int OH, int OW, int N, int IC, int OC, int sh,
                                int sw, int ph, int pw, alpha_stream_t stream)
{
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_deltaW(&s, X, deltaY, deltaW, stream);
}
int alpha_engine_dconv3D_deltaX(float* deltaX, int IH, int IW, const float* deltaY, int OH, int OW,
                                const float* W, int FH, int FW, int N, int IC, int OC, int sh,
                                int sw, int ph, int pw, alpha_stream_t stream)
{
    AlphaConvShape s = shape(N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw);
    return alpha_conv3d_deltaX(&s, deltaY, W, deltaX, stream);
}

}  // extern "C"
