/*
 * alpha_conv_b200 - C ABI of the B200 (sm_100a) convolution library for Dragon-Alpha.
 *
 * Three layers, all `extern "C"`, plain pointers and sizes:
 *
 *   1. alpha_conv3d_*            one call per contraction (forward, deltaX, deltaW); everything
 *                                above is a thin wrapper over these.
 *   2. alpha_Cuda_*              one function per `static native` of the reference's three JNI
 *                                classes, same argument order minus (JNIEnv*, jclass); the JNI shim
 *                                (Java_z_dragon_engine_cuda_impl_math_Cuda_1*) unpacks the stream
 *                                array and forwards here.
 *   3. alpha_engine_*            the four operator methods of CudaFloat32EngineBase that own this
 *                                path (conv3D, conv3D_biased, dconv3D_deltaW, dconv3D_deltaX) in
 *                                the Java argument order.
 *
 * Tensors are fp32, C-contiguous NHWC: X[N,IH,IW,IC], W[OC,FH,FW,IC], Y[N,OH,OW,OC]; deltaX,
 * deltaY, deltaW are laid out like X, Y, W.  N, IC and OC arrive rounded up to a multiple of 4 with
 * zero-filled padding lanes (src/alpha_src/z/dragon/engine/EngineCore.java:697-699), device
 * pointers are 16-byte aligned.  Every call only enqueues work on the given stream and returns; it
 * never synchronises.  All functions return 0 on success or a negative ALPHA_E_* code;
 * alpha_conv_last_error() gives the message of the calling thread's last failure.
 */
#ifndef ALPHA_CONV_B200_H
#define ALPHA_CONV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ALPHA_OK 0
#define ALPHA_E_ARG (-1)      /* bad shape, null or misaligned pointer */
#define ALPHA_E_CUDA (-2)     /* a CUDA runtime or driver call failed */
#define ALPHA_E_DEVICE (-3)   /* not an sm_100 device */
#define ALPHA_E_KERNEL (-4)   /* a kernel reported a protocol error in its status word */
#define ALPHA_E_NOSCRATCH (-5) /* the call needs more scratch than the fixed or caller-given block holds */
#define ALPHA_E_CAPTURE (-6)  /* the call would have to allocate while its stream is being captured */

/* math mode of the tensor-core kernels */
#define ALPHA_MATH_3XTF32 0 /* default: hi/lo split, three TF32 MMAs per product, fp32-faithful */
#define ALPHA_MATH_TF32 1   /* opt-in: one TF32 MMA per product */

/* kernel family */
#define ALPHA_ALGO_AUTO 0  /* tensor path where the shape allows it, plain fp32 kernels elsewhere */
#define ALPHA_ALGO_TENSOR 1 /* tensor path or ALPHA_E_ARG */
#define ALPHA_ALGO_SIMT 2   /* plain fp32 kernels */
#define ALPHA_ALGO_WINOGRAD 3 /* forward 3x3 stride 1 only: Winograd F(2,3) */

typedef struct AlphaConvShape {
    int N, IH, IW, IC, OC, FH, FW, OH, OW, sh, sw, ph, pw;
} AlphaConvShape;

typedef void* alpha_stream_t; /* a cudaStream_t */

/* ---- library state ------------------------------------------------------------------------- */

const char* alpha_conv_last_error(void);
int alpha_conv_version(void);
/* Process-wide defaults; the environment variables ALPHA_CONV_MATH={3xtf32,tf32} and
 * ALPHA_CONV_ALGO={auto,tensor,simt,winograd} seed them. */
int alpha_conv_set_math_mode(int mode);
int alpha_conv_get_math_mode(void);
int alpha_conv_set_algo(int algo);
int alpha_conv_get_algo(void);
/* Per-call math mode and kernel family: the same three contractions with the two settings as
 * arguments (-1 = the process default above), for hosts that run engines with different settings in
 * one process.  (The reference has no such switch: its kernels are fp32 FFMA only.) */
int alpha_conv3d_forward_ex(const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                            float* Y, int math_mode, int algo, alpha_stream_t stream);
int alpha_conv3d_deltaX_ex(const AlphaConvShape* s, const float* deltaY, const float* W, float* deltaX,
                           int math_mode, int algo, alpha_stream_t stream);
int alpha_conv3d_deltaW_ex(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW,
                           int math_mode, int algo, alpha_stream_t stream);
/* Tuning switches of the tile planners by name ("HALO_PAIR", "CONV_TILE", "SM_BUDGET", ...; an
 * "ALPHA_" prefix is accepted).  The environment variables ALPHA_<NAME> seed them once, at the first
 * call into the library; no call reads the environment afterwards.  SM_BUDGET = n makes the
 * persistent kernels spread over n SMs instead of all of them (0 = all), leaving the others to a
 * collective that runs beside them. */
int alpha_conv_set_option(const char* name, int value);
int alpha_conv_get_option(const char* name, int* value);
/* Reads (and clears) the current device's kernel status word; synchronises the device.
 * 0 = every kernel so far finished its barrier protocol, otherwise the first failure code. */
int alpha_conv_device_status(void);
/* Number of kernel launches this library has issued from the calling process. */
unsigned long long alpha_conv_launch_count(void);
/* Name of the kernel family the last call of this thread used ("igemm", "dw", "simt", ...). */
const char* alpha_conv_last_algo(void);
/* Tile plan of the last halo-tile launch of this thread (tile shape, buffers), for tuning. */
const char* alpha_conv_last_plan(void);
/* Tracing aid: with ALPHA_CONV_PROF=1 in the environment the halo-tile kernel records, for its first
 * CTA, the clock ticks each warp role spent waiting and working (slots: producer patch wait,
 * producer B wait, MMA patch wait, MMA B wait, MMA accumulator wait, MMA total, epilogue wait,
 * epilogue work, split wait, split work, kernel total).  Copies up to n slots of the last launch. */
int alpha_conv_debug_counters(unsigned long long* out, int n);

/* ---- scratch memory ----------------------------------------------------------------------------
 *
 * The reference's natives get every scratch block (CW, deltaW_buf) from the Java mempool
 * (CudaFloat32EngineBase.java:1370-1385, 1707-1722).  The kernels here need other scratch: the lo
 * plane of W in 3xTF32, transposed weights for deltaX, per-CTA partial sums of deltaW, the patch
 * matrix of the small-channel paths.  Per (device, stream) the library keeps ONE block for it; every
 * call carves what it needs from the start of its stream's block, so calls on one stream reuse the
 * same bytes and calls on different streams never share any.
 *   - By default the block is library-owned and grown on demand with cudaMalloc.  An outgrown block
 *     is freed once the work that could still use it has finished; nothing is synchronised.  If the
 *     stream is being captured into a CUDA graph a call that would have to grow the block fails with
 *     ALPHA_E_CAPTURE instead: run the step once eagerly, or alpha_conv_reserve_workspace, before
 *     capturing.  A block that a capture saw stays allocated until alpha_conv_release_workspace,
 *     because replays of that graph keep addressing it.
 *   - A host that owns all device memory hands in its own block with alpha_conv_set_workspace
 *     (256-byte aligned; NULL returns the stream to library-owned scratch).  The library then never
 *     allocates for calls on that stream: a call that needs more fails with ALPHA_E_NOSCRATCH.
 *     alpha_conv_workspace_bytes tells in advance what one call needs (op: ALPHA_OP_*; current math
 *     mode, algo and options; it sizes the call by walking its planner without launching anything).
 *   - alpha_conv_release_workspace synchronises the current device and frees every library-owned
 *     block, retired block and cached weight transform on it (graphs captured earlier are invalid
 *     afterwards).  alpha_conv_workspace_in_use reports the bytes currently held.
 *   - The natives of layer 2 additionally use the scratch their own signature carries: kernel_remode
 *     leaves the lo plane of W in CW for the conv3D_GemmR* natives, and the GemmSK natives put their
 *     partial sums into deltaW_buf when it is large enough. */
#define ALPHA_OP_FORWARD 0
#define ALPHA_OP_DELTAX 1
#define ALPHA_OP_DELTAW 2
#define ALPHA_OP_BIAS_GRAD 3
int alpha_conv_workspace_bytes(const AlphaConvShape* s, int op, size_t* bytes);
int alpha_conv_set_workspace(alpha_stream_t stream, void* block, size_t bytes);
int alpha_conv_reserve_workspace(alpha_stream_t stream, size_t bytes);
int alpha_conv_release_workspace(void);
size_t alpha_conv_workspace_in_use(void);

/* ---- weight-side transforms kept across calls --------------------------------------------------
 *
 * Weights change only when the optimizer updates them (the reference's tensors carry that contract:
 * src/alpha_src/z/dragon/engine/Tensor.java:208-221, Engine.java:341-350), yet every forward call
 * needs the lo plane of W and every deltaX call needs W transposed, rotated and split.  With
 * alpha_conv_weight_cache(1) the library keeps each transform in memory of its own, keyed by the
 * address and shape of W, and reuses it until alpha_conv_weights_updated(W) (NULL = every tensor)
 * says the values changed; the host calls that after its optimizer step.  Off by default: a host
 * that does not announce updates would compute with stale weights.  The first use of a tensor
 * allocates (not inside a stream capture: ALPHA_E_CAPTURE). */
int alpha_conv_weight_cache(int enable);
int alpha_conv_weights_updated(const float* W);

/* The same transforms in memory the CALLER owns, for hosts that schedule them themselves: a training loop can
 * enqueue the transforms of all layers on a side stream right after the optimizer step (they depend on W only)
 * and keep them off the critical path of the forward and backward chains; the library allocates nothing and
 * records no events, the caller orders prepare before use (stream order, or an event, or a graph edge).
 *   alpha_conv_prepared_weights_bytes  size of the transform op (ALPHA_OP_FORWARD / ALPHA_OP_DELTAX) needs for this
 *                                      shape under the current math mode and options; 0 = none (plain TF32 forward)
 *   alpha_conv_prepare_weights         enqueues the transform of W into `prepared` (256-byte aligned) on `stream`
 *   alpha_conv3d_forward_prepared /    the contraction with the transform taken from `prepared`; shape, W address,
 *   alpha_conv3d_deltaX_prepared       operator and math mode must be those of the prepare call (checked on the
 *                                      host: ALPHA_E_ARG otherwise).  prepared == NULL is the plain call. */
int alpha_conv_prepared_weights_bytes(const AlphaConvShape* s, int op, size_t* bytes);
int alpha_conv_prepare_weights(const AlphaConvShape* s, int op, const float* W, void* prepared, size_t bytes,
                               alpha_stream_t stream);
int alpha_conv3d_forward_prepared(const AlphaConvShape* s, const float* X, const float* W, const void* prepared,
                                  size_t bytes, const float* bias, float* Y, alpha_stream_t stream);
int alpha_conv3d_deltaX_prepared(const AlphaConvShape* s, const float* deltaY, const float* W, const void* prepared,
                                 size_t bytes, float* deltaX, alpha_stream_t stream);

/* ---- layer 1: one call per contraction ------------------------------------------------------ */

/* Y = conv(X, W) (+ bias per output channel when bias != NULL).
 * Replaces the kernels behind Cuda_conv3D's natives
 * (src/cu32_src/Cuda_conv3D/Cuda_conv3D/conv3D.cuh:84-1651) and, with bias, the extra
 * linear_dual2D_row pass of CudaFloat32EngineBase.conv3D_biased (CudaFloat32EngineBase.java:1548-1557). */
int alpha_conv3d_forward(const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                         float* Y, alpha_stream_t stream);

/* Y = leakyRelu(conv(X, W) + bias, k), the activation applied in the epilogue of the same kernel
 * instead of a second pass over Y: Engine.leakyRelu after conv3D(_biased), i.e. the kernel
 * src/cu32_src/Cuda_function/Cuda_function/type4_leakyRelu2D.cuh:32-59 (y = x * ((x > 0) + k * (x < 0)));
 * k = 0 is ReLU.  bias may be NULL.  The backward pass keeps using the reference's own
 * leakyRelu2D_deltaX on Y before alpha_conv3d_deltaX / deltaW. */
int alpha_conv3d_forward_leakyRelu(const AlphaConvShape* s, const float* X, const float* W, const float* bias,
                                   float k, float* Y, alpha_stream_t stream);

/* deltaX = transposed conv of deltaY with W (also Deconv3D's forward).
 * Replaces src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/dconv3D_dX.cuh:83-1769. */
int alpha_conv3d_deltaX(const AlphaConvShape* s, const float* deltaY, const float* W, float* deltaX,
                        alpha_stream_t stream);

/* deltaW = correlation of X with deltaY summed over the batch.
 * Replaces src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/dconv3d_dW.cuh:72-700 including the
 * split-K buffer sum (dconv3d_dW_GemmSK_bufSum.cuh:32-67).  The per-CTA partial sums live in the
 * stream's scratch block (see "scratch memory" above). */
int alpha_conv3d_deltaW(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW,
                        alpha_stream_t stream);

/* deltaB[oc] = sum over the `rows` = N*OH*OW rows of deltaY[rows][OC]: the bias gradient of a biased
 * convolution, Engine.field_sum(deltaY, OC) in the backward pass of nn/unit/simple/Conv3D.java:160
 * (Engine.java:6945 -> field_linear(X, row_length, 1, 0)).  OC is the padded channel count (a
 * multiple of 4).  One pass over deltaY at HBM speed plus a fixed-order sum of the per-CTA partial
 * rows; the result is the same bits on every run. */
int alpha_conv_bias_grad(const float* deltaY, long long rows, int OC, float* deltaB, alpha_stream_t stream);

/* deltaW and the bias gradient deltaB[oc] = sum over pixels of deltaY in one call: what Conv3D.__backward__
 * asks of the engine as dconv3D_deltaW followed by field_sum(deltaY, OC) (nn/unit/simple/Conv3D.java:150-160).
 * For stride-1 layers the deltaW kernel adds up the columns of the deltaY tiles it stages anyway (no second
 * pass over deltaY); other shapes run alpha_conv3d_deltaW and alpha_conv_bias_grad one after the other.
 * deltaB == NULL is alpha_conv3d_deltaW.  Results do not depend on scheduling (fixed summation orders). */
int alpha_conv3d_deltaW_bias(const AlphaConvShape* s, const float* X, const float* deltaY, float* deltaW,
                             float* deltaB, alpha_stream_t stream);

/* deltaW for callers that cannot allocate device memory when they call.
 * (No counterpart in the reference: its natives get every buffer, scratch included, from the Java
 * mempool.)  A host such as Dragon-Alpha's engine claims the card's memory for its own pool up front
 * and gives natives nothing but addresses, so a cudaMalloc inside a native can fail or stall; other
 * callers sit in code that must never block on the allocator.  This entry point therefore calls no
 * cudaMalloc, cudaFree or any allocating routine.  The split-K partial sums, which
 * alpha_conv3d_deltaW keeps in a growable workspace, go into one fixed array of
 * alpha_conv3d_deltaW_noalloc_capacity() bytes (32 MiB) that is part of the library image: every GPU
 * on which the library is loaded holds it until the process exits.
 *   - Shapes whose partial sums need more than that return ALPHA_E_NOSCRATCH; shapes the tensor-core
 *     kernel does not take (IC not a multiple of 32) return ALPHA_E_ARG.  It always runs the split-K
 *     im2col kernel.  alpha_conv3d_deltaW runs that kernel, with the same plan and then the same bits,
 *     for strided layers; for stride 1 it prefers its halo-tile kernel, whose pixel sum is ordered
 *     differently, so there the two results agree to rounding (1e-4 of the largest element, the
 *     parity bound), not bit for bit.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call before starting any stream capture.
 *   - All calls on one device share the array, and it keeps what the last call left in it.  The
 *     kernel overwrites every partial it later reads, so nothing has to be cleared between calls,
 *     but two calls whose GPU work overlaps (different streams) race on it: serialise them.
 *   - Kernel protocol errors of this entry point are reported by alpha_conv3d_deltaW_noalloc_status()
 *     (synchronises the device; 0 = clean), not by alpha_conv_device_status(). */
int alpha_conv3d_deltaW_noalloc(const AlphaConvShape* s, const float* X, const float* deltaY,
                                float* deltaW, alpha_stream_t stream);
size_t alpha_conv3d_deltaW_noalloc_capacity(void);
int alpha_conv3d_deltaW_noalloc_status(void);

/* ---- layer 2: the reference's natives ------------------------------------------------------- */
/* `streams` holds `length` cudaStream_t values as 64-bit integers, as the Java side passes them;
 * all work is enqueued on streams[0], which satisfies every Syncer the caller builds
 * (CudaFloat32EngineBase.java:526-582, 715-796). */

/* Cuda_conv3D natives: src/cu32_src/Cuda_conv3D/Cuda_conv3D/A.cu:14-244 */
int alpha_Cuda_conv3D_conv3D(const int64_t* streams, int length, float* X, int IH, int IW, float* W,
                             int FH, int FW, float* Y, int OH, int OW, int N, int IC, int OC, int sh,
                             int sw, int ph, int pw);
int alpha_Cuda_conv3D_conv3D_texture(const int64_t* streams, int length, float* X, int IH, int IW,
                                     float* W, int FH, int FW, float* Y, int OH, int OW, int N,
                                     int IC, int OC, int sh, int sw, int ph, int pw);
int alpha_Cuda_conv3D_conv3DV2(int useTexture, const int64_t* streams, int length, float* X, int IH,
                               int IW, float* W, int FH, int FW, float* Y, int OH, int OW, int N,
                               int IC, int OC, int sh, int sw, int ph, int pw);
int alpha_Cuda_conv3D_conv3D_np(const int64_t* streams, int length, float* X, int IH, int IW,
                                float* W, int FH, int FW, float* Y, int OH, int OW, int N, int IC,
                                int OC, int sh, int sw);
int alpha_Cuda_conv3D_conv3D_W1(const int64_t* streams, int length, float* X, int IH, int IW,
                                float* W, float* Y, int N, int IC, int OC);
int alpha_Cuda_conv3D_kernel_remode(int64_t stream, float* W, float* CW, int FH, int FW, int OC,
                                    int IC);
int alpha_Cuda_conv3D_conv3D_GemmR(const int64_t* streams, int length, float* X, int IH, int IW,
                                   float* W, float* CW, int FH, int FW, float* Y, int OH, int OW,
                                   int N, int IC, int OC, int sh, int sw, int ph, int pw);
int alpha_Cuda_conv3D_conv3D_GemmR_texture(const int64_t* streams, int length, float* X, int IH,
                                           int IW, float* W, float* CW, int FH, int FW, float* Y,
                                           int OH, int OW, int N, int IC, int OC, int sh, int sw,
                                           int ph, int pw);
int alpha_Cuda_conv3D_conv3D_GemmV2R(int useTexture, const int64_t* streams, int length, float* X,
                                     int IH, int IW, float* W, float* CW, int FH, int FW, float* Y,
                                     int OH, int OW, int N, int IC, int OC, int sh, int sw, int ph,
                                     int pw);
int alpha_Cuda_conv3D_conv3D_GemmR_W1(const int64_t* streams, int length, float* X, int IH, int IW,
                                      float* W, float* CW, float* Y, int N, int IC, int OC);

/* Cuda_dconv3D_deltaX natives: src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/A.cu:14-325 */
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1(const int64_t* streams, int length, float* deltaY,
                                                int OH, int OW, float* W, int FH, int FW,
                                                float* deltaX, int IH, int IW, int N, int IC, int OC,
                                                int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1_texture(const int64_t* streams, int length,
                                                        float* deltaY, int OH, int OW, float* W,
                                                        int FH, int FW, float* deltaX, int IH,
                                                        int IW, int N, int IC, int OC, int ph,
                                                        int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_V2_s1(int useTexture, const int64_t* streams,
                                                   int length, float* deltaY, int OH, int OW,
                                                   float* W, int FH, int FW, float* deltaX, int IH,
                                                   int IW, int N, int IC, int OC, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_W1(const int64_t* streams, int length, float* deltaY,
                                                float* W, float* deltaX, int IH, int IW, int N,
                                                int IC, int OC);
/* ks_remode / ks_remodev2 leave in CW what the kernel-split entries below need, because those
 * entries never see W.  This library's private CW layout is a plain copy of W[OC,FH,FW,IC]
 * (CW holds OC*CFH*CFW*IC*sh*sw >= OC*FH*FW*IC floats). */
int alpha_Cuda_dconv3D_deltaX_ks_remode(int64_t stream, float* W, int FH, int FW, float* CW, int CFH,
                                        int CFW, int OC, int IC, int sh, int sw);
int alpha_Cuda_dconv3D_deltaX_ks_remodev2(int64_t stream, float* W, int FH, int FW, float* CW,
                                          int CFH, int CFW, int OC, int IC, int sh, int sw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_kernelSplit(const int64_t* streams, int length,
                                                         float* deltaY, int OH, int OW, float* CW,
                                                         int FH, int FW, float* deltaX, int IH,
                                                         int IW, int N, int IC, int OC, int sh,
                                                         int sw, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR(const int64_t* streams, int length,
                                                    float* deltaY, int OH, int OW, float* CW, int FH,
                                                    int FW, float* deltaX, int IH, int IW, int N,
                                                    int IC, int OC, int sh, int sw, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR_texture(const int64_t* streams, int length,
                                                            float* deltaY, int OH, int OW, float* CW,
                                                            int FH, int FW, float* deltaX, int IH,
                                                            int IW, int N, int IC, int OC, int sh,
                                                            int sw, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R(const int64_t* streams, int length,
                                                     float* deltaY, int OH, int OW, float* CW,
                                                     int FH, int FW, float* deltaX, int IH, int IW,
                                                     int N, int IC, int OC, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R_texture(const int64_t* streams, int length,
                                                             float* deltaY, int OH, int OW,
                                                             float* CW, int FH, int FW,
                                                             float* deltaX, int IH, int IW, int N,
                                                             int IC, int OC, int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksV2_Ims2R(int useTexture, const int64_t* streams,
                                                        int length, float* deltaY, int OH, int OW,
                                                        float* CW, int FH, int FW, float* deltaX,
                                                        int IH, int IW, int N, int IC, int OC,
                                                        int ph, int pw);
int alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_crossAdd(const int64_t* streams, int length,
                                                      float* deltaY, int OH, int OW, float* W,
                                                      int FH, int FW, float* deltaX, int IH, int IW,
                                                      int N, int IC, int OC, int sh, int sw, int ph,
                                                      int pw);

/* Cuda_dconv3D_deltaW natives: src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/A.cu:16-154.
 * The GemmSK entries write the complete gradient into deltaW and zero the (GridZ-1)*sizeW floats
 * of deltaW_buf, so the caller's following buf_summary(deltaW += sum of buffers) adds zeros. */
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW(const int64_t* streams, int length, float* X, int IH,
                                             int IW, float* deltaY, int OH, int OW, float* deltaW,
                                             int FH, int FW, int N, int IC, int OC, int sh, int sw,
                                             int ph, int pw);
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_W1(const int64_t* streams, int length, float* X, int IH,
                                                int IW, float* deltaY, float* deltaW, int N, int IC,
                                                int OC);
int alpha_Cuda_dconv3D_deltaW_buf_summary(int64_t stream, float* deltaW_buf, float* deltaW, int part,
                                          int sizeW);
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK(const int64_t* streams, int length, int GridZ,
                                                    float* X, int IH, int IW, float* deltaY, int OH,
                                                    int OW, float* deltaW, float* deltaW_buf, int FH,
                                                    int FW, int N, int IC, int OC, int sh, int sw,
                                                    int ph, int pw);
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmV2SK(const int64_t* streams, int length, int GridZ,
                                                      float* X, int IH, int IW, float* deltaY,
                                                      int OH, int OW, float* deltaW,
                                                      float* deltaW_buf, int FH, int FW, int N,
                                                      int IC, int OC, int sh, int sw, int ph,
                                                      int pw);
int alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK_W1(const int64_t* streams, int length, int GridZ,
                                                       float* X, int IH, int IW, float* deltaY,
                                                       float* deltaW, float* deltaW_buf, int N,
                                                       int IC, int OC);

/* ---- layer 3: CudaFloat32EngineBase's operator methods ------------------------------------- */
/* Argument order of src/alpha_src/z/dragon/engine/cuda/CudaFloat32EngineBase.java:1355 (conv3D),
 * :1478 (conv3D_biased), :1666 (dconv3D_deltaW), :1796 (dconv3D_deltaX); addresses are device
 * pointers, the trailing stream replaces the engine's stream pool. */
int alpha_engine_conv3D(float* Y, int OH, int OW, const float* X, int IH, int IW, const float* W,
                        int FH, int FW, int N, int IC, int OC, int sh, int sw, int ph, int pw,
                        alpha_stream_t stream);
int alpha_engine_conv3D_biased(float* Y, int OH, int OW, const float* X, int IH, int IW,
                               const float* W, int FH, int FW, const float* Bias, int N, int IC,
                               int OC, int sh, int sw, int ph, int pw, alpha_stream_t stream);
int alpha_engine_dconv3D_deltaW(float* deltaW, int FH, int FW, const float* X, int IH, int IW,
                                const float* deltaY, int OH, int OW, int N, int IC, int OC, int sh,
                                int sw, int ph, int pw, alpha_stream_t stream);
int alpha_engine_dconv3D_deltaX(float* deltaX, int IH, int IW, const float* deltaY, int OH, int OW,
                                const float* W, int FH, int FW, int N, int IC, int OC, int sh,
                                int sw, int ph, int pw, alpha_stream_t stream);

/* ---- matrix products (the FullConnect path: the contraction next to the convolutions) ------------------
 *
 * Row-major fp32 matrices whose dimensions arrive padded to multiples of 4 like every tensor of the
 * engine.  A matrix product is a 1x1 convolution over rows, so each form runs on the kernels of the
 * contraction it maps to (forward / deltaX / deltaW), tensor cores, math modes and fallbacks included.
 * Replace the SIMT kernels behind src/cu32_src/Cuda_matMul/Cuda_matMul/matMul.cuh, matMulT1.cuh, matMulT2.cuh. */
/* C[N,M] = A[N,K] * B[K,M] (+ bias[M] per row when bias != NULL: matMul_biased, CudaFloat32EngineBase.java:1142-1168) */
int alpha_matMul(const float* A, const float* B, const float* bias, float* C, int N, int M, int K, alpha_stream_t stream);
/* C[N,M] = A[K,N]^T * B[K,M] (Cuda_matMul.matMulT1 / matMulT1SK + SKbuf_summary, CudaFloat32EngineBase.java:1185-1230) */
int alpha_matMulT1(const float* A, const float* B, float* C, int N, int M, int K, alpha_stream_t stream);
/* C[N,M] = A[N,K] * B[M,K]^T (+ bias[M], fused into the epilogue) (CudaFloat32EngineBase.java:1233-1245) */
int alpha_matMulT2(const float* A, const float* B, const float* bias, float* C, int N, int M, int K, alpha_stream_t stream);

/* Cuda_matMul natives: src/cu32_src/Cuda_matMul/Cuda_matMul/A.cu:18-120.  matMulT1SK writes the complete
 * product into C, uses the caller's Cbuf as scratch and leaves it zero; SKbuf_summary is C += sum of buffers. */
int alpha_Cuda_matMul_SKbuf_summary(int64_t stream, float* Cbuf, float* C, int part, int sizeC);
int alpha_Cuda_matMul_matMul(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K);
int alpha_Cuda_matMul_matMulT1(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K);
int alpha_Cuda_matMul_matMulT1SK(const int64_t* streams, int length, int GridZ, float* A, float* B, float* C,
                                 float* Cbuf, int N, int M, int K);
int alpha_Cuda_matMul_matMulT2(const int64_t* streams, int length, float* A, float* B, float* C, int N, int M, int K);

/* CudaFloat32EngineBase.matMul / matMul_biased / matMulT1 / matMulT2 in the Java argument order. */
int alpha_engine_matMul(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream);
int alpha_engine_matMul_biased(float* C, const float* A, const float* B, int N, int M, int K, const float* Bias,
                               alpha_stream_t stream);
int alpha_engine_matMulT1(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream);
int alpha_engine_matMulT2(float* C, const float* A, const float* B, int N, int M, int K, alpha_stream_t stream);

/* ---- batched matrix products (FullConnect / attention-style operators) ----------------------------------
 * Replace the SIMT kernels behind src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/batchMatMul.cuh,
 * batchMatMulT1.cuh, batchMatMulT2.cuh (the three forms are stated as CPU loops in its test.cuh:95-140).
 * Only the last dimension of a tensor is padded to a multiple of 4 in the engine's memory, so a row pitch can
 * exceed the row length (EngineCore.java:587-622 passes both).  Dense shapes with a reduction length that is a
 * multiple of 32 (16 for T1, which also wants M % 32 == 0) run the tensor-core kernels, one image with its own
 * weights per batch entry; every other shape runs a plain fp32 kernel with the reference's arithmetic. */
/* C[b][N][M] = A[b][N][AK](:, 0:BK) * B[b][BK][M] */
int alpha_batchMatMul(const float* A, const float* B, float* C, int Batch, int N, int M, int BK, int AK, alpha_stream_t stream);
/* C[b][CN][M] = (A[b][K][AN](:, 0:CN))^T * B[b][K][M] */
int alpha_batchMatMulT1(const float* A, const float* B, float* C, int Batch, int CN, int AN, int M, int K, alpha_stream_t stream);
/* C[b][N][CM](:, 0:BM) = A[b][N][K] * B[b][BM][K]^T; the columns BM..CM of C are left as they are */
int alpha_batchMatMulT2(const float* A, const float* B, float* C, int Batch, int N, int CM, int BM, int K, alpha_stream_t stream);

/* Cuda_batchMatMul natives: src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/A.cu:17 (batchMatMul), :38
 * (batchMatMul_texture), :66 (batchMatMulT1), :92 (batchMatMulT2), :112 (batchMatMulT2_texture); the texture
 * variants are the same call here. */
int alpha_Cuda_batchMatMul_batchMatMul(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N,
                                       int M, int BK, int AK);
int alpha_Cuda_batchMatMul_batchMatMul_texture(const int64_t* streams, int length, float* A, float* B, float* C, int Batch,
                                               int N, int M, int BK, int AK);
int alpha_Cuda_batchMatMul_batchMatMulT1(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int CN,
                                         int AN, int M, int K);
int alpha_Cuda_batchMatMul_batchMatMulT2(const int64_t* streams, int length, float* A, float* B, float* C, int Batch, int N,
                                         int CM, int BM, int K);
int alpha_Cuda_batchMatMul_batchMatMulT2_texture(const int64_t* streams, int length, float* A, float* B, float* C, int Batch,
                                                 int N, int CM, int BM, int K);

/* CudaFloat32EngineBase.batchMatMul / batchMatMulT1 / batchMatMulT2 (CudaFloat32EngineBase.java:1256-1318) in the
 * Java argument order. */
int alpha_engine_batchMatMul(float* C, const float* A, const float* B, int Batch, int N, int M, int BK, int AK,
                             alpha_stream_t stream);
int alpha_engine_batchMatMulT1(float* C, const float* A, const float* B, int Batch, int CN, int AN, int M, int K,
                               alpha_stream_t stream);
int alpha_engine_batchMatMulT2(float* C, const float* A, const float* B, int Batch, int N, int CM, int BM, int K,
                               alpha_stream_t stream);

/* ---- 2D pooling (the operators between the convolutions of a network) ---------------------------------------
 * Replace the kernels behind src/cu32_src/Cuda_pool2D/Cuda_pool2D/pool2D.cuh and
 * src/cu32_src/Cuda_upool2D/Cuda_upool2D/upool2D.cuh.  NHWC fp32, any channel count (16-byte accesses when
 * IC % 4 == 0, which the engine's padding guarantees).  HBM-bound elementwise kernels; the backward forms gather
 * (no atomics, no zero fill of deltaX needed, results independent of the launch).
 * OH = (IH + 2 ph - FH) / sh + 1, likewise OW; padding must be smaller than the window. */
typedef struct AlphaPoolShape {
    int N, IH, IW, IC;   /* X[N][IH][IW][IC] */
    int FH, FW;          /* window */
    int OH, OW;          /* Y[N][OH][OW][IC] */
    int sh, sw, ph, pw;
} AlphaPoolShape;

/* Y = max over the window positions inside the image (Cuda_pool2D.pool2D_max, pool2D_max_kernel.cuh:44-76) */
int alpha_pool2D_max(const AlphaPoolShape* s, const float* X, float* Y, alpha_stream_t stream);
/* the same, and Index[n][oh][ow][c] = offset into X (in floats, from X[0]) of the element that gave the maximum, the
 * last one of several equal ones (pool2D_max_indexed_kernel.cuh:41-96) */
int alpha_pool2D_max_indexed(const AlphaPoolShape* s, const float* X, float* Y, int* Index, alpha_stream_t stream);
/* Y = sum over the window positions inside the image / (FH * FW), or with ignore_padding / their number
 * (pool2D_avg_kernel.cuh, pool2D_avg_ip_kernel.cuh) */
int alpha_pool2D_avg(const AlphaPoolShape* s, const float* X, float* Y, int ignore_padding, alpha_stream_t stream);
/* deltaX = sum over the windows that contain the element of (X >= Y) * deltaY (upool2D_max_kernel.cuh:52-100) */
int alpha_upool2D_max(const AlphaPoolShape* s, const float* deltaY, const float* Y, const float* X, float* deltaX,
                      alpha_stream_t stream);
/* deltaX = sum over the windows that contain the element of (Index == its offset) * deltaY
 * (upool2d_max_indexed_kernel.cuh:44-100) */
int alpha_upool2D_max_indexed(const AlphaPoolShape* s, const float* deltaY, const int* Index, float* deltaX, alpha_stream_t stream);
/* deltaX = sum over the windows that contain the element of deltaY * (1 / (FH * FW)), or with ignore_padding of
 * deltaY / (positions of that window inside the image) (upool2D_avg_kernel.cuh:84-94, upool2D_avg_ip_kernel.cuh) */
int alpha_upool2D_avg(const AlphaPoolShape* s, const float* deltaY, float* deltaX, int ignore_padding, alpha_stream_t stream);

/* Cuda_pool2D natives (z/dragon/engine/cuda/impl/math/Cuda_pool2D.java:124, :183, :241, :298) */
int alpha_Cuda_pool2D_pool2D_max(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y, int OH,
                                 int OW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_pool2D_pool2D_max_indexed(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y,
                                         int* Index, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_pool2D_pool2D_avg(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW, float* Y, int OH,
                                 int OW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_pool2D_pool2D_avg_ignore_padding(const int64_t* streams, int length, float* X, int IH, int IW, int FH, int FW,
                                                float* Y, int OH, int OW, int N, int IC, int sh, int sw, int ph, int pw);
/* Cuda_upool2D natives (src/cu32_src/Cuda_upool2D/Cuda_upool2D/A.cu:9, :33, :57, :79, :102, :124); the tiled variants
 * (window == stride) are the same call here */
int alpha_Cuda_upool2D_upool2D_max(const int64_t* streams, int length, float* deltaY, float* Y, int OH, int OW, int FH, int FW,
                                   float* deltaX, float* X, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_upool2D_upool2D_max_Indexed(const int64_t* streams, int length, float* deltaY, int* Index, int OH, int OW, int FH,
                                           int FW, float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_upool2D_upool2D_avg(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW, float* deltaX,
                                   int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_upool2D_upool2D_avg_tiled(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW,
                                         float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_upool2D_upool2D_avg_ignore_padding(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH, int FW,
                                                  float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph, int pw);
int alpha_Cuda_upool2D_upool2D_avg_ignore_padding_tiled(const int64_t* streams, int length, float* deltaY, int OH, int OW, int FH,
                                                        int FW, float* deltaX, int IH, int IW, int N, int IC, int sh, int sw, int ph,
                                                        int pw);

#ifdef __cplusplus
}
#endif
#endif /* ALPHA_CONV_B200_H */
