// JNI entry points of the native classes this library replaces.  The exported names and
// signatures are those of the reference's shims (Cuda_conv3D/A.cu:14-244, Cuda_dconv3D_deltaX/A.cu:14-325,
// Cuda_dconv3D_deltaW/A.cu:16-154, Cuda_matMul/A.cu:18-120, Cuda_batchMatMul/A.cu:17-135): each unpacks the Java stream array and forwards to the
// alpha_Cuda_* function of the same name.  A non-zero status becomes a pending
// z.dragon.engine.cuda.impl.CudaException carrying the library's error text (the reference looks up
// the stale class path z/jcuda/exception/CudaException, Cuda_conv3D/JNITool.cuh:16).
#include "../../include/alpha_conv_b200.h"
#include "../../include/alpha_conv_jni.h"

namespace {

constexpr int kMaxStreams = 16;

struct Streams {
    int64_t v[kMaxStreams];
    int n;
};

inline Streams get_streams(JNIEnv* env, jlongArray arr, jint length)
{
    Streams s{};
    // a null array, or a length beyond the Java array (GetLongArrayRegion then leaves an
    // ArrayIndexOutOfBoundsException pending and the buffer unwritten), yields an empty list: the
    // native fails with "empty stream array" or the pending exception reaches the Java caller
    if (!arr) return s;
    s.n = length < 0 ? 0 : (length > kMaxStreams ? kMaxStreams : length);
    jlong tmp[kMaxStreams] = {};
    if (s.n > 0) env->GetLongArrayRegion(arr, 0, s.n, tmp);
    if (env->ExceptionCheck()) { s.n = 0; return s; }
    for (int i = 0; i < s.n; ++i) s.v[i] = tmp[i];
    return s;
}

inline void raise(JNIEnv* env, int rc)
{
    if (rc == ALPHA_OK || env->ExceptionCheck()) return;
    jclass cls = env->FindClass("z/dragon/engine/cuda/impl/CudaException");
    if (cls) env->ThrowNew(cls, alpha_conv_last_error());
}

inline float* fp(jlong a) { return reinterpret_cast<float*>(static_cast<intptr_t>(a)); }
inline int* ip(jlong a) { return reinterpret_cast<int*>(static_cast<intptr_t>(a)); }

}  // namespace

extern "C" {

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw,
    jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D(st.v, st.n, fp(X_address), IH, IW, fp(W_address), FH, FW,
    fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw,
    jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_texture(st.v, st.n, fp(X_address), IH, IW, fp(W_address),
    FH, FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3DV2(JNIEnv* env, jclass,
    jboolean useTexture, jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW,
    jlong W_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint
    OC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3DV2(useTexture ? 1 : 0, st.v, st.n, fp(X_address), IH, IW,
    fp(W_address), FH, FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1np(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_np(st.v, st.n, fp(X_address), IH, IW, fp(W_address), FH,
    FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1W1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    Y_address, jint N, jint IC, jint OC)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_W1(st.v, st.n, fp(X_address), IH, IW, fp(W_address),
    fp(Y_address), N, IC, OC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_kernel_1remode(JNIEnv* env, jclass,
    jlong stream_address, jlong W_address, jlong CW_address, jint FH, jint FW, jint OC, jint IC)
{
    raise(env, alpha_Cuda_conv3D_kernel_remode(stream_address, fp(W_address), fp(CW_address), FH,
    FW, OC, IC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC,
    jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_GemmR(st.v, st.n, fp(X_address), IH, IW, fp(W_address),
    fp(CW_address), FH, FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC,
    jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_GemmR_texture(st.v, st.n, fp(X_address), IH, IW,
    fp(W_address), fp(CW_address), FH, FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmV2R(JNIEnv* env, jclass,
    jboolean useTexture, jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW,
    jlong W_address, jlong CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint
    N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_GemmV2R(useTexture ? 1 : 0, st.v, st.n, fp(X_address), IH,
    IW, fp(W_address), fp(CW_address), FH, FW, fp(Y_address), OH, OW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR_1W1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jlong Y_address, jint N, jint IC, jint OC)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_conv3D_conv3D_GemmR_W1(st.v, st.n, fp(X_address), IH, IW, fp(W_address),
    fp(CW_address), fp(Y_address), N, IC, OC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1(st.v, st.n, fp(deltaY_address), OH, OW,
    fp(W_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_s1_texture(st.v, st.n, fp(deltaY_address),
    OH, OW, fp(W_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1V2_1s1(JNIEnv* env, jclass,
    jboolean useTexture, jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint
    OW, jlong W_address, jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint
    IC, jint OC, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_V2_s1(useTexture ? 1 : 0, st.v, st.n,
    fp(deltaY_address), OH, OW, fp(W_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph,
    pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1W1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jlong W_address, jlong
    deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_W1(st.v, st.n, fp(deltaY_address),
    fp(W_address), fp(deltaX_address), IH, IW, N, IC, OC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_ks_1remode(JNIEnv* env, jclass,
    jlong stream_address, jlong W_address, jint FH, jint FW, jlong CW_address, jint CFH, jint CFW,
    jint OC, jint IC, jint sh, jint sw)
{
    raise(env, alpha_Cuda_dconv3D_deltaX_ks_remode(stream_address, fp(W_address), FH, FW,
    fp(CW_address), CFH, CFW, OC, IC, sh, sw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_ks_1remodev2(JNIEnv* env, jclass,
    jlong stream_address, jlong W_address, jint FH, jint FW, jlong CW_address, jint CFH, jint CFW,
    jint OC, jint IC, jint sh, jint sw)
{
    raise(env, alpha_Cuda_dconv3D_deltaX_ks_remodev2(stream_address, fp(W_address), FH, FW,
    fp(CW_address), CFH, CFW, OC, IC, sh, sw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1kernelSplit(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_kernelSplit(st.v, st.n,
    fp(deltaY_address), OH, OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, sh,
    sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksImsR(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR(st.v, st.n, fp(deltaY_address), OH,
    OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksImsR_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksImsR_texture(st.v, st.n,
    fp(deltaY_address), OH, OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, sh,
    sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksIms2R(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R(st.v, st.n, fp(deltaY_address),
    OH, OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksIms2R_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksIms2R_texture(st.v, st.n,
    fp(deltaY_address), OH, OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph,
    pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksV2_1Ims2R(JNIEnv* env, jclass,
    jboolean useTexture, jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint
    OW, jlong CW_address, jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint
    IC, jint OC, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_ksV2_Ims2R(useTexture ? 1 : 0, st.v, st.n,
    fp(deltaY_address), OH, OW, fp(CW_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, ph,
    pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1crossAdd(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaX_dconv3D_deltaX_crossAdd(st.v, st.n, fp(deltaY_address),
    OH, OW, fp(W_address), FH, FW, fp(deltaX_address), IH, IW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong deltaY_address,
    jint OH, jint OW, jlong deltaW_address, jint FH, jint FW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW(st.v, st.n, fp(X_address), IH, IW,
    fp(deltaY_address), OH, OW, fp(deltaW_address), FH, FW, N, IC, OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1W1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong deltaY_address,
    jlong deltaW_address, jint N, jint IC, jint OC)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_W1(st.v, st.n, fp(X_address), IH, IW,
    fp(deltaY_address), fp(deltaW_address), N, IC, OC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_buf_1summary(JNIEnv* env, jclass,
    jlong stream_address, jlong deltaW_buf_address, jlong deltaW_address, jint part, jint sizeW)
{
    raise(env, alpha_Cuda_dconv3D_deltaW_buf_summary(stream_address, fp(deltaW_buf_address),
    fp(deltaW_address), part, sizeW));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmSK(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jint OH, jint OW, jlong deltaW_address, jlong deltaW_buf_address, jint FH,
    jint FW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK(st.v, st.n, GridZ, fp(X_address),
    IH, IW, fp(deltaY_address), OH, OW, fp(deltaW_address), fp(deltaW_buf_address), FH, FW, N, IC,
    OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmV2SK(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jint OH, jint OW, jlong deltaW_address, jlong deltaW_buf_address, jint FH,
    jint FW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmV2SK(st.v, st.n, GridZ, fp(X_address),
    IH, IW, fp(deltaY_address), OH, OW, fp(deltaW_address), fp(deltaW_buf_address), FH, FW, N, IC,
    OC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmSK_1W1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jlong deltaW_address, jlong deltaW_buf_address, jint N, jint IC, jint OC)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_dconv3D_deltaW_dconv3D_deltaW_GemmSK_W1(st.v, st.n, GridZ,
    fp(X_address), IH, IW, fp(deltaY_address), fp(deltaW_address), fp(deltaW_buf_address), N, IC,
    OC));
}

// ---- Cuda_matMul (src/cu32_src/Cuda_matMul/Cuda_matMul/A.cu:18-120) ---------------------------------

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_SKbuf_1summary(JNIEnv* env, jclass,
    jlong stream_address, jlong dCbuf_address, jlong dC_address, jint part, jint sizeC)
{
    raise(env, alpha_Cuda_matMul_SKbuf_summary(stream_address, fp(dCbuf_address), fp(dC_address), part, sizeC));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMul(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_matMul_matMul(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), N, M, K));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_matMul_matMulT1(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), N, M, K));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT1SK(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jint GridZ, jlong dA_address, jlong dB_address, jlong dC_address,
    jlong dCbuf_address, jint N, jint M, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_matMul_matMulT1SK(st.v, st.n, GridZ, fp(dA_address), fp(dB_address), fp(dC_address),
    fp(dCbuf_address), N, M, K));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT2(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_matMul_matMulT2(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), N, M, K));
}

// ---- Cuda_batchMatMul (src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/A.cu:17-135) -------------------

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMul(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint M,
    jint BK, jint AK)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_batchMatMul_batchMatMul(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), Batch, N, M, BK, AK));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMul_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint M,
    jint BK, jint AK)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_batchMatMul_batchMatMul_texture(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), Batch, N, M, BK, AK));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT1(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint CN, jint AN,
    jint M, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_batchMatMul_batchMatMulT1(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), Batch, CN, AN, M, K));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT2(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint CM,
    jint BM, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_batchMatMul_batchMatMulT2(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), Batch, N, CM, BM, K));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT2_1texture(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint CM,
    jint BM, jint K)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_batchMatMul_batchMatMulT2_texture(st.v, st.n, fp(dA_address), fp(dB_address), fp(dC_address), Batch, N, CM, BM, K));
}

// ---- Cuda_pool2D / Cuda_upool2D (src/cu32_src/Cuda_pool2D/Cuda_pool2D/A.cu, src/cu32_src/Cuda_upool2D/Cuda_upool2D/A.cu:9-145) ----

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1max(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_pool2D_pool2D_max(st.v, st.n, fp(dX_address), IH, IW, FH, FW, fp(dY_address), OH, OW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1max_1indexed(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jlong dIndex_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_pool2D_pool2D_max_indexed(st.v, st.n, fp(dX_address), IH, IW, FH, FW, fp(dY_address), ip(dIndex_address), OH, OW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1avg(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_pool2D_pool2D_avg(st.v, st.n, fp(dX_address), IH, IW, FH, FW, fp(dY_address), OH, OW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1avg_1ignore_1padding(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_pool2D_pool2D_avg_ignore_padding(st.v, st.n, fp(dX_address), IH, IW, FH, FW, fp(dY_address), OH, OW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1max(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jlong dY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jlong dX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_max(st.v, st.n, fp(d_deltaY_address), fp(dY_address), OH, OW, FH, FW, fp(d_deltaX_address), fp(dX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1max_1Indexed(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jlong dIndex_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_max_Indexed(st.v, st.n, fp(d_deltaY_address), ip(dIndex_address), OH, OW, FH, FW, fp(d_deltaX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_avg(st.v, st.n, fp(d_deltaY_address), OH, OW, FH, FW, fp(d_deltaX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1tiled(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_avg_tiled(st.v, st.n, fp(d_deltaY_address), OH, OW, FH, FW, fp(d_deltaX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1ignore_1padding(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_avg_ignore_padding(st.v, st.n, fp(d_deltaY_address), OH, OW, FH, FW, fp(d_deltaX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1ignore_1padding_1tiled(JNIEnv* env, jclass,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw)
{
    Streams st = get_streams(env, streamArray, length);
    raise(env, alpha_Cuda_upool2D_upool2D_avg_ignore_padding_tiled(st.v, st.n, fp(d_deltaY_address), OH, OW, FH, FW, fp(d_deltaX_address), IH, IW, N, IC, sh, sw, ph, pw));
}

}  // extern "C"
