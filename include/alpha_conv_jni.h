/*
 * JNI symbols exported by libalpha_conv_b200.so: the `static native` methods of
 * z.dragon.engine.cuda.impl.math.Cuda_conv3D, Cuda_dconv3D_deltaX and Cuda_dconv3D_deltaW, with the
 * signatures of the reference's generated headers (src/cu32_src/Cuda_conv3D/Cuda_conv3D/Cuda_conv3D.cuh,
 * src/cu32_src/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX/Cuda_dconv3D_deltaX.cuh,
 * src/cu32_src/Cuda_dconv3D_deltaW/Cuda_dconv3D_deltaW/Cuda_deconv3D_deltaW.cuh).  Loading the
 * library with System.load binds them; no Java source changes besides the library file filter.
 */
#ifndef ALPHA_CONV_JNI_H
#define ALPHA_CONV_JNI_H

#include "alpha_jni_min.h"

#ifdef __cplusplus
extern "C" {
#endif

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw,
    jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw,
    jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3DV2(JNIEnv* env, jclass cls,
    jboolean useTexture, jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW,
    jlong W_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint
    OC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1np(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jint
    FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC, jint sh, jint sw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1W1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    Y_address, jint N, jint IC, jint OC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_kernel_1remode(JNIEnv* env, jclass cls,
    jlong stream_address, jlong W_address, jlong CW_address, jint FH, jint FW, jint OC, jint IC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC,
    jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint N, jint IC, jint OC,
    jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmV2R(JNIEnv* env, jclass cls,
    jboolean useTexture, jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW,
    jlong W_address, jlong CW_address, jint FH, jint FW, jlong Y_address, jint OH, jint OW, jint
    N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1conv3D_conv3D_1GemmR_1W1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong W_address, jlong
    CW_address, jlong Y_address, jint N, jint IC, jint OC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1s1_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1V2_1s1(JNIEnv* env, jclass cls,
    jboolean useTexture, jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint
    OW, jlong W_address, jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint
    IC, jint OC, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1W1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jlong W_address, jlong
    deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_ks_1remode(JNIEnv* env, jclass cls,
    jlong stream_address, jlong W_address, jint FH, jint FW, jlong CW_address, jint CFH, jint CFW,
    jint OC, jint IC, jint sh, jint sw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_ks_1remodev2(JNIEnv* env, jclass cls,
    jlong stream_address, jlong W_address, jint FH, jint FW, jlong CW_address, jint CFH, jint CFW,
    jint OC, jint IC, jint sh, jint sw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1kernelSplit(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksImsR(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksImsR_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksIms2R(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksIms2R_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong CW_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint ph,
    jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1ksV2_1Ims2R(JNIEnv* env, jclass cls,
    jboolean useTexture, jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint
    OW, jlong CW_address, jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint
    IC, jint OC, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaX_dconv3D_1deltaX_1crossAdd(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong deltaY_address, jint OH, jint OW, jlong W_address,
    jint FH, jint FW, jlong deltaX_address, jint IH, jint IW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong deltaY_address,
    jint OH, jint OW, jlong deltaW_address, jint FH, jint FW, jint N, jint IC, jint OC, jint sh,
    jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1W1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong X_address, jint IH, jint IW, jlong deltaY_address,
    jlong deltaW_address, jint N, jint IC, jint OC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_buf_1summary(JNIEnv* env, jclass cls,
    jlong stream_address, jlong deltaW_buf_address, jlong deltaW_address, jint part, jint sizeW);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmSK(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jint OH, jint OW, jlong deltaW_address, jlong deltaW_buf_address, jint FH,
    jint FW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmV2SK(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jint OH, jint OW, jlong deltaW_address, jlong deltaW_buf_address, jint FH,
    jint FW, jint N, jint IC, jint OC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1dconv3D_1deltaW_dconv3D_1deltaW_1GemmSK_1W1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jint GridZ, jlong X_address, jint IH, jint IW, jlong
    deltaY_address, jlong deltaW_address, jlong deltaW_buf_address, jint N, jint IC, jint OC);

/* Cuda_matMul: src/cu32_src/Cuda_matMul/Cuda_matMul/A.cu:18 (SKbuf_summary), :36 (matMul), :59 (matMulT1),
 * :76 (matMulT1SK), :104 (matMulT2); Java declarations in z/dragon/engine/cuda/impl/math/Cuda_matMul.java. */
JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_SKbuf_1summary(JNIEnv* env, jclass cls,
    jlong stream_address, jlong dCbuf_address, jlong dC_address, jint part, jint sizeC);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMul(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT1SK(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jint GridZ, jlong dA_address, jlong dB_address, jlong dC_address,
    jlong dCbuf_address, jint N, jint M, jint K);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1matMul_matMulT2(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint N, jint M, jint K);

/* Cuda_batchMatMul: src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul/A.cu:17 (batchMatMul), :38 (batchMatMul_texture),
 * :66 (batchMatMulT1), :92 (batchMatMulT2), :112 (batchMatMulT2_texture); Java declarations in
 * z/dragon/engine/cuda/impl/math/Cuda_batchMatMul.java:91-270. */
JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMul(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint M,
    jint BK, jint AK);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMul_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint M,
    jint BK, jint AK);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT1(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint CN, jint AN,
    jint M, jint K);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT2(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint CM,
    jint BM, jint K);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1batchMatMul_batchMatMulT2_1texture(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dA_address, jlong dB_address, jlong dC_address, jint Batch, jint N, jint CM,
    jint BM, jint K);

/* Cuda_pool2D (z/dragon/engine/cuda/impl/math/Cuda_pool2D.java:124-302; src/cu32_src/Cuda_pool2D/Cuda_pool2D/A.cu) and
 * Cuda_upool2D (src/cu32_src/Cuda_upool2D/Cuda_upool2D/A.cu:9-145). */
JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1max(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1max_1indexed(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jlong dIndex_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1avg(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1pool2D_pool2D_1avg_1ignore_1padding(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong dX_address, jint IH, jint IW, jint FH, jint FW, jlong dY_address, jint OH, jint OW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1max(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jlong dY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jlong dX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1max_1Indexed(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jlong dIndex_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1tiled(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1ignore_1padding(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

JNIEXPORT void JNICALL Java_z_dragon_engine_cuda_impl_math_Cuda_1upool2D_upool2D_1avg_1ignore_1padding_1tiled(JNIEnv* env, jclass cls,
    jlongArray streamArray, jint length, jlong d_deltaY_address, jint OH, jint OW, jint FH, jint FW, jlong d_deltaX_address, jint IH, jint IW, jint N, jint IC, jint sh, jint sw, jint ph, jint pw);

#ifdef __cplusplus
}
#endif
#endif /* ALPHA_CONV_JNI_H */