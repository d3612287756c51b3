#!/bin/bash
# Builds the reference's three cu32 convolution libraries, its Cuda_reduce library (field_linear is
# what the engine's field_sum runs: the GPU oracle of the bias gradient) and its Cuda_matMul and
# Cuda_batchMatMul libraries (the GPU oracles of the matrix products) and its Cuda_pool2D / Cuda_upool2D
# libraries (the GPU oracles of the pooling operators), for sm_100 as a GPU-side oracle
# (TEST INFRASTRUCTURE).  Needs the reference checkout; writes only into oracle/_ref/ (git-ignored):
# a patched copy of the source directories (MSVC-only declarator lists and two locals that
# shadow a template parameter are rewritten, nothing else) and one shared object per library with
# the reference's own JNI entry points.  usage: build_ref_gpu.sh [reference root]
set -e
REF=${1:-/root/reference}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref/cu32
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
mkdir -p "$OUT"
for lib in Cuda_conv3D Cuda_dconv3D_deltaX Cuda_dconv3D_deltaW Cuda_reduce Cuda_matMul Cuda_pool2D Cuda_upool2D; do
    rm -rf "$OUT/$lib"
    cp -r "$REF/src/cu32_src/$lib/$lib" "$OUT/$lib"
    chmod -R u+w "$OUT/$lib"
done
# the batched products live in a solution directory of another name
rm -rf "$OUT/Cuda_batchMatMul"
cp -r "$REF/src/cu32_src/Cuda_batch_matMul/Cuda_batchMatMul" "$OUT/Cuda_batchMatMul"
chmod -R u+w "$OUT/Cuda_batchMatMul"
# MSVC accepts `int a, int b;` - standard C++ does not
sed -i -E 's/int X_fh, int X_fw;/int X_fh, X_fw;/' "$OUT"/Cuda_conv3D/*.cuh
sed -i -E 's/int GNr = GN \& 127, int GMr = /int GNr = GN \& 127; int GMr = /' "$OUT"/Cuda_conv3D/conv3D.cuh
# locals that redeclare the template parameter OH_OW
sed -i -E 's/const int OH_OW = OH \* OW, GK = N \* OH_OW;/const int GK = N * OH_OW;/' "$OUT"/Cuda_dconv3D_deltaW/dconv3d_dW_Gemm_kernel_EX2.cuh
sed -i -E 's/^\tint OH_OW = OH \* OW;\r?$//' "$OUT"/Cuda_dconv3D_deltaW/dconv3d_dW_GemmSK_kernel_EX2.cuh
# the sources were written on a case-insensitive file system: link the include names that differ in case
for lib in Cuda_reduce Cuda_matMul Cuda_batchMatMul Cuda_pool2D Cuda_upool2D; do
(cd "$OUT/$lib" && for inc in $(grep -ho '#include "[^"]*"' *.cu *.cuh | sed 's/#include "\(.*\)"/\1/' | sort -u); do
    if [ ! -e "$inc" ]; then m=$(ls | grep -i "^$inc$" | head -1); [ -n "$m" ] && ln -s "$m" "$inc"; fi
done; true)
done
for lib in Cuda_conv3D Cuda_dconv3D_deltaX Cuda_dconv3D_deltaW Cuda_reduce Cuda_matMul Cuda_batchMatMul Cuda_pool2D Cuda_upool2D; do
    echo "building $lib ..."
    (cd "$OUT/$lib" && "$NVCC" -gencode arch=compute_100,code=sm_100 -O2 -w -shared -Xcompiler -fPIC \
        -I"$HERE/jni_stub" -o "$HERE/_ref/libcu32_$lib.so" A.cu)
done
ls -la "$HERE"/_ref/libcu32_*.so
