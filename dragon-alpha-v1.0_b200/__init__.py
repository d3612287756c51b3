"""B200 (sm_100a) drop-in for Dragon-Alpha's cu32 convolution path.

The product is libalpha_conv_b200.so (csrc/), a C-ABI library of hand-written tcgen05/TMA kernels
for conv3D forward, dconv3D_deltaX and dconv3D_deltaW on NHWC fp32 tensors.  The Python modules are
the host-side mirror of the reference's Java operator interface, used by the tests and the
benchmark:

    lib       ctypes binding of the C ABI
    engine    CudaFloat32EngineBase / Engine operator methods
    sharding  batch-sharded multi-GPU layer (forward / deltaX local, deltaW all-reduced)
    synth     seeded synthetic inputs for the benchmark configurations
"""
from . import lib  # noqa: F401
