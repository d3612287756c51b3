"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset ships with this repository; every tensor is regenerated from a seed.  Layouts are
Dragon-Alpha's: NHWC activations, W[OC,FH,FW,IC].
"""
import numpy as np

# 3x3 stride-1 pad-1 layer sweep at batch 256: (H=W, C_in=C_out)
SWEEP_LAYERS = [(56, 64), (28, 128), (14, 256), (7, 512)]
SWEEP_BATCH = 256


def conv_flops(N, OH, OW, OC, FH, FW, IC):
    """Dense multiply-add count of one forward / deltaX / deltaW call (2*GN*GM*GK, the count the
    reference's own speed tests use: experiments/test_cuda/Cuda_conv3D_test.java:138-139)."""
    return 2.0 * N * OH * OW * OC * FH * FW * IC


def conv_bytes(N, IH, IW, IC, OH, OW, OC, FH, FW):
    """Algorithmic bytes of one call: each of X, W, Y touched once."""
    return 4.0 * (N * IH * IW * IC + OC * FH * FW * IC + N * OH * OW * OC)


def sweep_layer(hw, c, batch=SWEEP_BATCH, seed=0):
    """One layer of the 3x3 sweep: X = ReLU(N(0,1)), W He-normal, deltaY ~ N(0,1)."""
    rng = np.random.Generator(np.random.Philox(seed * 1000003 + hw * 1009 + c))
    X = np.maximum(rng.standard_normal((batch, hw, hw, c), dtype=np.float32), 0)
    W = rng.standard_normal((c, 3, 3, c), dtype=np.float32) * np.float32(np.sqrt(2.0 / (9 * c)))
    dY = rng.standard_normal((batch, hw, hw, c), dtype=np.float32)
    return X, W, dY


def single_conv(seed=0):
    """Configuration 1: X[4,32,32,16], W[32,3,3,16] uniform[-1,1], bias[32] uniform[-0.1,0.1]."""
    rng = np.random.Generator(np.random.Philox(seed + 11))
    X = rng.uniform(-1, 1, (4, 32, 32, 16)).astype(np.float32)
    W = rng.uniform(-1, 1, (32, 3, 3, 16)).astype(np.float32)
    B = rng.uniform(-0.1, 0.1, (32,)).astype(np.float32)
    return X, W, B


# ResNet-18-shaped conv stack on 32x32 images, the 20 convolutions of the reference's CIFAR-10 network
# (experiments/alpha_code/src/cifar10/resnet18/Net.java:24-77) in forward order: (IH, IC, OC, F, stride, pad).
# Every convolution is unbiased (nn.conv3D(false, ...)); the shortcut of a down-sampling block is a 3x3
# stride-2 convolution there (Net.java:30-34), not a 1x1 one.  The stem's 3 colour planes arrive padded to 4.
def _basic_block(ih, cin, cout, stride):
    oh = ih // stride
    convs = [(ih, cin, cout, 3, stride, 1), (oh, cout, cout, 3, 1, 1)]
    if stride != 1 or cin != cout:
        convs.append((ih, cin, cout, 3, stride, 1))
    return convs


RESNET18_CONVS = (
    [(32, 4, 64, 7, 2, 3)]
    + _basic_block(16, 64, 64, 1) + _basic_block(16, 64, 64, 1)
    + _basic_block(16, 64, 128, 2) + _basic_block(8, 128, 128, 1)
    + _basic_block(8, 128, 256, 2) + _basic_block(4, 256, 256, 1)
    + _basic_block(4, 256, 512, 2) + _basic_block(2, 512, 512, 1)
)
# 1x1 stride-2 shortcuts (the usual ResNet form), kept as parity-test shapes
SHORTCUT_1X1_CONVS = [(16, 64, 128, 1, 2, 0), (8, 128, 256, 1, 2, 0), (4, 256, 512, 1, 2, 0)]
RESNET18_BATCH = 512

# DCGAN-style generator as transposed convolutions: (IH_in, C_in, C_out), 4x4 stride 2 pad 1
DCGAN_DECONVS = [(4, 512, 256), (8, 256, 128), (16, 128, 64), (32, 64, 4)]
