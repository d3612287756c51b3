"""Two GPUs, one process each over NCCL: the batch-sharded layer with the real CUDA engine.

Each rank runs forward, deltaX and deltaW on its slice of the batch; deltaW goes straight into a view
of a GradientBucket and is summed over the ranks with one all-reduce.  The sharded results are
compared with the fp64 oracle of the FULL batch at the parity bounds.  Skipped on a box with one GPU.
No kernel of this library touches another GPU's memory: the exchange is NCCL's all-reduce.
"""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# (N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw); 11 images over 2 ranks is the ragged case (6 + 5)
CASES = [(16, 14, 14, 64, 128, 3, 3, 1, 1, 1, 1), (11, 16, 16, 32, 64, 3, 3, 2, 2, 1, 1)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(case, seed):
    N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
    OH, OW = (IH + 2 * ph - FH) // sh + 1, (IW + 2 * pw - FW) // sw + 1
    rng = np.random.default_rng(seed)
    X = rng.uniform(-1, 1, (N, IH, IW, IC)).astype(np.float32)
    W = rng.uniform(-1, 1, (OC, FH, FW, IC)).astype(np.float32)
    dY = rng.standard_normal((N, OH, OW, OC)).astype(np.float32)
    return X, W, dY


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import __graft_entry__ as g
    sharding = g.submodule("sharding")
    lib = g.submodule("lib")
    lib.set_math_mode("3xtf32")
    eng = g.submodule("engine").Engine()
    sc = sharding.ShardedConv(eng)
    out = {}
    shapes = [(c[4], c[5], c[6], c[3]) for c in CASES]
    bucket = sharding.GradientBucket([int(np.prod(s)) for s in shapes], dev)
    for i, case in enumerate(CASES):
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        X, W, dY = (torch.from_numpy(a).to(dev) for a in _inputs(case, 40 + i))
        Xs, dYs = sharding.shard_batch(X, rank, world).contiguous(), sharding.shard_batch(dY, rank, world).contiguous()
        out["Y%d" % i] = sc.forward(Xs, W, sh, sw, ph, pw).cpu().numpy()
        out["dX%d" % i] = sc.deltaX(dYs, W, IH, IW, sh, sw, ph, pw).cpu().numpy()
        # the kernel writes its partial gradient straight into the bucket view
        view = bucket.view(i, shapes[i])
        eng.base.dconv3D_deltaW(view, FH, FW, Xs, IH, IW, dYs, dYs.shape[1], dYs.shape[2], Xs.shape[0], IC, OC, sh, sw, ph, pw)
    bucket.all_reduce(async_op=True)
    bucket.wait()
    torch.cuda.synchronize()
    for i in range(len(CASES)):
        out["dW%d" % i] = bucket.view(i, shapes[i]).cpu().numpy()
    out["status"] = np.array([lib.device_status()])
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **out)
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_sharded_layer_against_the_full_batch_oracle(tmp_path, oracle_mod):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    O = oracle_mod
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % k)) for k in range(world)]
    assert int(r[0]["status"][0]) == 0 and int(r[1]["status"][0]) == 0
    for i, case in enumerate(CASES):
        N, IH, IW, IC, OC, FH, FW, sh, sw, ph, pw = case
        X, W, dY = _inputs(case, 40 + i)
        Y64, SY = O.conv3D_f64(X, W, sh, sw, ph, pw, threads=8)
        dX64, SX = O.deconv3D_deltaX_f64(dY, W, IH, IW, sh, sw, ph, pw, threads=8)
        dW64, SW = O.deconv3D_deltaW_f64(X, dY, FH, FW, sh, sw, ph, pw, threads=8)
        Y = np.concatenate([r[0]["Y%d" % i], r[1]["Y%d" % i]])
        dX = np.concatenate([r[0]["dX%d" % i], r[1]["dX%d" % i]])
        assert Y.shape == Y64.shape and dX.shape == dX64.shape
        for got, ref, S in ((Y, Y64, SY), (dX, dX64, SX), (r[0]["dW%d" % i], dW64, SW)):
            err = np.abs(got - ref)
            assert err.max() <= 1e-4 * np.abs(ref).max() and (err <= 1e-5 * S + 1e-30).all(), (i, err.max())
        # every rank holds the same reduced gradient
        assert np.array_equal(r[0]["dW%d" % i], r[1]["dW%d" % i])
