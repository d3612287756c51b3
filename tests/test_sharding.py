"""CPU tests of the batch-sharding layer: world_size-2 gloo ranks, the oracle standing in for the
CUDA engine so that only the host logic (shard bounds, all-reduce of deltaW, buckets) is tested."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleEngine:
    """Engine look-alike on CPU tensors backed by the oracle's loops."""

    def __init__(self, O):
        self.O = O

    def conv3D(self, X, W, sh, sw, ph, pw, Bias=None):
        return torch.from_numpy(self.O.conv3D_naive(X.numpy(), W.numpy(), sh, sw, ph, pw))

    def dconv3D_deltaX(self, dY, W, IH, IW, sh, sw, ph, pw):
        return torch.from_numpy(self.O.deconv3D_deltaX_img2col(dY.numpy(), W.numpy(), IH, IW, sh, sw, ph, pw))

    def dconv3D_deltaW(self, X, dY, FH, FW, sh, sw, ph, pw):
        return torch.from_numpy(self.O.deconv3d_deltaW_naive(X.numpy(), dY.numpy(), FH, FW, sh, sw, ph, pw))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as g
    import oracle as O
    sharding = g.submodule("sharding")
    rng = np.random.default_rng(3)
    N, IH, IW, IC, OC = 6, 7, 6, 4, 8
    X = torch.from_numpy(rng.standard_normal((N, IH, IW, IC)).astype(np.float32))
    W = torch.from_numpy(rng.standard_normal((OC, 3, 3, IC)).astype(np.float32))
    dY = torch.from_numpy(rng.standard_normal((N, IH, IW, OC)).astype(np.float32))
    sc = sharding.ShardedConv(OracleEngine(O))
    Xs, dYs = sharding.shard_batch(X, rank, world), sharding.shard_batch(dY, rank, world)
    Y = sc.forward(Xs, W, 1, 1, 1, 1)
    dX = sc.deltaX(dYs, W, IH, IW, 1, 1, 1, 1)
    dW, _ = sc.deltaW(Xs, dYs, 3, 3, 1, 1, 1, 1)
    # bucketed variant: two "layers" reduced by one collective
    bucket = sharding.GradientBucket([dW.numel(), 10], torch.device("cpu"))
    bucket.view(0, dW.shape).copy_(sc.engine.dconv3D_deltaW(Xs, dYs, 3, 3, 1, 1, 1, 1))
    bucket.view(1, (10,)).fill_(float(rank + 1))
    bucket.all_reduce(async_op=True)
    bucket.wait()
    # the same bucket reduced piece by piece in backward order, as an overlapped backward pass does
    numels = [12, 40, 7, 64, 20, 33]
    whole, parts = sharding.GradientBucket(numels, torch.device("cpu")), sharding.GradientBucket(numels, torch.device("cpu"))
    g = torch.Generator().manual_seed(100 + rank)
    for i, n in enumerate(numels):
        v = torch.randn(n, generator=g)
        whole.view(i, (n,)).copy_(v)
        parts.view(i, (n,)).copy_(v)
    whole.all_reduce(async_op=False)
    for lo, hi in parts.pieces(3):
        dist.all_reduce(parts.piece_view(lo, hi), op=dist.ReduceOp.SUM)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), Y=Y.numpy(), dX=dX.numpy(), dW=dW.numpy(),
             bW=bucket.view(0, dW.shape).numpy(), b1=bucket.view(1, (10,)).numpy(),
             whole=whole.flat.numpy(), parts=parts.flat.numpy())
    dist.destroy_process_group()


def test_shard_bounds(pkg):
    sh = pkg.submodule("sharding")
    for n in (1, 7, 8, 256, 513):
        for world in (1, 2, 3, 8):
            spans = [sh.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def test_bucket_pieces_cover_the_bucket_in_backward_order(pkg):
    sh = pkg.submodule("sharding")
    for numels in ([12, 40, 7, 64, 20, 33], [4], [1000, 4, 4, 4], [4, 4, 4, 1000], [36864] * 20):
        b = sh.GradientBucket(numels, torch.device("cpu"))
        for n in (1, 2, 3, 4, 8, 64):
            pieces = b.pieces(n)
            assert 1 <= len(pieces) <= min(n, len(numels))
            assert pieces[0][1] == len(numels) and pieces[-1][0] == 0
            assert all(a[0] == c[1] and a[0] < a[1] for a, c in zip(pieces, pieces[1:]))   # contiguous, last layers first
            assert sum(b.piece_view(lo, hi).numel() for lo, hi in pieces) == b.flat.numel()
            for lo, hi in pieces:   # a piece starts at its first layer and is 16-byte aligned like every view
                v = b.piece_view(lo, hi)
                assert v.data_ptr() == b.view(lo, (numels[lo],)).data_ptr() and v.data_ptr() % 16 == 0
        assert b.pieces(1) == [(0, len(numels))]


@pytest.mark.timeout(180)
def test_two_rank_batch_sharding_matches_single_rank(tmp_path, oracle_mod):
    O = oracle_mod
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(3)
    N, IH, IW, IC, OC = 6, 7, 6, 4, 8
    X = rng.standard_normal((N, IH, IW, IC)).astype(np.float32)
    W = rng.standard_normal((OC, 3, 3, IC)).astype(np.float32)
    dY = rng.standard_normal((N, IH, IW, OC)).astype(np.float32)
    Y = O.conv3D_naive(X, W, 1, 1, 1, 1)
    dX = O.deconv3D_deltaX_img2col(dY, W, IH, IW, 1, 1, 1, 1)
    dW64, S = O.deconv3D_deltaW_f64(X, dY, 3, 3, 1, 1, 1, 1)
    r = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % k)) for k in range(world)]
    # forward and deltaX: no communication, the shards concatenate to the full result bit for bit
    assert np.array_equal(np.concatenate([r[0]["Y"], r[1]["Y"]]), Y)
    assert np.array_equal(np.concatenate([r[0]["dX"], r[1]["dX"]]), dX)
    # deltaW: summed over ranks, identical on every rank, equal to the full-batch result up to order
    assert np.array_equal(r[0]["dW"], r[1]["dW"])
    assert (np.abs(r[0]["dW"] - dW64) <= 1e-6 * S + 1e-30).all()
    assert np.array_equal(r[0]["bW"], r[0]["dW"])
    assert np.array_equal(r[0]["b1"], np.full(10, 3.0, np.float32))
    # reducing the bucket in pieces gives the same bits as reducing it whole, on every rank
    assert np.array_equal(r[0]["whole"], r[0]["parts"]) and np.array_equal(r[0]["parts"], r[1]["parts"])
    assert np.abs(r[0]["whole"]).max() > 0
