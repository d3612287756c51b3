"""Batch-sharded multi-GPU layer: one process per GPU, torch.distributed for the plumbing.

Dragon-Alpha itself is single-GPU; this layer is new.  Forward and deltaX are independent per image,
so every rank runs them on its own slice of the batch with no communication.  deltaW is a sum over
the batch: every rank computes the partial gradient of its slice and the partials are summed with
one all-reduce (NCCL over NVLink on GPUs, gloo in the CPU tests).  The sum, not the mean, is taken
so that the result equals the single-GPU deltaW up to fp32 summation order.
"""
import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """Images [lo, hi) of a batch of n owned by `rank`; the first n % world ranks get one extra."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(t, rank, world):
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi]


class GradientBucket:
    """Flat fp32 buffer that deltaW tensors of several layers are carved from, reduced in one
    collective.  Kernels write their deltaW straight into views of the buffer (no packing copy)."""

    def __init__(self, numels, device):
        self.offsets = []
        total = 0
        for n in numels:
            self.offsets.append(total)
            total += (n + 3) & ~3  # keep every view 16-byte aligned
        self.flat = torch.zeros(total, dtype=torch.float32, device=device)
        self.numels = list(numels)
        self._work = None

    def view(self, i, shape):
        o = self.offsets[i]
        return self.flat[o:o + self.numels[i]].view(shape)

    def pieces(self, n):
        """The bucket as at most n contiguous runs of layers of about equal size, LAST layers first - the order in
        which a backward pass completes its weight gradients - as (first layer, last layer + 1) pairs.  Reducing
        piece after piece on a communication stream, each as soon as its layers' deltaW kernels are enqueued,
        overlaps the collective with the rest of the backward pass."""
        n = max(1, int(n))
        total = sum(self.numels)
        out, end, acc = [], len(self.numels), 0
        for i in range(len(self.numels) - 1, -1, -1):
            acc += self.numels[i]
            if acc >= total / n or i == 0:
                out.append((i, end))
                end, acc = i, 0
        return out

    def piece_view(self, lo, hi):
        """Flat view of the layers lo .. hi - 1 (with the alignment padding between them)."""
        a = self.offsets[lo]
        b = self.offsets[hi] if hi < len(self.offsets) else self.flat.numel()
        return self.flat[a:b]

    def all_reduce(self, group=None, async_op=True):
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            self._work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        return self._work

    def wait(self):
        if self._work is not None:
            self._work.wait()
            self._work = None


class ShardedConv:
    """The three contractions of one conv layer on this rank's batch shard.

    `engine` is any object with conv3D / dconv3D_deltaX / dconv3D_deltaW methods of the Engine
    class; the CPU tests pass an oracle-backed stand-in so that the sharding logic itself is covered
    without a GPU.
    """

    def __init__(self, engine, group=None):
        self.engine = engine
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def forward(self, X_shard, W, sh, sw, ph, pw, Bias=None):
        return self.engine.conv3D(X_shard, W, sh, sw, ph, pw, Bias=Bias)

    def deltaX(self, dY_shard, W, IH, IW, sh, sw, ph, pw):
        return self.engine.dconv3D_deltaX(dY_shard, W, IH, IW, sh, sw, ph, pw)

    def deltaW(self, X_shard, dY_shard, FH, FW, sh, sw, ph, pw, async_op=False):
        """Partial deltaW of the shard, summed over all ranks.  Returns (tensor, work-or-None)."""
        dW = self.engine.dconv3D_deltaW(X_shard, dY_shard, FH, FW, sh, sw, ph, pw)
        if not dW.is_contiguous():
            dW = dW.contiguous()
        work = None
        if self.world > 1:
            work = dist.all_reduce(dW, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        return dW, work
