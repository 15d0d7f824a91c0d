"""Batch sharding helpers for one-process-per-GPU runs.

Every operator of the hot path is independent per row and rows are batch-major
(src/cuda/shiftKernels.h:128-131 indexes delays by neuron only), so a batch splits across
ranks with no communication on the data path.  The only exchange a training step needs is
one all-reduce(SUM) of parameter gradients: the reference's losses are sums over the batch
(src/spikeLoss.py:58, :104) and so is the delay gradient (src/slayer.py:954), hence SUM and
not the mean that DistributedDataParallel would apply.
"""
import torch
import torch.distributed as dist


def shard_bounds(n, rank, world):
    """[lo, hi) of the contiguous slice of n batch samples that `rank` owns (sizes differ by <= 1)."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(tensor, rank=None, world=None):
    """This rank's contiguous slice of dimension 0."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    lo, hi = shard_bounds(tensor.shape[0], rank, world)
    return tensor[lo:hi].contiguous()


def allreduce_sum_(tensors, group=None):
    """In-place all-reduce(SUM) of a list of gradient tensors, flattened into one message."""
    tensors = [t for t in tensors if t is not None]
    if not tensors or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return tensors
    flat = torch.cat([t.reshape(-1) for t in tensors])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for t in tensors:
        t.copy_(flat[off:off + t.numel()].view_as(t))
        off += t.numel()
    return tensors
