"""Host-side logic of the multi-GPU path: how a batch is split over ranks and how the weight gradient is combined.

Images are independent, so forward, dX and quantised inference shard over the batch with no communication; only the
weight gradient of a training step is a sum over all images and is all-reduced (SUM) after the update transform,
which is linear and yields the smallest tensor of the dW chain (K*9*C values instead of 36*K*C).
The reference has no multi-GPU code at all (its only inter-device traffic is cudaMemcpy, src/descriptors.cu:107-142).
"""


def shard_bounds(batch, world_size, rank):
    """Half-open image range [first, last) of `rank` when `batch` images are split as evenly as possible."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, extra = divmod(batch, world_size)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def all_reduce_weight_gradient(dw, group=None):
    """In-place SUM all-reduce of a rank's partial dW (a torch tensor on CPU for gloo, on the GPU for NCCL)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dw, op=dist.ReduceOp.SUM, group=group)
    return dw
