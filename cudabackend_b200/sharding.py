"""Host-side logic of the multi-GPU path: how a batch is split over ranks, how the weight gradient is combined, and
how a rank finds out -- on the host, before it launches anything -- that a peer is gone or disagrees.

Images are independent, so forward, dX and quantised inference shard over the batch with no communication; only the
weight gradient of a training step is a sum over all images and is all-reduced (SUM) after the update transform,
which is linear and yields the smallest tensor of the dW chain (K*9*C values instead of 36*K*C).
The reference has no multi-GPU code at all (its only inter-device traffic is cudaMemcpy, src/descriptors.cu:107-142).

One process drives one GPU; torch.distributed provides the process group (NCCL on GPUs, gloo on CPU for the tests).
Nothing here touches a GPU: the checks are host round trips through the process group's key-value store or a small
host-side gather, made between steps, when none of the rank's kernels or collectives is in flight.
"""
import time


def shard_bounds(batch, world_size, rank):
    """Half-open image range [first, last) of `rank` when `batch` images are split as evenly as possible."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, extra = divmod(batch, world_size)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


class CollectiveMismatch(ValueError):
    """The ranks do not agree on what is about to be reduced (element count or dtype)."""


class PeerLeft(RuntimeError):
    """A peer announced that it has left, or stopped announcing its steps."""


def all_reduce_weight_gradient(dw, group=None):
    """In-place SUM all-reduce of a rank's partial dW (a torch tensor on CPU for gloo, on the GPU for NCCL)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dw, op=dist.ReduceOp.SUM, group=group)
    return dw


def agree_on_gradient(dw, group=None):
    """Checks, with one small host-side gather, that every rank is about to reduce a tensor of the same element count
    and dtype.  A mismatch raises CollectiveMismatch on EVERY rank, before the data collective is issued: an all-reduce
    over unequal buffers would hang or corrupt memory instead of failing."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    mine = (int(dw.numel()), str(dw.dtype))
    everyone = [None] * dist.get_world_size(group)
    dist.all_gather_object(everyone, mine, group=group)
    if any(other != everyone[0] for other in everyone):
        raise CollectiveMismatch("ranks disagree on the gradient to reduce: %s" % (everyone,))


def checked_all_reduce_weight_gradient(dw, group=None):
    """agree_on_gradient() followed by the SUM all-reduce; what a training loop calls once per layer shape."""
    agree_on_gradient(dw, group)
    return all_reduce_weight_gradient(dw, group)


class RankWatch:
    """Step hand-shake through the process group's key-value store.

    Before it enqueues step s, a rank calls enter_step(s): that publishes "I take part in step s" and waits until every
    peer has published the same, or has published that it left.  A rank that stops cleanly calls leave() INSTEAD of
    entering the next step, between steps, with nothing of its own in flight.  enter_step raises PeerLeft when a peer
    has left or has not entered the step within `timeout` seconds, so the caller stops BEFORE launching a collective
    that would never complete; a peer that dies without a word is caught by the same bounded wait."""

    def __init__(self, store, rank, world_size, timeout=5.0, prefix="rankwatch"):
        self.store = store
        self.rank = rank
        self.world_size = world_size
        self.timeout = timeout
        self.prefix = prefix

    def _key(self, kind, rank):
        return "%s/%s/%d" % (self.prefix, kind, rank)

    def leave(self):
        self.store.set(self._key("left", self.rank), "1")

    def _read(self, key):
        # check() does not block; get() would wait for the store's own (long) timeout on a missing key
        if not self.store.check([key]):
            return None
        return self.store.get(key).decode()

    def enter_step(self, step):
        """Publishes this rank's entry into `step` and returns once every peer has entered it too; raises PeerLeft otherwise."""
        self.store.set(self._key("step", self.rank), str(int(step)))
        deadline = time.monotonic() + self.timeout
        pending = [r for r in range(self.world_size) if r != self.rank]
        while True:
            still = []
            for r in pending:
                entered = self._read(self._key("step", r))
                if entered is not None and int(entered) >= step:
                    continue
                if self._read(self._key("left", r)) is not None:
                    raise PeerLeft("rank %d has left" % r)
                still.append(r)
            if not still:
                return
            if time.monotonic() > deadline:
                raise PeerLeft("rank(s) %s did not enter step %d within %.1f s" % (still, step, self.timeout))
            pending = still
            time.sleep(0.005)
