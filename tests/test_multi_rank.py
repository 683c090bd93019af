"""CPU tests (gloo, world size 2) of the multi-GPU host logic: batch sharding and the dW all-reduce.

Each rank computes, with the CPU oracle, the outputs and the partial weight gradient of its own shard; the shards of
y must tile the full-batch y exactly and the all-reduced dW must equal the full-batch dW.  No GPU is involved: the
per-rank GPU work is the single-GPU path the other tests cover.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from cudabackend_b200 import sharding


def test_shard_bounds_cover_the_batch():
    for batch in (0, 1, 7, 64, 255, 256):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharding.shard_bounds(batch, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == batch
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, queue):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle as o
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        r = np.random.default_rng(0)
        n, h, w, c, k = 5, 8, 8, 6, 4  # 5 images over 2 ranks: uneven shards
        x = r.uniform(-1, 1, (n, h, w, c))
        wt = r.normal(0, 0.3, (k, 3, 3, c))
        dy = r.uniform(-1, 1, (n, h, w, k))
        a, b = sharding.shard_bounds(n, world, rank)
        y_shard = o.conv2d_forward(x[a:b], wt)
        # the Winograd dW chain of one shard: gradient + input transform, contraction over the shard's tiles, update
        g = o.winograd_gradient_transform(dy[a:b], 4, 3)
        v = o.winograd_input_transform(x[a:b], 4, 3)
        dw = torch.from_numpy(o.winograd_update_transform(o.gemm_batched(g, v, trans_a=True), 4, 3))
        sharding.all_reduce_weight_gradient(dw)
        full_dw = o.conv2d_backward_weights(x, dy)
        full_y = o.conv2d_forward(x, wt)
        queue.put((rank, float(np.abs(dw.numpy() - full_dw).max()), float(np.abs(y_shard - full_y[a:b]).max())))
    finally:
        dist.destroy_process_group()


def test_sharded_training_step_matches_full_batch():
    import torch.multiprocessing as mp
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(rank, world, port, queue)) for rank in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, dw_err, y_err in results:
        assert dw_err < 1e-11, (rank, dw_err)
        assert y_err == 0.0, (rank, y_err)
