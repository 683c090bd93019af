"""GPU test of the one collective on the path: the NCCL all-reduce of dW in the batch-sharded training step.

Two ranks, one GPU each (skipped on a box with fewer than two).  Each rank runs forward, dW and dX of ITS shard of a
small batch through the C ABI, all-reduces its partial dW in place through a zero-copy view of the library's memory
(cudaGetMemoryPointer), and rank 0 compares: the reduced dW with the oracle's dW of the WHOLE batch, and its y / dx
shard with the matching slice of the whole-batch oracle results.  NVLS is switched off and nothing leaves mid-step.
"""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, queue):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from cudabackend_b200 import api, pipeline, sharding
    from oracle import oracle as o
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        n, h, w, c, k = 10, 24, 20, 64, 64  # 10 images over 2 ranks; 56-wide layers are covered by the single-GPU tests
        r = np.random.default_rng(5)
        x = r.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        wt = r.normal(0, np.sqrt(2.0 / (9 * c)), (k, 3, 3, c)).astype(np.float32)
        dy = r.uniform(-1, 1, (n, h, w, k)).astype(np.float32)
        a, b = sharding.shard_bounds(n, world, rank)
        ctx = api.Context(rank)
        p = pipeline.WinogradNonFused(ctx, b - a, h, w, c, k, "float32", None, 4, 3, device=rank, training=True)
        p.x.upload(ctx, x[a:b])
        p.wt.upload(ctx, wt)
        p.dy.upload(ctx, dy[a:b])
        p.training_step()

        class _View:
            pass
        holder = _View()
        holder.__cuda_array_interface__ = {"shape": p.dw.shape, "typestr": "<f4", "data": (p.dw.mem.pointer(), False), "version": 3}
        grad = torch.as_tensor(holder, device=torch.device("cuda", rank))
        stream = torch.cuda.ExternalStream(ctx.stream(), device=rank)
        with torch.cuda.stream(stream):  # on the library's stream: ordered after the update transform
            sharding.checked_all_reduce_weight_gradient(grad)
        ctx.synchronize()
        dw = p.dw.download(ctx)
        y = p.y.download(ctx)
        dx = p.dx.download(ctx)
        status = ctx.last_device_status()
        x64, w64, dy64 = x.astype(np.float64), wt.astype(np.float64), dy.astype(np.float64)
        errors = {"dw": o.error_metrics(dw, o.conv2d_backward_weights(x64, dy64))["elem"],
                  "y": o.error_metrics(y, o.conv2d_forward(x64, w64)[a:b])["elem"],
                  "dx": o.error_metrics(dx, o.conv2d_backward_data(dy64, w64, (h, w))[a:b])["elem"]}
        queue.put((rank, errors, status))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_training_step_with_nccl_all_reduce(device_count):
    if device_count < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(rank, world, port, queue)) for rank in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, errors, status in results:
        assert status == 0
        assert errors["dw"] <= 1e-3 and errors["y"] <= 1e-3 and errors["dx"] <= 1e-3, (rank, errors)
