"""CPU tests (gloo, world size 2) of what a rank does when the collective of the training step cannot complete.

No GPU is involved and nothing is made to fault: the failures are made on the host.  Three cases:
  * the ranks disagree on the gradient they are about to reduce -> every rank raises before any data collective;
  * a rank leaves cleanly between two steps -> its peer learns of it from the store before issuing the next all-reduce;
  * a rank dies without a word between two steps -> its peer's wait for it to enter the next step runs out (a short,
    bounded wait on the host), and a collective issued all the same ends with an error instead of hanging.
"""
import datetime
import os
import socket
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=20):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    return dist


def _mismatch_worker(rank, world, port, queue):
    dist = _init(rank, world, port)
    import torch
    from cudabackend_b200 import sharding
    try:
        dw = torch.ones(36864 if rank == 0 else 36800, dtype=torch.float32)  # rank 1 built its layer with another shape
        try:
            sharding.checked_all_reduce_weight_gradient(dw)
            queue.put((rank, "reduced"))
        except sharding.CollectiveMismatch:
            # nothing was reduced: the buffer is untouched
            queue.put((rank, "mismatch" if float(dw.sum()) == dw.numel() else "corrupted"))
        # the group is still usable after the refusal
        ok = torch.ones(4)
        sharding.checked_all_reduce_weight_gradient(ok)
        queue.put((rank, "then %d" % int(ok[0])))
    finally:
        dist.destroy_process_group()


def _leave_worker(rank, world, port, queue):
    dist = _init(rank, world, port)
    import torch
    from cudabackend_b200 import sharding
    store = dist.distributed_c10d._get_default_store()
    watch = sharding.RankWatch(store, rank, world, timeout=5.0)
    try:
        for step in range(3):
            if step == 2 and rank == 1:
                watch.leave()  # between steps: nothing of this rank is in flight
                queue.put((rank, "left before step 2"))
                return
            try:
                watch.enter_step(step)
            except sharding.PeerLeft as error:
                queue.put((rank, "stopped before step %d: %s" % (step, error)))
                return
            dw = torch.full((8,), float(rank + 1))
            sharding.all_reduce_weight_gradient(dw)
            assert float(dw[0]) == 3.0
        queue.put((rank, "ran all steps"))
    finally:
        # no destroy_process_group(): it is a collective itself, and the peer is gone
        pass


def _vanish_worker(rank, world, port, queue):
    dist = _init(rank, world, port, timeout_s=4)
    import torch
    from cudabackend_b200 import sharding
    store = dist.distributed_c10d._get_default_store()
    watch = sharding.RankWatch(store, rank, world, timeout=1.0)
    watch.enter_step(0)
    dw = torch.ones(8)
    sharding.all_reduce_weight_gradient(dw)  # step 0 works
    if rank == 1:
        os._exit(0)  # dies between steps without a word
    t0 = time.monotonic()
    try:
        watch.enter_step(1)  # rank 1 never enters step 1
        queue.put((rank, "no failure seen"))
    except sharding.PeerLeft:
        waited = time.monotonic() - t0
        # a collective issued all the same must end with an error within the group's timeout, not hang
        t1 = time.monotonic()
        try:
            sharding.all_reduce_weight_gradient(torch.ones(8))
            outcome = "collective completed"
        except Exception:
            outcome = "collective failed"
        queue.put((rank, "peer lost after %.1f s; %s after %.1f s" % (waited, outcome, time.monotonic() - t1)))
    queue.close()
    queue.join_thread()  # the result must be on its way before this process ends without the usual clean-up
    os._exit(0)


def _run(worker, world=2, expect=2, timeout=90):
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(rank, world, port, queue)) for rank in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=timeout) for _ in range(expect)]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    return results


def test_size_mismatch_is_refused_on_every_rank_before_the_collective():
    results = _run(_mismatch_worker, expect=4)
    by_rank = {0: [], 1: []}
    for rank, what in results:
        by_rank[rank].append(what)
    for rank in (0, 1):
        assert by_rank[rank] == ["mismatch", "then 2"], by_rank


def test_rank_that_leaves_between_steps_is_seen_before_the_next_collective():
    results = dict(_run(_leave_worker, expect=2))
    assert results[1] == "left before step 2"
    assert results[0].startswith("stopped before step 2: rank 1 has left"), results


def test_rank_that_vanishes_is_caught_by_a_bounded_host_wait():
    results = _run(_vanish_worker, expect=1, timeout=60)
    rank, what = results[0]
    assert rank == 0 and what.startswith("peer lost after"), results
    assert "collective failed" in what, results
