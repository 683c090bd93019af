"""Failure detection without a GPU fault.

Every wait inside the tensor-core kernels is bounded; when one runs out the kernel records an error bit in the
context's device status word and returns.  The self test below makes such a wait run out on purpose (a barrier that
nothing signals, limit 200 microseconds), then checks that the bit is reported, that reading it clears it, and that
the same context still computes a correct product afterwards.  Host-side failures (bad handles, bad shapes) are
rejected before any launch; tests/test_abi.py covers those on the CPU.
"""
import time

import numpy as np
import pytest

from cudabackend_b200 import api
from oracle import oracle as o

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_context_survives(library, device_count):
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    ctx = api.Context(0)
    assert ctx.last_device_status() == 0
    t0 = time.perf_counter()
    api.call("cudaRunBoundedWaitSelfTest", ctx.handle, 200)
    ctx.synchronize()
    assert time.perf_counter() - t0 < 5.0  # the kernel gave up on its own
    assert ctx.last_device_status() == 1 << 5
    assert ctx.last_device_status() == 0  # reading clears

    # the context is intact: a tensor-core product right after is correct
    r = np.random.default_rng(3)
    a = r.uniform(-1, 1, (4, 256, 64))
    b = r.uniform(-1, 1, (4, 64, 64))
    A, B, C = api.DeviceTensor(a.shape, "float16"), api.DeviceTensor(b.shape, "float16"), api.DeviceTensor((4, 256, 64), "float16")
    a64, b64 = A.upload(ctx, a), B.upload(ctx, b)
    api.call("cudaGemmBatched", ctx.handle, api.GEMM_N, api.GEMM_T, None, A.desc.handle, A.mem.handle, B.desc.handle, B.mem.handle, None, C.desc.handle,
             C.mem.handle)
    assert o.error_metrics(C.download(ctx), o.gemm_batched(a64, b64, False, True))["elem"] <= 1e-3
    assert ctx.last_device_status() == 0
    ctx.destroy()


def test_self_test_rejects_silly_limits(ctx):
    assert api.call_status("cudaRunBoundedWaitSelfTest", ctx.handle, 0) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaRunBoundedWaitSelfTest", -1, 100) == api.STATUS["INTERNAL_ERROR"]
