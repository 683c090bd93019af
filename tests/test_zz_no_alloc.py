"""GPU test of cudaConvolutionWinogradFusedForwardNoAlloc, the entry point for callers that may not allocate.

A serving process that has given the whole GPU to its own memory pool, or that is forbidden to allocate once it is
running, cannot use cudaConvolutionWinogradFusedForward: that call cudaMalloc's the context's scratch buffer on first
use.  The NoAlloc variant keeps the scratch in a fixed array inside the library, so it must (1) give exactly the
result of the allocating entry point, (2) keep doing so when called again on the array the previous call left
behind, and (3) refuse, rather than trim, a problem that does not fit the array.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu


def build(ctx, n, h, w, c, k, dtype, seed):
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape, extra=seed))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c, extra=seed))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1, extra=seed))
    z = d.set_z(common.uniform("z", d.y.shape, extra=seed))
    return d, x, wt, b, z


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_no_alloc_matches_allocating_entry_point_twice_in_a_row(ctx, dtype):
    f = lambda v: float(np.float32(v))
    # two different layers, back to back: the second call finds the first one's data in the shared array
    for seed, (n, h, w, c, k) in enumerate([(2, 16, 16, 64, 64), (3, 13, 10, 32, 96)]):
        d, x, wt, b, z = build(ctx, n, h, w, c, k, dtype, seed)
        y0 = common.uniform("y", d.y.shape, extra=seed)

        d.y.upload(ctx, y0)
        d.winograd_fused(alpha1=1.1, alpha2=1.2, beta=0.1, activation="relu")
        expected = d.y.download_raw(ctx)

        d.y.upload(ctx, y0)
        d.winograd_fused_no_alloc(alpha1=1.1, alpha2=1.2, beta=0.1, activation="relu")
        got = d.y.download_raw(ctx)

        # same kernels in the same order: the two entry points agree bit for bit ...
        assert np.array_equal(got, expected)
        # ... and no bounded wait ran out on either path (the fixed array's own error word is read here too)
        assert ctx.last_device_status() == 0
        # ... and both are within the stated tolerance of the float64 oracle
        y0_stored = api.to_storage(y0, dtype)[1]
        ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y0_stored, alpha1=f(1.1), alpha2=f(1.2), beta=f(0.1), activation="relu")
        assert o.error_metrics(api.from_storage(got, dtype), ref)["elem"] <= common.TOLERANCE[dtype]


def test_no_alloc_second_call_takes_no_device_memory(ctx):
    """The claim in the name: once the first call on the device has been made, further calls leave the amount of free
    device memory exactly where it was (the array and the kernels were placed by that first call)."""
    torch = pytest.importorskip("torch")
    d, _, _, _, _ = build(ctx, 2, 16, 16, 64, 64, "float16", 5)
    d.winograd_fused_no_alloc(activation="relu")
    ctx.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        d.winograd_fused_no_alloc(activation="relu")
    ctx.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before


def test_no_alloc_two_kernel_form_when_y_is_misaligned(ctx):
    """y eight bytes off a 16-byte boundary: the single-kernel contraction + output transform does not apply, both entry
    points write the products out and run the output transform as a kernel of its own -- still bit-identical."""
    d, x, wt, b, z = build(ctx, 2, 12, 12, 32, 32, "float16", 7)
    backing = api.Memory(d.y.desc.nbytes + 16, 0)
    aligned_mem, d.y.mem = d.y.mem, backing.view(d.y.desc.nbytes, 8)
    d.winograd_fused(alpha2=0.5, activation="relu")
    expected = d.y.download_raw(ctx)
    d.y.mem.zero(ctx)
    d.winograd_fused_no_alloc(alpha2=0.5, activation="relu")
    got = d.y.download_raw(ctx)
    assert np.array_equal(got, expected)
    ref = o.conv2d_forward(x, wt, bias=b, z=z, alpha2=0.5, activation="relu")
    assert o.error_metrics(api.from_storage(got, "float16"), ref)["elem"] <= common.TOLERANCE["float16"]
    assert ctx.last_device_status() == 0
    d.y.mem = aligned_mem


def test_no_alloc_error_word_reaches_the_caller(ctx):
    """A bounded wait that runs out on this path is recorded in a word inside the fixed array; cudaGetLastDeviceStatus
    must report it (and clear it) like the context's own word.  The self test makes such a wait run out harmlessly."""
    d, _, _, _, _ = build(ctx, 1, 8, 8, 32, 32, "float16", 9)
    d.winograd_fused_no_alloc()  # resolves the array's address on this device
    assert ctx.last_device_status() == 0
    api.call("cudaRunBoundedWaitSelfTestNoAlloc", ctx.handle, 200)
    assert ctx.last_device_status() == 1 << 5
    assert ctx.last_device_status() == 0
    d.winograd_fused_no_alloc()  # the path still works afterwards
    assert ctx.last_device_status() == 0


def test_no_alloc_rejects_what_does_not_fit(ctx):
    # 16 * 2 * (K*C + tiles*C) with tiles = 8*28*28 is about 13 MB, beyond the 8 MiB array
    d, _, _, _, _ = build(ctx, 8, 56, 56, 64, 64, "float16", 0)
    need = 32 * (64 * 64 + 8 * 28 * 28 * 64)
    assert need > api.NO_ALLOC_SCRATCH_BYTES
    with pytest.raises(api.AvocadoError) as failure:
        d.winograd_fused_no_alloc()
    assert failure.value.status == api.STATUS["BAD_PARAM"]
    # float32 tensors are outside this entry point
    d32 = pipeline.DirectConvolution(ctx, 1, 8, 8, 16, 16, "float32")
    with pytest.raises(api.AvocadoError) as failure:
        d32.winograd_fused_no_alloc()
    assert failure.value.status == api.STATUS["UNSUPPORTED_DATATYPE"]
