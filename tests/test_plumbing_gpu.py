"""GPU tests of the descriptor plumbing (reference src/descriptors.cu:48-253)."""
import ctypes

import numpy as np
import pytest

from cudabackend_b200 import api

pytestmark = pytest.mark.gpu


def test_memory_copy_round_trip_and_views(ctx):
    data = np.arange(4096, dtype=np.float32)
    mem = api.Memory(data.nbytes)
    mem.from_host(ctx, data)
    back = np.empty_like(data)
    mem.to_host(ctx, back)
    ctx.synchronize()
    assert np.array_equal(back, data)
    view = mem.view(1024, 2048)
    part = np.empty(256, dtype=np.float32)
    view.to_host(ctx, part)
    ctx.synchronize()
    assert np.array_equal(part, data[512:768])
    # a view of a view is refused, like a negative offset
    h = ctypes.c_int64(-1)
    assert api.call_status("cudaCreateMemoryView", ctypes.byref(h), view.handle, 16, 0) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaCreateMemoryView", ctypes.byref(h), mem.handle, 16, -4) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaCreateMemoryView", ctypes.byref(h), mem.handle, 16, data.nbytes) == api.STATUS["BAD_PARAM"]


@pytest.mark.parametrize("pattern_size", [1, 2, 4, 8, 16])
def test_set_memory_patterns(ctx, pattern_size):
    mem = api.Memory(4096)
    mem.zero(ctx)
    pattern = bytes(range(1, pattern_size + 1))
    buf = ctypes.create_string_buffer(pattern, pattern_size)
    api.call("cudaSetMemory", ctx.handle, mem.handle, 1024, 2048, ctypes.cast(buf, ctypes.c_void_p), pattern_size)
    out = np.empty(4096, dtype=np.uint8)
    mem.to_host(ctx, out)
    ctx.synchronize()
    assert not out[:1024].any() and not out[3072:].any()
    assert out[1024:3072].tobytes() == pattern * (2048 // pattern_size)
    assert api.call_status("cudaSetMemory", ctx.handle, mem.handle, 0, 100, ctypes.cast(buf, ctypes.c_void_p), 3) == api.STATUS["BAD_PARAM"]


def test_device_copy_and_default_context(library, device_count):
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    ctx = api.Context.default(0)
    a = api.Memory(1024)
    b = api.Memory(1024)
    data = np.random.default_rng(0).integers(0, 255, 1024, dtype=np.uint8)
    a.from_host(ctx, data)
    api.call("cudaCopyMemory", ctx.handle, b.handle, 0, a.handle, 0, 1024)
    out = np.empty_like(data)
    b.to_host(ctx, out)  # synchronous on a default context
    assert np.array_equal(out, data)
    assert api.call_status("cudaDestroyContextDescriptor", ctx.handle) == api.STATUS["BAD_PARAM"]
    possible = ctypes.c_bool(False)
    api.call("cudaIsCopyPossible", 0, 0, ctypes.byref(possible))
    assert possible.value


def test_context_ready_and_properties(ctx):
    ctx.synchronize()
    assert ctx.is_ready()
    name = ctypes.create_string_buffer(256)
    api.call("cudaGetDeviceProperty", 0, 0, ctypes.cast(name, ctypes.c_void_p))
    assert len(name.value) > 0
    sms = (ctypes.c_int32 * 64)()
    api.call("cudaGetDeviceProperty", 0, 1, ctypes.cast(sms, ctypes.c_void_p))
    assert sms[0] > 0
    assert ctx.last_device_status() == 0


def test_contexts_can_be_ordered_without_blocking_the_host(library, device_count):
    """cudaContextWaitForContext: work on one context runs after work on another; also as parallel branches of a captured graph"""
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    import numpy as np
    from cudabackend_b200 import pipeline
    from oracle import oracle as o
    from tests import common
    main, side = api.Context(0), api.Context(0)
    p = pipeline.WinogradNonFused(main, 4, 16, 16, 64, 64, "float16", "float32", 4, 3, side_ctx=side)
    x = p.x.upload(main, common.uniform("x", p.x.shape))
    w1 = common.he_normal_weights(64, 3, 64)
    wt = p.wt.upload(main, w1)
    main.synchronize()
    p.forward()                                     # weight transform on `side`, joined before the contraction
    ref = o.conv2d_forward(x, wt)
    assert o.error_metrics(p.y.download(main), ref)["elem"] <= 1e-2
    graph = main.capture(p.forward)                 # the same with the side branch captured into the graph
    for scale in (2.0, -0.5):
        wt = p.wt.upload(main, w1 * scale)
        p.y.mem.zero(main)
        main.synchronize()
        graph.launch()
        main.synchronize()
        assert o.error_metrics(p.y.download(main), o.conv2d_forward(x, wt))["elem"] <= 1e-2
    graph.destroy()
    side.destroy()
    main.destroy()


def test_two_threads_with_their_own_contexts(library, device_count):
    """Handles, pools and per-device one-time set-up are shared by all threads of a process: two threads, each with its own
    context and tensors, run convolutions at the same time and must both get the right answer."""
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    import threading
    from cudabackend_b200 import pipeline
    from oracle import oracle as o
    from tests import common
    failures = []

    def worker(index):
        try:
            ctx = api.Context(0)
            shape = [(3, 12, 14, 64, 72), (2, 17, 9, 40, 64)][index]
            n, h, w, c, k = shape
            d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "float16")
            x = d.x.upload(ctx, common.uniform(["x", "z"][index], d.x.shape))
            wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
            ref = o.conv2d_forward(x, wt, activation="relu")
            for repeat in range(25):
                d.y.mem.zero(ctx)
                (d.winograd_fused if repeat % 2 else d.implicit_gemm)(activation="relu")
                err = o.error_metrics(d.y.download(ctx), ref)["elem"]
                if err > 1e-2:
                    failures.append((index, repeat, err))
            if ctx.last_device_status() != 0:
                failures.append((index, "device status"))
            ctx.destroy()
        except Exception as error:  # noqa: BLE001 - reported through the list, the main thread asserts
            failures.append((index, repr(error)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures
