"""CPU tests of the C-ABI boundary: the shared library loads, exports every symbol the headers declare, and the
descriptor logic that needs no device behaves like the reference's (src/descriptors.cu:255-368)."""
import ctypes
import os
import re

import pytest

from cudabackend_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for header in ("cuda_backend.h", "cuda_backend_ext.h"):
        text = open(os.path.join(ROOT, "include", "Avocado", header)).read()
        names += re.findall(r"DLL_PUBLIC\s+\w+\s+(\w+)\s*\(", text)
    return names


def test_every_declared_symbol_is_exported(library):
    names = declared_symbols()
    assert len(names) >= 68 + 4
    missing = [n for n in names if not hasattr(library, n)]
    assert missing == []


def test_binding_covers_every_declared_symbol():
    assert sorted(set(api.SIGNATURES) | set(api.UNSUPPORTED_SYMBOLS)) == sorted(declared_symbols())


def test_out_of_scope_entry_points_return_not_supported(library):
    for name in api.UNSUPPORTED_SYMBOLS:
        fn = getattr(library, name)
        fn.restype = ctypes.c_int
        # arguments are ignored by these entry points; pass enough zero words for the longest signature
        assert fn(*([ctypes.c_int64(0)] * 6)) == api.STATUS["NOT_SUPPORTED"], name


def test_tensor_descriptor_round_trip(library):
    t = api.TensorDescriptor((12, 13, 14, 135), "float16")
    dtype, nb = ctypes.c_int(-1), ctypes.c_int(-1)
    dims = (ctypes.c_int * 8)()
    api.call("cudaGetTensorDescriptor", t.handle, ctypes.byref(dtype), ctypes.byref(nb), dims)
    assert dtype.value == api.DTYPES["float16"] and nb.value == 4 and list(dims)[:4] == [12, 13, 14, 135]
    too_many = (ctypes.c_int * 9)(*([1] * 9))
    assert api.call_status("cudaSetTensorDescriptor", t.handle, api.DTYPES["float32"], 9, too_many) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaSetTensorDescriptor", t.handle, api.DTYPES["float32"], 2, None) == api.STATUS["BAD_PARAM"]
    handle = t.handle
    t.destroy()
    # a destroyed handle is rejected, and the slot's next owner gets a different handle
    assert api.call_status("cudaGetTensorDescriptor", handle, ctypes.byref(dtype), ctypes.byref(nb), dims) == api.STATUS["INTERNAL_ERROR"]
    t2 = api.TensorDescriptor((1,), "float32")
    assert t2.handle != handle


def test_convolution_descriptor_round_trip(library):
    value = (ctypes.c_float * 4)(0.5, 0, 0, 0)
    c = api.ConvolutionDescriptor(api.CROSS_CORRELATION_MODE, (-1, -2), (1, 1), (1, 1), 1, padding_value=bytes(value))
    mode, nb, groups = ctypes.c_int(-1), ctypes.c_int(-1), ctypes.c_int(-1)
    pad, stride, dil = (ctypes.c_int * 3)(), (ctypes.c_int * 3)(), (ctypes.c_int * 3)()
    pv = (ctypes.c_float * 4)()
    api.call("cudaGetConvolutionDescriptor", c.handle, ctypes.byref(mode), ctypes.byref(nb), pad, stride, dil, ctypes.byref(groups),
             ctypes.cast(pv, ctypes.c_void_p))
    assert (mode.value, nb.value, groups.value) == (api.CROSS_CORRELATION_MODE, 2, 1)
    assert list(pad)[:2] == [-1, -2] and list(stride)[:2] == [1, 1] and list(dil)[:2] == [1, 1]
    assert pv[0] == 0.5


def test_optimizer_descriptor_and_workspace(library):
    h = ctypes.c_int64(-1)
    api.call("cudaCreateOptimizerDescriptor", ctypes.byref(h))
    coef = (ctypes.c_double * 4)(0.9, 0.999, 0, 0)
    flags = (ctypes.c_bool * 4)(True, False, False, False)
    w = api.TensorDescriptor((64, 3, 3, 64), "float32")
    size = ctypes.c_int64(-1)
    api.call("cudaSetOptimizerDescriptor", h.value, 0, 0, 0.01, coef, flags)  # SGD with momentum
    api.call("cudaGetOptimizerWorkspaceSize", h.value, w.handle, ctypes.byref(size))
    assert size.value == 64 * 9 * 64 * 4
    api.call("cudaSetOptimizerDescriptor", h.value, 1, 0, 0.01, coef, flags)  # Adam
    api.call("cudaGetOptimizerWorkspaceSize", h.value, w.handle, ctypes.byref(size))
    assert size.value == 2 * 64 * 9 * 64 * 4
    api.call("cudaDestroyOptimizerDescriptor", h.value)
    assert api.call_status("cudaDestroyOptimizerDescriptor", h.value) == api.STATUS["FREE_FAILED"]


def test_invalid_devices_and_handles(library):
    n = api.number_of_devices()
    assert n >= 0
    assert library.cudaGetDefaultContext(n) == -1
    assert library.cudaGetDefaultContext(-1) == -1
    h = ctypes.c_int64(-1)
    assert api.call_status("cudaCreateContextDescriptor", ctypes.byref(h), n) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaCreateContextDescriptor", None, 0) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaCreateMemoryDescriptor", ctypes.byref(h), n, 16) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaSynchronizeWithContext", 12345) == api.STATUS["INTERNAL_ERROR"]
    ready = ctypes.c_bool(False)
    assert api.call_status("cudaIsContextReady", -1, ctypes.byref(ready)) == api.STATUS["INTERNAL_ERROR"]
    assert api.call_status("cudaDestroyMemoryDescriptor", -1) == api.STATUS["FREE_FAILED"]


def test_operator_calls_reject_bad_handles_before_any_launch(library):
    # every handle is invalid: the lookup fails on the host and nothing is enqueued
    assert api.call_status("cudaWinogradInputTransform", -1, -1, 4, -1, -1, -1, -1, -1) == api.STATUS["INTERNAL_ERROR"]
    assert api.call_status("cudaGemmBatched", -1, 0, 1, None, -1, -1, -1, -1, None, -1, -1) == api.STATUS["INTERNAL_ERROR"]
    assert api.call_status("cudaConvolutionImplicitGemmForward", -1, -1, None, -1, -1, -1, -1, -1, -1, None, -1, -1, None, -1, -1, 0) \
        == api.STATUS["INTERNAL_ERROR"]
