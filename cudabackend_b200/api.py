"""ctypes binding of libAvocadoCudaBackend.so -- the call a user of the library makes.

Function names, argument order and meaning are those of include/Avocado/cuda_backend.h (which mirrors the
reference's include/Avocado/cuda_backend.h); this module only adds the handle bookkeeping that a C caller would
write by hand.  There is no fallback of any kind: if the shared library is missing or a call fails, an exception
is raised.
"""
import ctypes
import os

import numpy as np

# enum values of include/Avocado/backend_defs.h
STATUS_NAMES = ["SUCCESS", "ALLOC_FAILED", "BAD_ALLOC", "FREE_FAILED", "BAD_PARAM", "ARCH_MISMATCH", "INTERNAL_ERROR", "NOT_SUPPORTED",
                "UNSUPPORTED_DATATYPE", "EXECUTION_FAILED", "INSUFFICIENT_DRIVER", "DEVICE_TYPE_MISMATCH"]
STATUS = {name: i for i, name in enumerate(STATUS_NAMES)}
DTYPES = {"unknown": 0, "uint8": 1, "int8": 2, "int16": 3, "int32": 4, "int64": 5, "float16": 6, "bfloat16": 7, "float32": 8, "float64": 9,
          "complex32": 10, "complex64": 11}
DTYPE_SIZES = {"uint8": 1, "int8": 1, "int16": 2, "int32": 4, "int64": 8, "float16": 2, "bfloat16": 2, "float32": 4, "float64": 8}
ACTIVATIONS = {"linear": 0, "sigmoid": 1, "tanh": 2, "relu": 3, "selu": 4, "elu": 5, "exponential": 6, "softplus": 7, "softsign": 8}
CONVOLUTION_MODE, CROSS_CORRELATION_MODE = 0, 1
GEMM_N, GEMM_T = 0, 1
INVALID = -1
NO_ALLOC_SCRATCH_BYTES = 8 * 1024 * 1024  # AVOCADO_NO_ALLOC_SCRATCH_BYTES
FUSE_WEIGHTS, FUSE_OUTPUT = 1, 2  # AVOCADO_WINOGRAD_FUSE_*

_H = ctypes.c_int64  # every descriptor handle
_I64 = ctypes.c_int64
_INT = ctypes.c_int
_VP = ctypes.c_void_p
_conv_args = [_H, _H, _VP, _H, _H, _H, _H, _H, _H, _VP, _H, _H, _VP, _H, _H, _INT]

SIGNATURES = {
    "cudaGetNumberOfDevices": (_INT, []),
    "cudaGetDeviceProperty": (_INT, [_INT, _INT, _VP]),
    "cudaIsCopyPossible": (_INT, [_INT, _INT, ctypes.POINTER(ctypes.c_bool)]),
    "cudaCreateContextDescriptor": (_INT, [ctypes.POINTER(_H), _INT]),
    "cudaDestroyContextDescriptor": (_INT, [_H]),
    "cudaGetDefaultContext": (_H, [_INT]),
    "cudaSynchronizeWithContext": (_INT, [_H]),
    "cudaIsContextReady": (_INT, [_H, ctypes.POINTER(ctypes.c_bool)]),
    "cudaCreateMemoryDescriptor": (_INT, [ctypes.POINTER(_H), _INT, _I64]),
    "cudaCreateMemoryView": (_INT, [ctypes.POINTER(_H), _H, _I64, _I64]),
    "cudaDestroyMemoryDescriptor": (_INT, [_H]),
    "cudaSetMemory": (_INT, [_H, _H, _I64, _I64, _VP, _I64]),
    "cudaCopyMemory": (_INT, [_H, _H, _I64, _H, _I64, _I64]),
    "cudaCopyMemoryToHost": (_INT, [_H, _VP, _H, _I64, _I64]),
    "cudaCopyMemoryFromHost": (_INT, [_H, _H, _I64, _VP, _I64]),
    "cudaPageLock": (_INT, [_VP, _I64]),
    "cudaPageUnlock": (_INT, [_VP]),
    "cudaCreateTensorDescriptor": (_INT, [ctypes.POINTER(_H)]),
    "cudaDestroyTensorDescriptor": (_INT, [_H]),
    "cudaSetTensorDescriptor": (_INT, [_H, _INT, _INT, ctypes.POINTER(_INT)]),
    "cudaGetTensorDescriptor": (_INT, [_H, ctypes.POINTER(_INT), ctypes.POINTER(_INT), ctypes.POINTER(_INT)]),
    "cudaCreateConvolutionDescriptor": (_INT, [ctypes.POINTER(_H)]),
    "cudaDestroyConvolutionDescriptor": (_INT, [_H]),
    "cudaSetConvolutionDescriptor": (_INT, [_H, _INT, _INT, ctypes.POINTER(_INT), ctypes.POINTER(_INT), ctypes.POINTER(_INT), _INT, _VP]),
    "cudaGetConvolutionDescriptor": (_INT, [_H, ctypes.POINTER(_INT), ctypes.POINTER(_INT), ctypes.POINTER(_INT), ctypes.POINTER(_INT),
                                             ctypes.POINTER(_INT), ctypes.POINTER(_INT), _VP]),
    "cudaCreateOptimizerDescriptor": (_INT, [ctypes.POINTER(_H)]),
    "cudaDestroyOptimizerDescriptor": (_INT, [_H]),
    "cudaSetOptimizerDescriptor": (_INT, [_H, _INT, _I64, ctypes.c_double, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_bool)]),
    "cudaGetOptimizerDescriptor": (_INT, [_H, ctypes.POINTER(_INT), ctypes.POINTER(_I64), ctypes.POINTER(ctypes.c_double),
                                           ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_bool)]),
    "cudaGetOptimizerWorkspaceSize": (_INT, [_H, _H, ctypes.POINTER(_I64)]),
    "cudaWinogradWeightTransform": (_INT, [_H, _H, _INT, _H, _H, _H, _H]),
    "cudaWinogradInputTransform": (_INT, [_H, _H, _INT, _H, _H, _H, _H, _H]),
    "cudaWinogradOutputTransform": (_INT, [_H, _H, _INT, _H, _VP, _H, _H, _H, _H, _H, _H, _VP, _H, _H, _VP, _INT]),
    "cudaWinogradGradientTransform": (_INT, [_H, _H, _INT, _H, _H, _H, _H, _H]),
    "cudaWinogradUpdateTransform": (_INT, [_H, _H, _INT, _VP, _H, _H, _VP, _H, _H]),
    "cudaGemmBatched": (_INT, [_H, _INT, _INT, _VP, _H, _H, _H, _H, _VP, _H, _H]),
    "cudaGemm": (_INT, [_H, _INT, _INT, _VP, _H, _H, _H, _H, _VP, _H, _H]),
    "cudaConvolutionWinogradFusedForward": (_INT, _conv_args),
    "cudaConvolutionImplicitGemmForward": (_INT, _conv_args),
    # additive entry points of include/Avocado/cuda_backend_ext.h
    "cudaSetConvolutionQuantization": (_INT, [_H, _H]),
    "cudaGetMemoryPointer": (_INT, [_H, ctypes.POINTER(_VP)]),
    "cudaGetContextStream": (_INT, [_H, ctypes.POINTER(_VP)]),
    "cudaGetLastDeviceStatus": (_INT, [_H, ctypes.POINTER(_INT)]),
    "cudaContextBeginCapture": (_INT, [_H]),
    "cudaContextEndCapture": (_INT, [_H, ctypes.POINTER(_I64)]),
    "cudaContextLaunchGraph": (_INT, [_H, _I64]),
    "cudaDestroyCapturedGraph": (_INT, [_I64]),
    "cudaConvolutionWinogradFusedForwardNoAlloc": (_INT, _conv_args),
    "cudaRunBoundedWaitSelfTest": (_INT, [_H, _INT]),
    "cudaRunBoundedWaitSelfTestNoAlloc": (_INT, [_H, _INT]),
    "cudaContextWaitForContext": (_INT, [_H, _H]),
    "cudaContextSetWinogradFusion": (_INT, [_H, _INT]),
    "cudaIm2Row": (_INT, [_H, _H, _H, _H, _H, _H, _H]),
    "cudaOptimizerLearn": (_INT, [_H, _H, _VP, _H, _H, _VP, _H, _H, _H]),
    "cudaAddBias": (_INT, [_H, _VP, _VP, _H, _H, _H, _H, _H, _H, _VP, _VP, _VP, _H, _INT]),
    "cudaActivationForward": (_INT, [_H, _INT, _VP, _H, _H, _VP, _H, _H]),
}

# exported for link compatibility, return NOT_SUPPORTED
UNSUPPORTED_SYMBOLS = ["cudaChangeType", "cudaConcatTensors", "cudaSplitTensors", "cudaTranspose", "cudaScaleTensor", "cudaAddScalarToTensor",
                       "cudaAddTensors", "cudaBinaryOp", "cudaUnaryOp", "cudaReduceTensor",
                       "cudaActivationBackward", "cudaSoftmaxForward", "cudaSoftmaxBackward", "cudaAffineForward", "cudaBatchNormInference",
                       "cudaBatchNormForward", "cudaBatchNormBackward", "cudaDropoutForward", "cudaDropoutBackward", "cudaPoolingForward",
                       "cudaPoolingBackward", "cudaMetricFunction", "cudaLossFunction", "cudaLossGradient",
                       "cudaRegularizerL2"]


class AvocadoError(RuntimeError):
    def __init__(self, function, status):
        self.function = function
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__("%s returned AVOCADO_STATUS_%s" % (function, name))


def library_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libAvocadoCudaBackend.so")


_lib = None


def load():
    """Loads the C-ABI library and attaches the signatures.  Raises if the library has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError("%s is missing: build it with `python -m cudabackend_b200.build` (there is no fallback path)" % path)
        handle = ctypes.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(function, status):
    if status != 0:
        raise AvocadoError(function, status)


def call(name, *args):
    """Calls an entry point that returns avStatus_t and raises AvocadoError unless it succeeded."""
    check(name, getattr(load(), name)(*args))


def call_status(name, *args):
    """Calls an entry point and returns its avStatus_t unchanged (for tests of the error behaviour)."""
    return getattr(load(), name)(*args)


def number_of_devices():
    return int(load().cudaGetNumberOfDevices())


class Context:
    """avContextDescriptor_t with its own stream; `Context.default(device)` gives the default context."""

    def __init__(self, device=0, handle=None):
        self.device = device
        self._owned = handle is None
        if handle is None:
            h = _H(INVALID)
            call("cudaCreateContextDescriptor", ctypes.byref(h), device)
            handle = h.value
        self.handle = handle

    @classmethod
    def default(cls, device=0):
        return cls(device, handle=load().cudaGetDefaultContext(device))

    def synchronize(self):
        call("cudaSynchronizeWithContext", self.handle)

    def is_ready(self):
        r = ctypes.c_bool(False)
        call("cudaIsContextReady", self.handle, ctypes.byref(r))
        return bool(r.value)

    def stream(self):
        p = _VP()
        call("cudaGetContextStream", self.handle, ctypes.byref(p))
        return p.value or 0

    def last_device_status(self):
        r = _INT(0)
        call("cudaGetLastDeviceStatus", self.handle, ctypes.byref(r))
        return int(r.value)

    def set_winograd_fusion(self, flags):
        """flags: 0, FUSE_WEIGHTS (the weight transform rides in the input transform's launch), FUSE_OUTPUT (cudaGemmBatched +
        cudaWinogradOutputTransform of an F(4x4,3x3) pipeline run as one kernel; the products M are then not written), or both.
        True means both."""
        if flags is True:
            flags = FUSE_WEIGHTS | FUSE_OUTPUT
        call("cudaContextSetWinogradFusion", self.handle, int(flags))

    def wait_for(self, other):
        """Work enqueued on this context from now on runs after the work already enqueued on `other` (no host blocking)."""
        call("cudaContextWaitForContext", self.handle, other.handle)

    def capture(self, fn):
        """Runs fn() once for its side effects on the stream, then records a second run of it into a graph."""
        fn()
        self.synchronize()
        call("cudaContextBeginCapture", self.handle)
        try:
            fn()
        finally:
            g = _I64(0)
            status = call_status("cudaContextEndCapture", self.handle, ctypes.byref(g))
        check("cudaContextEndCapture", status)
        return Graph(self, g.value)

    def destroy(self):
        if self._owned and self.handle != INVALID:
            call("cudaDestroyContextDescriptor", self.handle)
        self.handle = INVALID

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Graph:
    """A recorded sequence of API calls on one context (cudaContextBeginCapture / EndCapture), replayed by launch()."""

    def __init__(self, ctx, handle):
        self.ctx = ctx
        self.handle = handle
        self._launch = load().cudaContextLaunchGraph

    def launch(self):
        status = self._launch(self.ctx.handle, self.handle)
        if status != 0:
            raise AvocadoError("cudaContextLaunchGraph", status)

    def destroy(self):
        if self.handle:
            call("cudaDestroyCapturedGraph", self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class Memory:
    """avMemoryDescriptor_t: an owning device allocation (or a view of one)."""

    def __init__(self, size, device=0, handle=None, owned=True):
        self.size = int(size)
        self.device = device
        self._owned = owned
        if handle is None:
            h = _H(INVALID)
            call("cudaCreateMemoryDescriptor", ctypes.byref(h), device, self.size)
            handle = h.value
        self.handle = handle

    def view(self, size, offset):
        h = _H(INVALID)
        call("cudaCreateMemoryView", ctypes.byref(h), self.handle, int(size), int(offset))
        return Memory(size, self.device, handle=h.value)

    def pointer(self):
        p = _VP()
        call("cudaGetMemoryPointer", self.handle, ctypes.byref(p))
        return p.value or 0

    def from_host(self, ctx, array, offset=0):
        array = np.ascontiguousarray(array)
        call("cudaCopyMemoryFromHost", ctx.handle, self.handle, int(offset), array.ctypes.data_as(_VP), array.nbytes)

    def to_host(self, ctx, array, offset=0):
        assert array.flags["C_CONTIGUOUS"]
        call("cudaCopyMemoryToHost", ctx.handle, array.ctypes.data_as(_VP), self.handle, int(offset), array.nbytes)
        return array

    def zero(self, ctx):
        call("cudaSetMemory", ctx.handle, self.handle, 0, self.size, None, 0)

    def destroy(self):
        if self.handle != INVALID:
            call("cudaDestroyMemoryDescriptor", self.handle)
        self.handle = INVALID

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class TensorDescriptor:
    def __init__(self, shape, dtype):
        h = _H(INVALID)
        call("cudaCreateTensorDescriptor", ctypes.byref(h))
        self.handle = h.value
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        dims = (_INT * len(self.shape))(*self.shape)
        call("cudaSetTensorDescriptor", self.handle, DTYPES[dtype], len(self.shape), dims)

    @property
    def nbytes(self):
        n = DTYPE_SIZES[self.dtype]
        for s in self.shape:
            n *= s
        return n

    def destroy(self):
        if self.handle != INVALID:
            call("cudaDestroyTensorDescriptor", self.handle)
        self.handle = INVALID

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class ConvolutionDescriptor:
    def __init__(self, mode=CONVOLUTION_MODE, padding=(-1, -1), strides=(1, 1), dilation=(1, 1), groups=1, padding_value=None):
        h = _H(INVALID)
        call("cudaCreateConvolutionDescriptor", ctypes.byref(h))
        self.handle = h.value
        n = len(padding)
        pv = None
        if padding_value is not None:
            raw = bytes(padding_value)
            pv = ctypes.create_string_buffer(raw + b"\0" * (16 - len(raw)), 16)
        call("cudaSetConvolutionDescriptor", self.handle, mode, n, (_INT * n)(*padding), (_INT * n)(*strides), (_INT * n)(*dilation), groups,
             ctypes.cast(pv, _VP) if pv is not None else None)

    def set_quantization(self, scales_memory):
        call("cudaSetConvolutionQuantization", self.handle, scales_memory.handle if scales_memory is not None else INVALID)

    def destroy(self):
        if self.handle != INVALID:
            call("cudaDestroyConvolutionDescriptor", self.handle)
        self.handle = INVALID

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


# ---- numpy <-> storage dtype helpers (host-side data preparation only) -------------------------------------

def float_to_bfloat16_bits(a):
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bfloat16_bits_to_float(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_storage(a, dtype):
    """Rounds a float array to the storage dtype; returns (array to upload, the same values as float64)."""
    if dtype == "float16":
        s = np.ascontiguousarray(a, dtype=np.float32).astype(np.float16)
        return s, s.astype(np.float64)
    if dtype == "bfloat16":
        s = float_to_bfloat16_bits(a)
        return s, bfloat16_bits_to_float(s).astype(np.float64)
    if dtype == "float32":
        s = np.ascontiguousarray(a, dtype=np.float32)
        return s, s.astype(np.float64)
    if dtype == "float64":
        s = np.ascontiguousarray(a, dtype=np.float64)
        return s, s
    if dtype in ("int8", "int32"):
        s = np.ascontiguousarray(a, dtype=getattr(np, dtype))
        return s, s.astype(np.float64)
    raise ValueError(dtype)


def host_buffer(shape, dtype):
    np_dtype = {"float16": np.float16, "bfloat16": np.uint16, "float32": np.float32, "float64": np.float64, "int8": np.int8,
                "int32": np.int32}[dtype]
    return np.empty(shape, dtype=np_dtype)


def from_storage(a, dtype):
    if dtype == "bfloat16":
        return bfloat16_bits_to_float(a).astype(np.float64)
    return np.asarray(a).astype(np.float64)


class DeviceTensor:
    """A tensor descriptor together with the device memory it describes."""

    def __init__(self, shape, dtype, device=0):
        self.desc = TensorDescriptor(shape, dtype)
        self.mem = Memory(max(self.desc.nbytes, 1), device)
        self.shape = self.desc.shape
        self.dtype = dtype

    def upload(self, ctx, values):
        """Rounds `values` to the storage dtype, copies them to the device and returns them as float64."""
        stored, as_f64 = to_storage(np.asarray(values).reshape(self.shape), self.dtype)
        self.mem.from_host(ctx, stored)
        return as_f64

    def download(self, ctx):
        buf = host_buffer(self.shape, self.dtype)
        self.mem.to_host(ctx, buf)
        ctx.synchronize()
        return from_storage(buf, self.dtype)

    def download_raw(self, ctx):
        buf = host_buffer(self.shape, self.dtype)
        self.mem.to_host(ctx, buf)
        ctx.synchronize()
        return buf


def scalar_pointer(value, dtype):
    """Host scalar in the type the C API expects: double for float64 tensors, float otherwise; None stays null."""
    if value is None:
        return None, None
    holder = ctypes.c_double(value) if dtype == "float64" else ctypes.c_float(value)
    return ctypes.cast(ctypes.byref(holder), _VP), holder
