"""GPU parity tests of cudaGemm / cudaGemmBatched against a float64 contraction.

The reference tests cudaGemm only, on 23 x 45 x 67 with the four transpose combinations (test/test_gemm.cpp);
the same shape is used here for both entry points, plus the Winograd-shaped batched products that take the
tensor-core kernel.
"""
import ctypes

import numpy as np
import pytest

from cudabackend_b200 import api
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu


def run_gemm(ctx, entry, a, b, c0, dtype, trans_a, trans_b, alpha, beta, out_dtype=None):
    out_dtype = out_dtype or dtype
    A = api.DeviceTensor(a.shape, dtype)
    B = api.DeviceTensor(b.shape, dtype)
    C = api.DeviceTensor(c0.shape, out_dtype)
    a64 = A.upload(ctx, a)
    b64 = B.upload(ctx, b)
    c64 = C.upload(ctx, c0)
    scalar = "float64" if dtype == "float64" else "float32"
    pa, ka = api.scalar_pointer(alpha, scalar)
    pb, kb = api.scalar_pointer(beta, scalar)
    api.call(entry, ctx.handle, api.GEMM_T if trans_a else api.GEMM_N, api.GEMM_T if trans_b else api.GEMM_N, pa, A.desc.handle, A.mem.handle,
             B.desc.handle, B.mem.handle, pb, C.desc.handle, C.mem.handle)
    return C.download(ctx), a64, b64, c64


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32", "float64"])
@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_batched_reference_shape(ctx, dtype, trans_a, trans_b):
    batch, m, n, k = 5, 23, 45, 67
    r = np.random.default_rng(11)
    a = r.uniform(-1, 1, (batch, k, m) if trans_a else (batch, m, k))
    b = r.uniform(-1, 1, (batch, n, k) if trans_b else (batch, k, n))
    c0 = r.uniform(-1, 1, (batch, m, n))
    got, a64, b64, c64 = run_gemm(ctx, "cudaGemmBatched", a, b, c0, dtype, trans_a, trans_b, 1.1, 0.1)
    f = (lambda v: float(np.float32(v))) if dtype != "float64" else (lambda v: v)
    ref = o.gemm_batched(a64, b64, trans_a, trans_b, f(1.1), f(0.1), c64)
    assert o.error_metrics(got, ref)["elem"] <= {"float64": 1e-12, "float32": 1e-5, "float16": 2e-3, "bfloat16": 1.5e-2}[dtype]


@pytest.mark.parametrize("dtype", ["float16", "float32", "float64"])
def test_gemm_2d(ctx, dtype):
    m, n, k = 23, 45, 67
    r = np.random.default_rng(12)
    for trans_a in (False, True):
        for trans_b in (False, True):
            a = r.uniform(-1, 1, (k, m) if trans_a else (m, k))
            b = r.uniform(-1, 1, (n, k) if trans_b else (k, n))
            got, a64, b64, _ = run_gemm(ctx, "cudaGemm", a, b, np.zeros((m, n)), dtype, trans_a, trans_b, None, None)
            ref = o.gemm_batched(a64[None], b64[None], trans_a, trans_b)[0]
            assert o.error_metrics(got, ref)["elem"] <= {"float64": 1e-12, "float32": 1e-5, "float16": 2e-3}[dtype]


def test_gemm_int8(ctx):
    """int8 x int8 -> int32, exact (reference src/gemm.cpp:42-57)"""
    m, n, k = 24, 40, 64
    r = np.random.default_rng(13)
    a = r.integers(-127, 128, (m, k), dtype=np.int8)
    b = r.integers(-127, 128, (n, k), dtype=np.int8)
    got, _, _, _ = run_gemm(ctx, "cudaGemm", a, b, np.zeros((m, n), dtype=np.int32), "int8", False, True, None, None, out_dtype="int32")
    assert np.array_equal(got.astype(np.int64), a.astype(np.int64) @ b.astype(np.int64).T)


@pytest.mark.parametrize("shape", [(300, 64, 576), (1000, 128, 1152), (129, 72, 2304), (77, 200, 144), (4000, 256, 64), (128, 16, 16)])
def test_gemm_int8_tensor_core(ctx, shape):
    """the int8 product at the sizes of a lowered convolution (rows of im2row times filters): tcgen05 kind::i8, exact;
    row counts that are not multiples of 128, filter counts between the column blocks, several tiles per CTA"""
    m, n, k = shape
    r = np.random.default_rng(18)
    a = r.integers(-127, 128, (m, k), dtype=np.int8)
    b = r.integers(-127, 128, (n, k), dtype=np.int8)
    c0 = np.full((m, n), 7, dtype=np.int32)  # must be overwritten everywhere
    got, _, _, _ = run_gemm(ctx, "cudaGemm", a, b, c0, "int8", False, True, None, None, out_dtype="int32")
    assert np.array_equal(got.astype(np.int64), a.astype(np.int64) @ b.astype(np.int64).T)
    # beta = 1 accumulates onto C (CUDA-core kernel): same exact arithmetic
    got, _, _, _ = run_gemm(ctx, "cudaGemm", a, b, c0, "int8", False, True, None, 1.0, out_dtype="int32")
    assert np.array_equal(got.astype(np.int64), a.astype(np.int64) @ b.astype(np.int64).T + 7)


# (batch, rows of A, rows of B, contraction): Winograd-shaped products for the tensor-core kernel; the odd row
# counts exercise the clipped last tile, 200/72 the partial contraction block and the N tail.
TC_SHAPES = [(36, 128, 64, 64), (36, 392, 64, 64), (16, 1000, 128, 128), (36, 130, 32, 64), (4, 77, 72, 200), (3, 300, 256, 64), (2, 129, 320, 96)]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_gemm_batched_tensor_core(ctx, dtype, shape):
    batch, m, n, k = shape
    r = np.random.default_rng(14)
    a = r.uniform(-1, 1, (batch, m, k))
    b = r.normal(0, np.sqrt(2.0 / k), (batch, n, k))
    c0 = np.full((batch, m, n), 7.0)  # must be overwritten everywhere
    got, a64, b64, _ = run_gemm(ctx, "cudaGemmBatched", a, b, c0, dtype, False, True, None, None)
    ref = o.gemm_batched(a64, b64, False, True)
    # float32 accumulation, one rounding on store
    assert o.error_metrics(got, ref)["elem"] <= {"float16": 1e-3, "bfloat16": 8e-3}[dtype]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_gemm_batched_tensor_core_16bit_nn(ctx, dtype, shape):
    """op(B) = B (the dX contraction of a 16-bit layer): B is transposed into scratch and the tensor-core kernel runs"""
    batch, m, n, k = shape
    r = np.random.default_rng(17)
    a = r.uniform(-1, 1, (batch, m, k))
    b = r.normal(0, np.sqrt(2.0 / k), (batch, k, n))
    c0 = np.full((batch, m, n), 7.0)
    got, a64, b64, _ = run_gemm(ctx, "cudaGemmBatched", a, b, c0, dtype, False, False, 0.75, None)
    ref = o.gemm_batched(a64, b64, False, False, alpha=0.75)
    assert o.error_metrics(got, ref)["elem"] <= {"float16": 1e-3, "bfloat16": 8e-3}[dtype]


def test_gemm_batched_tensor_core_alpha_and_determinism(ctx):
    batch, m, n, k = 36, 392, 64, 64
    r = np.random.default_rng(15)
    a = r.uniform(-1, 1, (batch, m, k))
    b = r.uniform(-1, 1, (batch, n, k))
    got1, a64, b64, _ = run_gemm(ctx, "cudaGemmBatched", a, b, np.zeros((batch, m, n)), "float16", False, True, 0.5, None)
    got2, _, _, _ = run_gemm(ctx, "cudaGemmBatched", a, b, np.zeros((batch, m, n)), "float16", False, True, 0.5, None)
    ref = o.gemm_batched(a64, b64, False, True, alpha=0.5)
    assert o.error_metrics(got1, ref)["elem"] <= 1e-3
    assert np.array_equal(got1, got2)


def test_gemm_shape_mismatch(ctx):
    A = api.DeviceTensor((2, 8, 16), "float32")
    B = api.DeviceTensor((2, 8, 24), "float32")
    C = api.DeviceTensor((2, 8, 8), "float32")
    status = api.call_status("cudaGemmBatched", ctx.handle, api.GEMM_N, api.GEMM_T, None, A.desc.handle, A.mem.handle, B.desc.handle, B.mem.handle, None,
                             C.desc.handle, C.mem.handle)
    assert status == api.STATUS["BAD_PARAM"]


@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("trans_b", [True, False])
def test_gemm_batched_tensor_core_float32(ctx, shape, trans_b):
    """float32 on the tensor cores: three TF32 passes over a hi/lo split must stay at float32-level accuracy"""
    batch, m, n, k = shape
    r = np.random.default_rng(16)
    a = r.uniform(-1, 1, (batch, m, k))
    b = r.normal(0, np.sqrt(2.0 / k), (batch, n, k) if trans_b else (batch, k, n))
    c0 = np.full((batch, m, n), 7.0)
    got, a64, b64, _ = run_gemm(ctx, "cudaGemmBatched", a, b, c0, "float32", False, trans_b, 1.25, None)
    ref = o.gemm_batched(a64, b64, False, trans_b, alpha=1.25)
    assert o.error_metrics(got, ref)["elem"] <= 2e-5


# (batch, contraction length, rows of the result, columns of the result)
TN_SHAPES = [(36, 392, 64, 64), (36, 6272, 64, 64), (4, 1000, 72, 200), (3, 77, 20, 36), (2, 33, 128, 64), (1, 4096, 256, 136),
             (4, 100, 20, 36), (2, 33, 64, 40), (6, 900, 33, 64)]  # the last three: two batch entries per MMA, ragged blocks


@pytest.mark.parametrize("shape", TN_SHAPES)
@pytest.mark.parametrize("beta", [None, 0.5])
def test_gemm_batched_weight_gradient_contraction_float32(ctx, shape, beta):
    """C = A^T * B with both operands stored contraction-index-outermost: the dW product of the Winograd backward pass"""
    batch, kc, m, n = shape
    r = np.random.default_rng(17)
    a = r.uniform(-1, 1, (batch, kc, m))
    b = r.uniform(-1, 1, (batch, kc, n))
    c0 = r.uniform(-1, 1, (batch, m, n))
    got, a64, b64, c64 = run_gemm(ctx, "cudaGemmBatched", a, b, c0, "float32", True, False, 0.75, beta)
    ref = o.gemm_batched(a64, b64, True, False, alpha=0.75, beta=beta or 0.0, c=c64)
    assert o.error_metrics(got, ref)["elem"] <= 2e-5
    again, _, _, _ = run_gemm(ctx, "cudaGemmBatched", a, b, c0, "float32", True, False, 0.75, beta)
    assert np.array_equal(got, again)  # fixed-order split reduction: bitwise reproducible
