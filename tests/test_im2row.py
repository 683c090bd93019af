"""cudaIm2Row (explicit lowering of a convolution) against the numpy restatement of the reference's kernel, and the
lowering route end to end: im2row followed by cudaGemm with op(B) = T is the convolution."""
import ctypes

import numpy as np
import pytest

from cudabackend_b200 import api
from oracle import oracle as o
from tests import common


def test_oracle_im2row_times_filters_is_the_convolution():
    """CPU: the restated lowering reproduces the float64 direct convolution, for both kernel orders"""
    r = np.random.default_rng(5)
    x = r.uniform(-1, 1, (2, 6, 7, 5))
    w = r.uniform(-1, 1, (4, 3, 3, 5))
    for rotate in (False, True):
        rows = o.im2row(x, (3, 3), (-1, -1), rotate=rotate)
        got = (rows @ w.reshape(4, -1).T).reshape(2, 6, 7, 4)
        ref = o.conv2d_forward(x, w, mode=1 if rotate else 0)
        assert np.max(np.abs(got - ref)) < 1e-12
    rows = o.im2row(x, (3, 3), (0, 0))                      # no padding: 4 x 5 outputs
    got = (rows @ w.reshape(4, -1).T).reshape(2, 4, 5, 4)
    # the direct-convolution oracle keeps the output as large as the input; its top-left 4 x 5 block is the unpadded result
    assert np.max(np.abs(got - o.conv2d_forward(x, w, padding=(0, 0))[:, :4, :5, :])) < 1e-12


def lower(ctx, x, kernel, padding, mode, dtype, padding_value=None):
    n, h, w, c = x.shape
    kh, kw = kernel
    ho, wo = h - 2 * padding[0] - (kh - 1), w - 2 * padding[1] - (kw - 1)
    src = api.DeviceTensor(x.shape, dtype)
    src.mem.from_host(ctx, x)
    filt = api.TensorDescriptor((1, kh, kw, c), dtype)
    rows = api.DeviceTensor((n * ho * wo, kh * kw * c), dtype)
    conv = api.ConvolutionDescriptor(mode, padding, padding_value=padding_value)
    api.call("cudaIm2Row", ctx.handle, conv.handle, filt.handle, src.desc.handle, src.mem.handle, rows.desc.handle, rows.mem.handle)
    return rows


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,np_dtype", [("int8", np.int8), ("float16", np.float16), ("float32", np.float32), ("float64", np.float64)])
@pytest.mark.parametrize("shape,kernel,padding", [((3, 9, 10, 24), (3, 3), (-1, -1)), ((2, 7, 5, 13), (3, 3), (-1, -1)), ((2, 8, 8, 16), (5, 5), (-2, -2)),
                                                   ((2, 6, 7, 8), (3, 3), (0, 0)), ((1, 5, 5, 3), (1, 1), (0, 0))])
def test_im2row_matches_the_restated_reference(ctx, dtype, np_dtype, shape, kernel, padding):
    r = np.random.default_rng(21)
    x = (r.integers(-100, 100, shape) if dtype == "int8" else r.uniform(-1, 1, shape)).astype(np_dtype)
    for mode, rotate in ((api.CONVOLUTION_MODE, False), (api.CROSS_CORRELATION_MODE, True)):
        rows = lower(ctx, x, kernel, padding, mode, dtype)
        got = rows.download_raw(ctx)
        assert np.array_equal(got, o.im2row(x, kernel, padding, rotate=rotate)), (mode, shape)


@pytest.mark.gpu
def test_im2row_padding_value(ctx):
    x = np.random.default_rng(22).uniform(-1, 1, (2, 5, 6, 8)).astype(np.float32)
    rows = lower(ctx, x, (3, 3), (-1, -1), api.CONVOLUTION_MODE, "float32", padding_value=np.float32(-7.5).tobytes())
    assert np.array_equal(rows.download_raw(ctx), o.im2row(x, (3, 3), (-1, -1), padding_value=np.float32(-7.5)))


@pytest.mark.gpu
def test_im2row_rejects_a_row_tensor_of_the_wrong_size(ctx):
    src = api.DeviceTensor((1, 4, 4, 8), "float32")
    filt = api.TensorDescriptor((1, 3, 3, 8), "float32")
    rows = api.DeviceTensor((16, 8 * 8), "float32")
    conv = api.ConvolutionDescriptor(api.CONVOLUTION_MODE, (-1, -1))
    with pytest.raises(api.AvocadoError) as failure:
        api.call("cudaIm2Row", ctx.handle, conv.handle, filt.handle, src.desc.handle, src.mem.handle, rows.desc.handle, rows.mem.handle)
    assert failure.value.status == api.STATUS["BAD_PARAM"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float16", "float32"])
def test_lowering_route_is_the_convolution(ctx, dtype):
    """cudaIm2Row + cudaGemm(N, T) against the float64 direct convolution (the route of the reference's test_implicit_gemm)"""
    n, h, w, c, k = 4, 14, 14, 64, 72
    x64 = api.to_storage(common.uniform("x", (n, h, w, c)), dtype)
    wt64 = api.to_storage(common.he_normal_weights(k, 3, c), dtype)
    rows = lower(ctx, x64[0], (3, 3), (-1, -1), api.CONVOLUTION_MODE, dtype)
    wmat = api.DeviceTensor((k, 9 * c), dtype)
    wmat.mem.from_host(ctx, wt64[0].reshape(k, 9 * c))
    y = api.DeviceTensor((n * h * w, k), dtype)
    api.call("cudaGemm", ctx.handle, api.GEMM_N, api.GEMM_T, None, rows.desc.handle, rows.mem.handle, wmat.desc.handle, wmat.mem.handle, None,
             y.desc.handle, y.mem.handle)
    got = y.download(ctx).reshape(n, h, w, k)
    ref = o.conv2d_forward(x64[1], wt64[1])
    assert o.error_metrics(got, ref)["elem"] <= {"float16": 1.5e-3, "float32": 2e-5}[dtype]
