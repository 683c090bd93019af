"""GPU parity tests of the five Winograd transforms against the float64 oracle.

Shapes and scalars are those of the reference's own tests (test/test_winograd.cpp:28-240): x = {12,13,14,135},
w = {21,3,3,135} or {21,5,5,135}, transform sizes 2 and 4, alpha1 = 1.1, alpha2 = 1.2, beta = 0.1 and the four
(bias, z) combinations; gradient and update transforms for float32 / float64 only.  Each transform's only error
is arithmetic in float (double) plus one rounding to the storage type, so the bound is a few storage epsilons of
the largest output magnitude.
"""
import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu

CONFIGS = [(2, 3), (4, 3), (2, 5)]
DTYPES = ["float16", "bfloat16", "float32", "float64"]


def bound(values, dtype, factor=4.0):
    return factor * common.EPS[dtype] * max(float(np.abs(values).max()), 1e-30) + (1e-6 if dtype == "float32" else 0.0)


def make(ctx, ts, ks, dtype, mdtype=None, shape=(12, 13, 14, 135), k=21, training=False):
    n, h, w, c = shape
    return pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, mdtype, ts, ks, training=training)


@pytest.mark.parametrize("ts,ks", CONFIGS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rotated", [False, True])
def test_weight_transform(ctx, ts, ks, dtype, rotated):
    p = make(ctx, ts, ks, dtype)
    w = p.wt.upload(ctx, common.he_normal_weights(p.k, ks, p.c))
    p.weight_transform(rotated=rotated)
    got = p.u.download(ctx)
    ref = o.winograd_weight_transform(w, ts, invert=rotated)
    assert np.abs(got - ref).max() <= bound(ref, dtype)


@pytest.mark.parametrize("ts,ks", CONFIGS)
@pytest.mark.parametrize("dtype", DTYPES)
def test_input_transform(ctx, ts, ks, dtype):
    p = make(ctx, ts, ks, dtype)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    p.input_transform()
    got = p.v.download(ctx)
    ref = o.winograd_input_transform(x, ts, ks, padding=p.padding)
    assert np.abs(got - ref).max() <= bound(ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "float16"])
def test_input_transform_padding_value_and_offset(ctx, dtype):
    """non-zero padding value and a padding offset that is not -(ks/2) (reference :336-343)"""
    n, h, w, c, k = 2, 9, 11, 6, 4
    np_dtype = {"float32": np.float32, "float16": np.float16}[dtype]
    value = np_dtype(0.75)
    conv = api.ConvolutionDescriptor(api.CONVOLUTION_MODE, (-2, 0), padding_value=value.tobytes())
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, None, 4, 3)
    p.conv = conv
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    p.input_transform()
    got = p.v.download(ctx)
    ref = o.winograd_input_transform(x, 4, 3, padding=(-2, 0), padding_value=0.75)
    assert np.abs(got - ref).max() <= bound(ref, dtype)


@pytest.mark.parametrize("ts,ks", CONFIGS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("use_bias,use_z", [(True, True), (True, False), (False, True), (False, False)])
def test_output_transform(ctx, ts, ks, dtype, use_bias, use_z):
    p = make(ctx, ts, ks, dtype)
    m = p.m.upload(ctx, common.uniform("x", p.m.shape, extra=1))
    y0 = p.y.upload(ctx, common.uniform("y", p.y.shape))
    bias = p.set_bias(common.uniform("b", (p.k,))) if use_bias else None
    z = p.set_z(common.uniform("z", p.y.shape)) if use_z else None
    p.output_transform(alpha1=1.1, alpha2=1.2, beta=0.1, activation="linear")
    got = p.y.download(ctx)
    f32 = lambda v: float(np.float32(v)) if dtype != "float64" else v
    ref = o.winograd_output_transform(m, p.y.shape, ts, ks, bias=bias, z=z, y=y0, alpha1=f32(1.1), alpha2=f32(1.2), beta=f32(0.1))
    assert np.abs(got - ref).max() <= bound(ref, dtype)


@pytest.mark.parametrize("activation", ["sigmoid", "tanh", "relu", "selu", "elu", "exponential", "softplus", "softsign"])
def test_output_transform_activations(ctx, activation):
    p = make(ctx, 4, 3, "float32", shape=(2, 9, 10, 16), k=8)
    m = p.m.upload(ctx, common.uniform("x", p.m.shape, extra=2))
    bias = p.set_bias(common.uniform("b", (p.k,)))
    p.output_transform(activation=activation)
    got = p.y.download(ctx)
    ref = o.winograd_output_transform(m, p.y.shape, 4, 3, bias=bias, activation=activation)
    assert np.abs(got - ref).max() <= 1e-5 * max(1.0, float(np.abs(ref).max()))


@pytest.mark.parametrize("ts,ks", CONFIGS)
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_gradient_and_update_transform(ctx, ts, ks, dtype):
    p = make(ctx, ts, ks, dtype, training=True)
    dy = p.dy.upload(ctx, common.uniform("dy", p.dy.shape))
    p.gradient_transform()
    got = p.g.download(ctx)
    ref = o.winograd_gradient_transform(dy, ts, ks)
    assert np.abs(got - ref).max() <= bound(ref, dtype)

    mw = p.mw.upload(ctx, common.uniform("x", p.mw.shape, extra=3))
    dw0 = p.dw.upload(ctx, common.uniform("w", p.dw.shape, extra=3))
    p.update_transform(alpha=1.1, beta=0.1)
    got = p.dw.download(ctx)
    f32 = lambda v: float(np.float32(v)) if dtype != "float64" else v
    ref = o.winograd_update_transform(mw, ts, ks, dw=dw0, alpha=f32(1.1), beta=f32(0.1))
    assert np.abs(got - ref).max() <= bound(ref, dtype)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_gradient_transform_rejects_16_bit(ctx, dtype):
    """the reference dispatches gradient/update for float32 and float64 only (:971-979, :991-999)"""
    p = make(ctx, 4, 3, dtype, shape=(1, 8, 8, 8), k=8, training=True)
    status = api.call_status("cudaWinogradGradientTransform", ctx.handle, p.conv.handle, 4, p.wt.desc.handle, p.dy.desc.handle, p.dy.mem.handle,
                             p.g.desc.handle, p.g.mem.handle)
    assert status == api.STATUS["UNSUPPORTED_DATATYPE"]


def test_unsupported_tile_configuration(ctx):
    p = make(ctx, 4, 3, "float32", shape=(1, 8, 8, 8), k=8)
    status = api.call_status("cudaWinogradWeightTransform", ctx.handle, p.conv.handle, 3, p.wt.desc.handle, p.wt.mem.handle, p.u.desc.handle,
                             p.u.mem.handle)
    assert status == api.STATUS["NOT_SUPPORTED"]
    wrong = api.DeviceTensor((36, 7, 8), "float32")
    status = api.call_status("cudaWinogradWeightTransform", ctx.handle, p.conv.handle, 4, p.wt.desc.handle, p.wt.mem.handle, wrong.desc.handle,
                             wrong.mem.handle)
    assert status == api.STATUS["BAD_PARAM"]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_mixed_precision_matrices(ctx, dtype):
    """16-bit activations with float32 transform-domain tensors"""
    p = make(ctx, 4, 3, dtype, "float32", shape=(2, 10, 9, 24), k=16)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    w = p.wt.upload(ctx, common.he_normal_weights(p.k, 3, p.c))
    p.weight_transform()
    p.input_transform()
    assert np.abs(p.u.download(ctx) - o.winograd_weight_transform(w, 4)).max() <= bound(w, "float32", 16)
    assert np.abs(p.v.download(ctx) - o.winograd_input_transform(x, 4, 3)).max() <= bound(x, "float32", 64)


def test_empty_batch(ctx):
    p = make(ctx, 4, 3, "float32", shape=(0, 8, 8, 8), k=8)
    p.input_transform()
    p.output_transform()
    ctx.synchronize()
