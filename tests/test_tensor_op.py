"""cudaAddBias and cudaActivationForward (the element-wise steps right behind an unfused convolution) against the float64
restatement of the reference's formulas."""
import numpy as np
import pytest

from cudabackend_b200 import api
from oracle import oracle as o
from tests import common

TOL = {"float16": 1.5e-3, "bfloat16": 1e-2, "float32": 2e-6, "float64": 1e-13}


def test_oracle_activation_matches_the_c_oracle():
    """CPU: the numpy activations equal the ones inside the C convolution oracle (a 1x1 identity convolution applies them)"""
    x = np.random.default_rng(41).uniform(-3, 3, (1, 4, 5, 6))
    w = np.eye(6).reshape(6, 1, 1, 6)
    for name in api.ACTIVATIONS:
        ref = o.conv2d_forward(x, w, padding=(0, 0), activation=name)
        assert np.max(np.abs(o.activation(x, name) - ref)) < 1e-14, name


def f(v, dtype):
    return v if dtype == "float64" else float(np.float32(v))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32", "float64"])
@pytest.mark.parametrize("shape", [(4, 14, 14, 64), (3, 5, 7, 21)])
@pytest.mark.parametrize("activation,use_z,beta3", [("relu", False, None), ("linear", True, 0.25), ("tanh", True, None), ("sigmoid", False, 0.5)])
def test_add_bias(ctx, dtype, shape, activation, use_z, beta3):
    x = api.DeviceTensor(shape, dtype)
    y = api.DeviceTensor(shape, dtype)
    z = api.DeviceTensor(shape, dtype)
    b = api.DeviceTensor(shape[-1:], "float64" if dtype == "float64" else "float32")
    x64 = x.upload(ctx, common.uniform("x", shape))
    y64 = y.upload(ctx, common.uniform("y", shape))
    z64 = z.upload(ctx, common.uniform("z", shape))
    b64 = b.upload(ctx, common.uniform("b", shape[-1:], -0.5, 0.5))
    scalars = {"alpha1": 1.1, "alpha2": 0.9, "beta1": 0.7 if use_z else None, "beta2": 0.3 if use_z else None, "beta3": beta3}
    ptrs = {k: api.scalar_pointer(v, dtype) for k, v in scalars.items()}
    api.call("cudaAddBias", ctx.handle, ptrs["alpha1"][0], ptrs["alpha2"][0], x.desc.handle, x.mem.handle, b.desc.handle, b.mem.handle, y.desc.handle,
             y.mem.handle, ptrs["beta1"][0], ptrs["beta2"][0], ptrs["beta3"][0], z.mem.handle if use_z else api.INVALID, api.ACTIVATIONS[activation])
    ref = o.add_bias(x64, b64, z64 if use_z else None, y64, f(1.1, dtype), f(0.9, dtype), f(0.7, dtype) if use_z else 0.0, f(0.3, dtype) if use_z else 0.0,
                     f(beta3, dtype) if beta3 else 0.0, activation)
    assert o.error_metrics(y.download(ctx), ref)["elem"] <= TOL[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32", "float64"])
@pytest.mark.parametrize("activation", list(api.ACTIVATIONS))
def test_activation_forward(ctx, dtype, activation):
    shape = (3, 9, 10, 24) if activation in ("relu", "linear") else (2, 5, 7, 9)
    x = api.DeviceTensor(shape, dtype)
    y = api.DeviceTensor(shape, dtype)
    x64 = x.upload(ctx, common.uniform("x", shape, -2, 2))
    y64 = y.upload(ctx, common.uniform("y", shape))
    a, ka = api.scalar_pointer(1.25, dtype)
    b, kb = api.scalar_pointer(0.5, dtype)
    api.call("cudaActivationForward", ctx.handle, api.ACTIVATIONS[activation], a, x.desc.handle, x.mem.handle, b, y.desc.handle, y.mem.handle)
    ref = f(1.25, dtype) * o.activation(x64, activation) + f(0.5, dtype) * y64
    assert o.error_metrics(y.download(ctx), ref)["elem"] <= TOL[dtype]


@pytest.mark.gpu
def test_add_bias_rejects_a_bias_that_does_not_match(ctx):
    x = api.DeviceTensor((2, 4, 4, 8), "float32")
    b = api.DeviceTensor((7,), "float32")
    with pytest.raises(api.AvocadoError) as failure:
        api.call("cudaAddBias", ctx.handle, None, None, x.desc.handle, x.mem.handle, b.desc.handle, b.mem.handle, x.desc.handle, x.mem.handle, None, None, None,
                 api.INVALID, 0)
    assert failure.value.status == api.STATUS["BAD_PARAM"]
