"""cudaOptimizerLearn (the weight update after the dW all-reduce) against the float64 restatement of the reference's formulas."""
import ctypes

import numpy as np
import pytest

from cudabackend_b200 import api
from oracle import oracle as o

pytestmark = pytest.mark.gpu

SGD, ADAM = 0, 1


class Optimizer:
    def __init__(self, kind, learning_rate, coef=(0.0, 0.0, 0.0, 0.0), flags=(False, False, False, False), steps=0):
        h = api._H(api.INVALID)
        api.call("cudaCreateOptimizerDescriptor", ctypes.byref(h))
        self.handle = h.value
        api.call("cudaSetOptimizerDescriptor", self.handle, kind, steps, float(learning_rate), (ctypes.c_double * 4)(*coef), (ctypes.c_bool * 4)(*flags))

    def steps(self):
        kind, steps, lr = api._INT(), api._I64(), ctypes.c_double()
        coef, flags = (ctypes.c_double * 4)(), (ctypes.c_bool * 4)()
        api.call("cudaGetOptimizerDescriptor", self.handle, ctypes.byref(kind), ctypes.byref(steps), ctypes.byref(lr), coef, flags)
        return steps.value

    def workspace_bytes(self, w_desc):
        size = api._I64()
        api.call("cudaGetOptimizerWorkspaceSize", self.handle, w_desc.handle, ctypes.byref(size))
        return size.value


def learn(ctx, opt, w, dw, workspace, alpha=None, beta=None):
    a, ka = api.scalar_pointer(alpha, w.dtype)
    b, kb = api.scalar_pointer(beta, w.dtype)
    api.call("cudaOptimizerLearn", ctx.handle, opt.handle, a, dw.desc.handle, dw.mem.handle, b, w.desc.handle, w.mem.handle,
             workspace.handle if workspace is not None else api.INVALID)


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("momentum,nesterov", [(False, False), (True, False), (True, True)])
def test_sgd(ctx, dtype, momentum, nesterov):
    shape = (64, 3, 3, 64)
    r = np.random.default_rng(31)
    w = api.DeviceTensor(shape, dtype)
    dw = api.DeviceTensor(shape, dtype)
    w64 = w.upload(ctx, r.normal(0, 0.1, shape))
    opt = Optimizer(SGD, 0.05, coef=(0.9, 0, 0, 0), flags=(momentum, nesterov, False, False))
    assert opt.workspace_bytes(w.desc) == (w.desc.nbytes if momentum else 0)
    workspace = api.Memory(w.desc.nbytes) if momentum else None
    if workspace is not None:
        workspace.zero(ctx)
    state = np.zeros(shape) if momentum else None
    eps = np.finfo(np.float32 if dtype == "float32" else np.float64).eps
    for step in range(3):
        g64 = dw.upload(ctx, r.normal(0, 1, shape))
        learn(ctx, opt, w, dw, workspace, alpha=1.0, beta=1.0)
        w64, state = o.optimizer_learn("sgd", w64, g64, state, 0.05, (0.9, 0.0), momentum, nesterov, alpha=1.0, beta=1.0, eps=eps)
        got = w.download(ctx)
        assert np.max(np.abs(got - w64)) <= (1e-6 if dtype == "float32" else 1e-14)
        w64 = got  # continue from the stored values so that rounding does not accumulate in the comparison


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_adam(ctx, dtype):
    shape = (21, 5, 5, 13)
    r = np.random.default_rng(32)
    w = api.DeviceTensor(shape, dtype)
    dw = api.DeviceTensor(shape, dtype)
    w64 = w.upload(ctx, r.normal(0, 0.1, shape))
    opt = Optimizer(ADAM, 1e-3, coef=(0.9, 0.999, 0, 0))
    assert opt.workspace_bytes(w.desc) == 2 * w.desc.nbytes
    workspace = api.Memory(2 * w.desc.nbytes)
    workspace.zero(ctx)
    state = (np.zeros(shape), np.zeros(shape))
    eps = np.finfo(np.float32 if dtype == "float32" else np.float64).eps
    for step in range(4):
        g64 = dw.upload(ctx, r.normal(0, 1, shape))
        learn(ctx, opt, w, dw, workspace, alpha=1.0, beta=1.0)
        w64, state = o.optimizer_learn("adam", w64, g64, state, 1e-3, (0.9, 0.999), steps=step, alpha=1.0, beta=1.0, eps=eps)
        got = w.download(ctx)
        assert np.all(np.isfinite(got))
        assert np.max(np.abs(got - w64)) <= (2e-6 if dtype == "float32" else 1e-13)
        assert opt.steps() == step + 1
        w64 = got


def test_optimizer_rejects_a_small_workspace_and_other_dtypes(ctx):
    w = api.DeviceTensor((8, 8), "float32")
    dw = api.DeviceTensor((8, 8), "float32")
    opt = Optimizer(ADAM, 1e-3, coef=(0.9, 0.999, 0, 0))
    small = api.Memory(w.desc.nbytes)
    with pytest.raises(api.AvocadoError) as failure:
        learn(ctx, opt, w, dw, small)
    assert failure.value.status == api.STATUS["INTERNAL_ERROR"]
    wh = api.DeviceTensor((8, 8), "float16")
    dh = api.DeviceTensor((8, 8), "float16")
    with pytest.raises(api.AvocadoError) as failure:
        learn(ctx, Optimizer(SGD, 0.1), wh, dh, None)
    assert failure.value.status == api.STATUS["UNSUPPORTED_DATATYPE"]
