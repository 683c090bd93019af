"""Seeded random shapes and option combinations through every entry point of the path, against the oracles.

The fixed-shape tests pin the configurations of the baseline and the reference's own test shapes; these cases walk the
space between them (odd image sizes, channel counts on both sides of every kernel's block sizes, every epilogue option),
so that a dispatch boundary that only a particular shape reaches does not stay untested.
"""
import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [1, 2])
def test_one_call_convolutions_16bit(ctx, seed):
    r = np.random.default_rng(100 + seed)
    f = lambda v: float(np.float32(v))
    for _ in range(14):
        n, h, w = int(r.integers(1, 9)), int(r.integers(3, 40)), int(r.integers(3, 40))
        c, k = 8 * int(r.integers(1, 33)), 8 * int(r.integers(1, 33))
        dtype = ["float16", "bfloat16"][int(r.integers(0, 2))]
        act = ["linear", "relu", "tanh"][int(r.integers(0, 3))]
        use_z, use_beta, use_bias = (bool(r.integers(0, 2)) for _ in range(3))
        d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
        x = d.x.upload(ctx, r.uniform(-1, 1, d.x.shape))
        wt = d.wt.upload(ctx, r.normal(0, np.sqrt(2.0 / (9 * c)), (k, 3, 3, c)))
        b = d.set_bias(r.uniform(-0.1, 0.1, k)) if use_bias else None
        z = d.set_z(r.uniform(-1, 1, d.y.shape)) if use_z else None
        y0 = r.uniform(-1, 1, d.y.shape)
        ref = None
        for entry in ("winograd_fused", "implicit_gemm"):
            y064 = d.y.upload(ctx, y0)
            if ref is None:
                ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y064 if use_beta else None, alpha1=f(1.1), alpha2=f(0.7), beta=f(0.3) if use_beta else 0.0,
                                       activation=act)
            getattr(d, entry)(alpha1=1.1, alpha2=0.7 if use_z else None, beta=0.3 if use_beta else None, activation=act)
            err = o.error_metrics(d.y.download(ctx), ref)["elem"]
            assert err <= 1e-2, (entry, (n, h, w, c, k), dtype, act, use_z, use_beta, use_bias, err)


@pytest.mark.parametrize("seed", [1, 2])
def test_int8_convolutions_bit_exact(ctx, seed):
    r = np.random.default_rng(200 + seed)
    for _ in range(16):
        n, h, w = int(r.integers(1, 17)), int(r.integers(3, 30)), int(r.integers(3, 30))
        c = [16, 32, 128, 256, 20, 384][int(r.integers(0, 6))]
        k = [16, 32, 64, 96, 256, 272, 12][int(r.integers(0, 7))]
        act = ["linear", "relu"][int(r.integers(0, 2))]
        use_z = bool(r.integers(0, 2))
        alpha1 = [None, None, 0.75][int(r.integers(0, 3))]
        int32_out = bool(r.integers(0, 4) == 0)
        d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8", out_dtype="int32" if int32_out else "int8")
        x = r.integers(-127, 128, (n, h, w, c), dtype=np.int8)
        wt = r.integers(-127, 128, (k, 3, 3, c), dtype=np.int8)
        bias = r.integers(-1000, 1001, k, dtype=np.int32)
        d.x.upload(ctx, x)
        d.wt.upload(ctx, wt)
        d.set_bias(bias)
        scales = z = None
        if not int32_out:
            scales = r.uniform(2e-5, 2e-4, k).astype(np.float32)
            d.set_scales(scales)
            if use_z:
                z = r.integers(-127, 128, (n, h, w, k), dtype=np.int8)
                d.set_z(z)
        d.implicit_gemm(alpha1=None if int32_out else alpha1, alpha2=0.5 if z is not None else None, activation="linear" if int32_out else act)
        ref = o.conv2d_forward_int8(x, wt, bias, scales, z, alpha1=1.0 if (alpha1 is None or int32_out) else alpha1, alpha2=0.5,
                                    activation="linear" if int32_out else act, int32_output=int32_out)
        assert np.array_equal(d.y.download_raw(ctx), ref), ((n, h, w, c, k), act, use_z, alpha1, int32_out)


@pytest.mark.parametrize("seed", [1, 2])
def test_non_fused_pipeline_forward_and_backward(ctx, seed):
    r = np.random.default_rng(300 + seed)
    for _ in range(10):
        n, h, w = int(r.integers(1, 7)), int(r.integers(4, 30)), int(r.integers(4, 30))
        c = [8, 24, 32, 64, 64, 72, 128, 21][int(r.integers(0, 8))]
        k = [8, 16, 64, 64, 40, 128, 13][int(r.integers(0, 7))]
        ts = [2, 4][int(r.integers(0, 2))]
        dtype = ["float32", "float32", "float16"][int(r.integers(0, 3))]
        training = dtype == "float32"
        p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, "float32", ts, 3, training=training)
        x = p.x.upload(ctx, r.uniform(-1, 1, p.x.shape))
        wt = p.wt.upload(ctx, r.normal(0, np.sqrt(2.0 / (9 * c)), (k, 3, 3, c)))
        tol = 1e-3 if dtype == "float32" else 1e-2
        if training:
            dy = p.dy.upload(ctx, r.uniform(-1, 1, p.dy.shape))
            p.training_step()
            assert o.error_metrics(p.dx.download(ctx), o.conv2d_backward_data(dy, wt, (h, w)))["elem"] <= tol, ("dx", n, h, w, c, k, ts)
            assert o.error_metrics(p.dw.download(ctx), o.conv2d_backward_weights(x, dy))["elem"] <= tol, ("dw", n, h, w, c, k, ts)
        else:
            p.forward()
        assert o.error_metrics(p.y.download(ctx), o.conv2d_forward(x, wt))["elem"] <= tol, ("y", n, h, w, c, k, ts, dtype)
