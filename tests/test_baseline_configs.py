"""GPU parity tests of the five benchmark configurations at their STATED sizes, through the C ABI, whole output compared.

The persistent tensor-core kernels walk several tiles per CTA only at these sizes (a TMEM accumulator ring that wraps,
barrier phases that flip more than once), so the reduced-batch cases of test_conv_pipeline.py do not reach the code
the benchmark numbers are measured on; these do.  Inputs are the seeded distributions the configurations name.

Tolerances (max |err| / max(|ref|, rms(ref)) against the float64 direct convolution): 1e-3 float32, 1e-2 float16 /
bfloat16.  The float16-matrices variant of configuration 2 is the one exception: F(4x4,3x3) with a 10-bit-mantissa
transform domain has an error floor near 5e-2 for any implementation (the reference, which also accumulates in
float16, is worse), so it is held to 8e-2 element-wise and 8e-3 rms, and the float32-matrices variant to 1e-2.
"""
import numpy as np
import pytest

from cudabackend_b200 import pipeline
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu


def test_config1_stated_size(ctx):
    """N=2, 16x16, C=K=32, float32, non-fused F(4x4,3x3), bias 0"""
    p = pipeline.WinogradNonFused(ctx, 2, 16, 16, 32, 32, "float32", None, 4, 3)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(32, 3, 32))
    p.set_bias(np.zeros(32))
    p.forward()
    err = o.error_metrics(p.y.download(ctx), o.conv2d_forward(x, wt))
    assert err["elem"] <= common.TOLERANCE["float32"], err


@pytest.mark.parametrize("matrices,elem_bound,rms_bound", [("float16", 8e-2, 8e-3), ("float32", 1e-2, 1e-3)])
def test_config2_stated_size(ctx, matrices, elem_bound, rms_bound):
    """N=64, 56x56, C=K=64, float16, non-fused F(4x4,3x3): 12 544 tiles, 3 528 GEMM tiles on 296 CTAs"""
    p = pipeline.WinogradNonFused(ctx, 64, 56, 56, 64, 64, "float16", matrices, 4, 3)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(64, 3, 64))
    p.forward()
    err = o.error_metrics(p.y.download(ctx), o.conv2d_forward(x, wt))
    assert err["elem"] <= elem_bound and err["rms"] <= rms_bound, err


def test_config2_stated_size_fused_output(ctx):
    """the same layer with the contraction and the output transform in one kernel (opt-in fusion of the context)"""
    if not hasattr(pipeline.WinogradNonFused, "enable_fusion"):
        pytest.skip("fusion of the contraction with the output transform is not built")
    p = pipeline.WinogradNonFused(ctx, 64, 56, 56, 64, 64, "float16", "float16", 4, 3)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(64, 3, 64))
    p.enable_fusion(True)
    try:
        p.forward()
        got = p.y.download(ctx)
    finally:
        p.enable_fusion(False)
    err = o.error_metrics(got, o.conv2d_forward(x, wt))
    assert err["elem"] <= 8e-2 and err["rms"] <= 8e-3, err


def test_config3_stated_size(ctx):
    """N=128, 28x28, C=K=128, bfloat16, one-call Winograd with bias + ReLU"""
    d = pipeline.DirectConvolution(ctx, 128, 28, 28, 128, 128, "bfloat16")
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(128, 3, 128))
    b = d.set_bias(common.uniform("b", (128,), -0.1, 0.1))
    d.winograd_fused(activation="relu")
    err = o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt, bias=b, activation="relu"))
    assert err["elem"] <= common.TOLERANCE["bfloat16"], err


def test_config3_stated_size_implicit_gemm(ctx):
    """the same layer through the implicit-GEMM entry point (float32 accumulation: only the final rounding remains)"""
    d = pipeline.DirectConvolution(ctx, 128, 28, 28, 128, 128, "bfloat16")
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(128, 3, 128))
    b = d.set_bias(common.uniform("b", (128,), -0.1, 0.1))
    d.implicit_gemm(activation="relu")
    err = o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt, bias=b, activation="relu"))
    assert err["elem"] <= common.TOLERANCE["bfloat16"], err


@pytest.mark.parametrize("scale_range", [(1e-3, 1e-2), (5e-5, 2e-4)], ids=["stated_scales", "unsaturated_scales"])
def test_config4_stated_size_bit_exact(ctx, scale_range):
    """N=256, 14x14, C=K=256, int8 with int32 bias and per-channel scales: 392 tiles on 148 CTAs, bit exact.
    With the stated scales most outputs saturate, so the second case uses scales that keep them inside the range."""
    n, h, w, c, k = 256, 14, 14, 256, 256
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8")
    x = common.int8_uniform("x", (n, h, w, c))
    wt = common.int8_uniform("w", (k, 3, 3, c))
    bias = common.rng("b").integers(-1000, 1001, k, dtype=np.int32)
    scales = common.rng("scales").uniform(scale_range[0], scale_range[1], k).astype(np.float32)
    d.x.upload(ctx, x)
    d.wt.upload(ctx, wt)
    d.set_bias(bias)
    d.set_scales(scales)
    d.implicit_gemm()
    assert np.array_equal(d.y.download_raw(ctx), o.conv2d_forward_int8(x, wt, bias, scales))


@pytest.mark.parametrize("batch", [32, 256], ids=["per_gpu_share_of_8", "whole_batch"])
def test_config5_stated_size(ctx, batch):
    """56x56, C=K=64, float32 training step (forward, dX, dW) at the whole batch of 256 and at the 32 images one of 8 GPUs gets"""
    h, w, c, k = 56, 56, 64, 64
    p = pipeline.WinogradNonFused(ctx, batch, h, w, c, k, "float32", None, 4, 3, training=True)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    dy = p.dy.upload(ctx, common.uniform("dy", p.dy.shape))
    p.training_step()
    y, dx, dw = p.y.download(ctx), p.dx.download(ctx), p.dw.download(ctx)
    assert o.error_metrics(y, o.conv2d_forward(x, wt))["elem"] <= common.TOLERANCE["float32"]
    assert o.error_metrics(dx, o.conv2d_backward_data(dy, wt, (h, w)))["elem"] <= common.TOLERANCE["float32"]
    assert o.error_metrics(dw, o.conv2d_backward_weights(x, dy))["elem"] <= common.TOLERANCE["float32"]
