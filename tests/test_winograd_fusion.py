"""GPU tests of the opt-in fusion of cudaGemmBatched with cudaWinogradOutputTransform (F(4x4,3x3), 16-bit tensors).

With cudaContextSetWinogradFusion on, the batched GEMM of the pipeline is held back and the output transform that
consumes its result runs ONE kernel (contraction on tcgen05, products kept in TMEM, output transform in the epilogue).
Two things are checked:
  * the arithmetic: y against the float64 oracle applied to the same stored V and U (the fused kernel never rounds the
    products to 16 bits, so its only error is float32 accumulation plus the final rounding), over ragged tile counts,
    channel and filter counts that are not multiples of the kernel's blocks, every epilogue combination and both
    16-bit types;
  * the deferral: whatever the caller does between the two calls, or instead of the second, the observable result is
    that of the unfused calls, except that the products are not written when the fusion takes place.
"""
import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu


def make(ctx, shape, k, dtype, mdtype=None):
    n, h, w, c = shape
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, mdtype, 4, 3)
    v = p.v.upload(ctx, common.uniform("x", p.v.shape, extra=11))
    u = p.u.upload(ctx, common.uniform("w", p.u.shape, -0.5, 0.5, extra=11))
    return p, v, u


def tolerance(ref, dtype):
    # float32 accumulation of C products per plane, 36 planes combined with coefficients up to 8, one final rounding
    return 4.0 * common.EPS[dtype] * max(float(np.abs(ref).max()), 1e-30)


# 2x7x9: two tile rows, ragged edges; 40 channels: a partial 64-channel block; 24 filters: a partial 16-filter block;
# 5x20x24: 150 tiles (more than one block of 128); 3x56x56x64 -> 64: the ResNet geometry, 588 tiles
SHAPES = [((2, 7, 9, 40), 24), ((5, 20, 24, 64), 64), ((3, 56, 56, 64), 64), ((1, 4, 4, 8), 8), ((2, 13, 30, 136), 72)]


@pytest.mark.parametrize("shape,k", SHAPES)
@pytest.mark.parametrize("dtype,mdtype", [("float16", "float16"), ("bfloat16", "bfloat16"), ("bfloat16", "float16")])
def test_fused_contraction_and_output_transform(ctx, shape, k, dtype, mdtype):
    p, v, u = make(ctx, shape, k, dtype, mdtype)
    bias = p.set_bias(common.uniform("b", (k,)))
    p.enable_fusion(True)
    p.gemm(p.v, p.u, p.m, False, True)
    p.output_transform(activation="relu", use_z=False)
    got = p.y.download(ctx)
    p.enable_fusion(False)
    ref = o.winograd_output_transform(o.gemm_batched(v, u, trans_b=True), p.y.shape, 4, 3, bias=bias, activation="relu")
    assert np.abs(got - ref).max() <= tolerance(ref, dtype)


@pytest.mark.parametrize("use_bias,use_z", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("activation", ["linear", "relu", "tanh"])
def test_fused_epilogue_combinations(ctx, use_bias, use_z, activation):
    p, v, u = make(ctx, (2, 10, 11, 32), 24, "float16")
    bias = p.set_bias(common.uniform("b", (24,))) if use_bias else None
    z = p.set_z(common.uniform("z", p.y.shape)) if use_z else None
    y0 = p.y.upload(ctx, common.uniform("y", p.y.shape))
    p.enable_fusion(True)
    p.gemm(p.v, p.u, p.m, False, True)
    p.output_transform(alpha1=1.1, alpha2=1.2, beta=0.1, activation=activation)
    got = p.y.download(ctx)
    p.enable_fusion(False)
    f32 = lambda value: float(np.float32(value))
    ref = o.winograd_output_transform(o.gemm_batched(v, u, trans_b=True), p.y.shape, 4, 3, bias=bias, z=z, y=y0, alpha1=f32(1.1), alpha2=f32(1.2),
                                      beta=f32(0.1), activation=activation)
    assert np.abs(got - ref).max() <= tolerance(ref, "float16")


def test_products_are_not_written_when_the_fusion_takes_place(ctx):
    """the one observable difference of the opt-in: the workspace of M keeps what it held"""
    p, v, u = make(ctx, (2, 12, 12, 64), 32, "float16")
    marker = np.full(p.m.shape, 7.0)
    p.m.upload(ctx, marker)
    p.enable_fusion(True)
    p.gemm(p.v, p.u, p.m, False, True)
    p.output_transform(use_bias=False, use_z=False)
    y = p.y.download(ctx)
    assert np.array_equal(p.m.download(ctx), marker)
    p.enable_fusion(False)
    ref = o.winograd_output_transform(o.gemm_batched(v, u, trans_b=True), p.y.shape, 4, 3)
    assert np.abs(y - ref).max() <= tolerance(ref, "float16")


def test_any_other_call_launches_the_held_back_gemm(ctx):
    """reading M, synchronising, or transforming another tensor after the GEMM: M must be there, as without fusion"""
    p, v, u = make(ctx, (2, 12, 12, 64), 32, "float16")
    m_ref = o.gemm_batched(v, u, trans_b=True)
    near = lambda got: np.abs(got - m_ref).max() <= 4 * common.EPS["float16"] * np.abs(m_ref).max()
    p.enable_fusion(True)

    p.m.upload(ctx, np.zeros(p.m.shape))
    p.gemm(p.v, p.u, p.m, False, True)
    assert near(p.m.download(ctx))  # the copy to the host is "another call"

    p.m.upload(ctx, np.zeros(p.m.shape))
    p.gemm(p.v, p.u, p.m, False, True)
    ctx.synchronize()
    assert near(p.m.download(ctx))

    # an output transform of a DIFFERENT tensor does not consume the held-back product
    other = api.DeviceTensor(p.m.shape, "float16")
    other_values = other.upload(ctx, common.uniform("x", p.m.shape, extra=12))
    p.m.upload(ctx, np.zeros(p.m.shape))
    p.gemm(p.v, p.u, p.m, False, True)
    p.output_transform(matrices=other, use_bias=False, use_z=False)
    y = p.y.download(ctx)
    assert near(p.m.download(ctx))
    ref = o.winograd_output_transform(other_values, p.y.shape, 4, 3)
    assert np.abs(y - ref).max() <= tolerance(ref, "float16")

    # two GEMMs in a row: the first is launched when the second arrives
    second = api.DeviceTensor(p.m.shape, "float16")
    p.m.upload(ctx, np.zeros(p.m.shape))
    p.gemm(p.v, p.u, p.m, False, True)
    p.gemm(p.v, p.u, second, False, True)
    assert near(p.m.download(ctx)) and near(second.download(ctx))

    # freeing memory while a product is held back: the GEMM is launched before the memory goes
    p.m.upload(ctx, np.zeros(p.m.shape))
    p.gemm(p.v, p.u, p.m, False, True)
    other.mem.destroy()
    assert near(p.m.download(ctx))
    p.enable_fusion(False)


def test_cases_outside_the_fused_kernel_take_the_two_kernel_path(ctx):
    """float32 matrices, F(2x2,3x3), alpha != 1: nothing is held back, results are those of the unfused calls"""
    n, h, w, c, k = 2, 9, 10, 16, 8
    for dtype, mdtype, ts in (("float16", "float32", 4), ("float16", "float16", 2), ("float32", None, 4)):
        p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, mdtype, ts, 3)
        x = p.x.upload(ctx, common.uniform("x", p.x.shape))
        wt = p.wt.upload(ctx, common.he_normal_weights(k, 3, c))
        p.enable_fusion(True)
        p.forward()
        got = p.y.download(ctx)
        p.enable_fusion(False)
        err = o.error_metrics(got, o.conv2d_forward(x, wt))["elem"]
        assert err <= (8e-2 if (mdtype == "float16" and ts == 4) else common.TOLERANCE[dtype]), (dtype, mdtype, ts, err)


def test_fused_pipeline_in_a_captured_graph(ctx):
    """the deferral is host-side state: capturing the four calls records three kernels, replay gives the same y"""
    n, h, w, c, k = 4, 28, 28, 64, 64
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, "float16", None, 4, 3)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    p.enable_fusion(True)
    graph = ctx.capture(p.forward)
    p.y.mem.zero(ctx)
    graph.launch()
    graph.launch()
    got = p.y.download(ctx)
    graph.destroy()
    p.enable_fusion(False)
    err = o.error_metrics(got, o.conv2d_forward(x, wt))
    assert err["elem"] <= 8e-2 and err["rms"] <= 8e-3, err


def test_weight_transform_rides_with_the_input_transform(ctx):
    """FUSE_WEIGHTS: U and V are what the separate launches give, bit for bit, whichever launch computed U; a weight
    transform that is not followed by an input transform still happens"""
    for dtype, mdtype, ts, shape, k in (("float16", None, 4, (2, 9, 11, 40), 24), ("bfloat16", "float16", 2, (3, 14, 14, 64), 32),
                                        ("float32", None, 4, (2, 12, 12, 32), 16), ("float16", "float32", 4, (1, 8, 8, 16), 8)):
        n, h, w, c = shape
        p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, mdtype, ts, 3)
        p.x.upload(ctx, common.uniform("x", p.x.shape))
        p.wt.upload(ctx, common.he_normal_weights(k, 3, c))
        for rotated in (False, True):
            p.weight_transform(rotated=rotated)
            p.input_transform()
            u_ref, v_ref = p.u.download_raw(ctx), p.v.download_raw(ctx)
            p.u.mem.zero(ctx)
            p.v.mem.zero(ctx)
            p.enable_fusion(api.FUSE_WEIGHTS)
            p.weight_transform(rotated=rotated)
            p.input_transform()
            assert np.array_equal(p.u.download_raw(ctx), u_ref) and np.array_equal(p.v.download_raw(ctx), v_ref), (dtype, mdtype, ts, rotated)
            p.u.mem.zero(ctx)
            p.weight_transform(rotated=rotated)  # held back ...
            assert np.array_equal(p.u.download_raw(ctx), u_ref)  # ... until the copy to the host asks for it
            p.enable_fusion(0)
    # a 5x5 kernel and float64 are outside the ride: nothing is held back, results unchanged
    p = pipeline.WinogradNonFused(ctx, 1, 6, 5, 6, 4, "float64", None, 2, 5)
    w64 = p.wt.upload(ctx, common.he_normal_weights(4, 5, 6))
    p.enable_fusion(api.FUSE_WEIGHTS)
    p.weight_transform()
    p.enable_fusion(0)
    assert np.abs(p.u.download(ctx) - o.winograd_weight_transform(w64, 2)).max() <= 1e-12


def test_fusion_flags_are_validated(ctx):
    assert api.call_status("cudaContextSetWinogradFusion", ctx.handle, 4) == api.STATUS["BAD_PARAM"]
    assert api.call_status("cudaContextSetWinogradFusion", ctx.handle, 3) == api.STATUS["SUCCESS"]
    assert api.call_status("cudaContextSetWinogradFusion", ctx.handle, 0) == api.STATUS["SUCCESS"]


def test_default_context_cannot_fuse(library, device_count):
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    assert api.call_status("cudaContextSetWinogradFusion", api.load().cudaGetDefaultContext(0), 1) == api.STATUS["BAD_PARAM"]
