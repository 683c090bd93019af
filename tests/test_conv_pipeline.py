"""GPU parity tests of whole convolutions through the C ABI against the float64 direct-convolution oracle.

Tolerances are the ones the task states: max error relative to max(|ref|, rms(ref)) <= 1e-3 for float32 and
<= 1e-2 for float16 / bfloat16.  F(4x4,3x3) with 16-bit transform-domain tensors cannot meet 1e-2 (its error is
set by the 10-bit mantissa of the stored matrices, about 5e-2); that variant is checked against its own bound
and the float32-matrices variant against 1e-2.
"""
import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from tests import common

pytestmark = pytest.mark.gpu


def forward_case(ctx, n, h, w, c, k, dtype, mdtype, ts, ks=3, bias=False, activation="linear"):
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, mdtype, ts, ks)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(k, ks, c))
    b = p.set_bias(common.uniform("b", (k,), -0.1, 0.1)) if bias else None
    p.forward(activation=activation)
    got = p.y.download(ctx)
    ref = o.conv2d_forward(x, wt, bias=b, padding=p.padding, activation=activation)
    return o.error_metrics(got, ref)


def test_config1_fp32_f43(ctx):
    """N=2, 16x16, C=K=32, float32, F(4x4,3x3)"""
    err = forward_case(ctx, 2, 16, 16, 32, 32, "float32", None, 4)
    assert err["elem"] <= common.TOLERANCE["float32"], err


@pytest.mark.parametrize("ts,ks", [(2, 3), (4, 3), (2, 5)])
@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_reference_test_shape(ctx, ts, ks, dtype):
    """the awkward shape of the reference's tests: 12x13x14x135 -> 21 filters"""
    err = forward_case(ctx, 12, 13, 14, 135, 21, dtype, None, ts, ks, bias=True, activation="relu")
    assert err["elem"] <= common.TOLERANCE[dtype], err


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_f23_16bit(ctx, dtype):
    err = forward_case(ctx, 4, 28, 28, 64, 64, dtype, None, 2)
    assert err["elem"] <= (1e-2 if dtype == "float16" else 4e-2), err


def test_config2_shape_fp16_matrices_fp16(ctx):
    """cfg 2 geometry at reduced batch with float16 matrices: error is bounded by the fp16 transform domain"""
    err = forward_case(ctx, 8, 56, 56, 64, 64, "float16", "float16", 4)
    assert err["elem"] <= 8e-2 and err["rms"] <= 8e-3, err


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_config2_shape_fp32_matrices(ctx, dtype):
    """16-bit activations, float32 transform domain: within the stated 1e-2"""
    err = forward_case(ctx, 8, 56, 56, 64, 64, dtype, "float32", 4)
    assert err["elem"] <= common.TOLERANCE[dtype], err


def test_training_step_fp32(ctx):
    """cfg 5 geometry at reduced batch: forward, dX and dW"""
    n, h, w, c, k = 4, 56, 56, 64, 64
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, "float32", None, 4, 3, training=True)
    x = p.x.upload(ctx, common.uniform("x", p.x.shape))
    wt = p.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    dy = p.dy.upload(ctx, common.uniform("dy", p.dy.shape))
    p.training_step()
    y, dx, dw = p.y.download(ctx), p.dx.download(ctx), p.dw.download(ctx)
    assert o.error_metrics(y, o.conv2d_forward(x, wt))["elem"] <= 1e-3
    assert o.error_metrics(dx, o.conv2d_backward_data(dy, wt, (h, w)))["elem"] <= 1e-3
    assert o.error_metrics(dw, o.conv2d_backward_weights(x, dy))["elem"] <= 1e-3


@pytest.mark.parametrize("entry", ["implicit_gemm", "winograd_fused"])
@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32", "float64"])
def test_one_call_convolution_small(ctx, entry, dtype):
    n, h, w, c, k = 2, 9, 10, 24, 16
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    z = d.set_z(common.uniform("z", d.y.shape))
    y0 = d.y.upload(ctx, common.uniform("y", d.y.shape))
    getattr(d, entry)(alpha1=1.1, alpha2=1.2, beta=0.1, activation="relu")
    got = d.y.download(ctx)
    f = (lambda v: float(np.float32(v))) if dtype != "float64" else (lambda v: v)
    ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y0, alpha1=f(1.1), alpha2=f(1.2), beta=f(0.1), activation="relu")
    assert o.error_metrics(got, ref)["elem"] <= common.TOLERANCE[dtype]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 16, 16, 64, 64),     # 192 tiles: two blocks, the second half full
                                   (5, 14, 18, 128, 72),    # 315 tiles: three blocks, the last one partial; filters end inside a block
                                   (1, 20, 22, 72, 136),    # 110 tiles: less than one block; partial channel block, three filter blocks
                                   (9, 13, 15, 40, 24)])    # 504 tiles (ragged edges): four blocks, fewer filters than half a block
def test_one_call_winograd_block_edges(ctx, dtype, shape):
    """the one-call F(2x2,3x3) convolution at the edges of its contraction + output kernel's blocks (128 tiles x 64 filters x
    64 channels): odd block counts, partial tile, filter and channel blocks, every epilogue term"""
    n, h, w, c, k = shape
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    d.winograd_fused(activation="relu")
    bound = 1e-2 if dtype == "float16" else 4e-2  # bfloat16 tensors, float16 transform domain
    assert o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt, bias=b, activation="relu"))["elem"] <= bound
    z = d.set_z(common.uniform("z", d.y.shape))
    y0 = d.y.upload(ctx, common.uniform("y", d.y.shape))
    d.winograd_fused(alpha1=1.1, alpha2=1.2, beta=0.1, activation="tanh")
    f = lambda v: float(np.float32(v))
    ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y0, alpha1=f(1.1), alpha2=f(1.2), beta=f(0.1), activation="tanh")
    assert o.error_metrics(d.y.download(ctx), ref)["elem"] <= bound
    assert ctx.last_device_status() == 0


def test_config3_shape_fused_bf16(ctx):
    """cfg 3 geometry at reduced batch: bf16, bias + ReLU"""
    n, h, w, c, k = 4, 28, 28, 128, 128
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "bfloat16")
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    d.winograd_fused(activation="relu")
    got = d.y.download(ctx)
    ref = o.conv2d_forward(x, wt, bias=b, activation="relu")
    assert o.error_metrics(got, ref)["elem"] <= common.TOLERANCE["bfloat16"]


def int8_case(ctx, n, h, w, c, k, scale_range, activation="linear", with_z=False, int32_output=False, ks=3, rotated=False):
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8", out_dtype="int32" if int32_output else "int8", kernel_size=ks)
    if rotated:
        d.conv = api.ConvolutionDescriptor(api.CROSS_CORRELATION_MODE, (-(ks // 2), -(ks // 2)))
    x = common.int8_uniform("x", (n, h, w, c))
    wt = common.int8_uniform("w", (k, ks, ks, c))
    bias = common.rng("b").integers(-1000, 1001, k, dtype=np.int32)
    d.x.upload(ctx, x)
    d.wt.upload(ctx, wt)
    d.set_bias(bias)
    scales = None
    z = None
    if not int32_output:
        scales = common.rng("scales").uniform(scale_range[0], scale_range[1], k).astype(np.float32)
        d.set_scales(scales)
        if with_z:
            z = common.int8_uniform("z", (n, h, w, k))
            d.set_z(z)
    d.implicit_gemm(alpha2=0.5 if with_z else None, activation=activation)
    got = d.y.download_raw(ctx)
    w_eff = np.ascontiguousarray(wt[:, ::-1, ::-1, :]) if rotated else wt
    pad = -(ks // 2)
    ref = o.conv2d_forward_int8(x, w_eff, bias, scales, z, padding=(pad, pad), alpha2=0.5, activation=activation, int32_output=int32_output)
    return got, ref


def test_int8_bit_exact_config4_distribution(ctx):
    """cfg 4 geometry at reduced batch with the stated scales (most outputs saturate)"""
    got, ref = int8_case(ctx, 8, 14, 14, 256, 256, (1e-3, 1e-2))
    assert np.array_equal(got, ref)


def test_int8_bit_exact_unsaturated(ctx):
    """scales chosen so that nearly all outputs stay inside (-128, 127): rounding is what is being tested"""
    got, ref = int8_case(ctx, 8, 14, 14, 256, 256, (5e-5, 2e-4), activation="relu", with_z=True)
    assert np.array_equal(got, ref)
    assert np.mean(np.abs(ref.astype(np.int32)) < 127) > 0.9


def test_int8_int32_output_and_ragged_channels(ctx):
    got, ref = int8_case(ctx, 2, 7, 9, 20, 12, None, int32_output=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, 2, 7, 9, 20, 12, (5e-4, 2e-3))
    assert np.array_equal(got, ref)


def test_int8_round_half_to_even(ctx):
    d = pipeline.DirectConvolution(ctx, 1, 1, 1, 16, 16, "int8")
    x = np.zeros((1, 1, 1, 16), dtype=np.int8)
    x[0, 0, 0, 0] = 1
    wt = np.zeros((16, 3, 3, 16), dtype=np.int8)
    values = [1, 3, 5, -1, -3, 127, -127, 7, 9, 11, -5, -7, 2, 4, 0, 13]
    for k, v in enumerate(values):
        wt[k, 1, 1, 0] = v
    d.x.upload(ctx, x)
    d.wt.upload(ctx, wt)
    d.set_scales(np.full(16, 0.5, dtype=np.float32))
    d.implicit_gemm()
    got = d.y.download_raw(ctx).reshape(-1)
    expect = o.conv2d_forward_int8(x, wt, None, np.full(16, 0.5, dtype=np.float32)).reshape(-1)
    assert got.tolist() == expect.tolist() == [0, 2, 2, 0, -2, 64, -64, 4, 4, 6, -2, -4, 1, 2, 0, 6]


@pytest.mark.parametrize("shape", [(8, 14, 14, 128, 64), (3, 20, 17, 256, 96), (16, 7, 9, 384, 272), (32, 28, 28, 128, 256)])
def test_int8_tensor_core_shapes(ctx, shape):
    """shapes that take the tcgen05 kernel: ragged pixel counts, K below / between / above the column-block sizes,
    and more 256-filter tiles than CTA pairs (every pair walks several tiles)"""
    n, h, w, c, k = shape
    got, ref = int8_case(ctx, n, h, w, c, k, (5e-5, 2e-4), activation="relu", with_z=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, n, h, w, c, k, None, int32_output=True)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("shape", [(3, 8, 16, 128, 64),    # 384 pixels: three 128-pixel blocks, the last pair's second CTA has no rows; 9 contraction blocks
                                   (1, 15, 20, 256, 128),  # 300 pixels: the second CTA's block is partial; 18 contraction blocks, 128-filter tile
                                   (2, 10, 13, 64, 272),   # 260 pixels, partial channel block (64 of 128), filters end inside the second 256-block
                                   (5, 9, 9, 384, 16),     # 27 contraction blocks (odd: the last stage holds one block), smallest filter count
                                   (2, 8, 8, 128, 256)])   # exactly 128 pixels: stays on the single-CTA kernel
def test_int8_cta_pair_edges(ctx, shape):
    """the CTA-pair kernel's own edges: odd block counts, stages that hold one contraction block instead of two, every
    filter-tile width"""
    n, h, w, c, k = shape
    got, ref = int8_case(ctx, n, h, w, c, k, (5e-5, 2e-4), activation="relu", with_z=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, n, h, w, c, k, None, int32_output=True)
    assert np.array_equal(got, ref)
    assert ctx.last_device_status() == 0


def test_int8_tensor_core_rotated_and_5x5(ctx):
    got, ref = int8_case(ctx, 8, 14, 14, 128, 64, (5e-5, 2e-4), rotated=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, 8, 14, 14, 128, 64, (2e-5, 8e-5), ks=5)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(8, 14, 14, 128, 128), (4, 28, 28, 64, 72), (2, 30, 31, 192, 320)])
def test_implicit_gemm_tensor_core_16bit(ctx, dtype, shape):
    n, h, w, c, k = shape
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    z = d.set_z(common.uniform("z", d.y.shape))
    y0 = d.y.upload(ctx, common.uniform("y", d.y.shape))
    d.implicit_gemm(alpha1=1.1, alpha2=1.2, beta=0.1, activation="relu")
    got = d.y.download(ctx)
    f = lambda v: float(np.float32(v))
    ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y0, alpha1=f(1.1), alpha2=f(1.2), beta=f(0.1), activation="relu")
    # float32 accumulation: the error is the rounding of the stored result
    assert o.error_metrics(got, ref)["elem"] <= {"float16": 1.5e-3, "bfloat16": 1e-2}[dtype]


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("activation", ["linear", "relu", "tanh"])
def test_implicit_gemm_tensor_core_16bit_bias_only(ctx, dtype, activation):
    """without z and beta the kernel takes its short epilogue (linear, relu) or the general one (tanh)"""
    n, h, w, c, k = 4, 28, 28, 64, 72
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    d.implicit_gemm(alpha1=0.9, activation=activation)
    ref = o.conv2d_forward(x, wt, bias=b, alpha1=float(np.float32(0.9)), activation=activation)
    assert o.error_metrics(d.y.download(ctx), ref)["elem"] <= {"float16": 1.5e-3, "bfloat16": 1e-2}[dtype]


def test_int8_short_and_general_epilogue_agree(ctx):
    """alpha1 != 1 and a transcendental activation take the general epilogue; both stay bit-exact against the oracle"""
    n, h, w, c, k = 8, 14, 14, 128, 64
    for alpha1, activation in ((None, "relu"), (0.75, "relu"), (None, "sigmoid")):
        d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8")
        x = common.int8_uniform("x", (n, h, w, c))
        wt = common.int8_uniform("w", (k, 3, 3, c))
        bias = common.rng("b").integers(-1000, 1001, k, dtype=np.int32)
        scales = common.rng("scales").uniform(5e-5, 2e-4, k).astype(np.float32)
        z = common.int8_uniform("z", (n, h, w, k))
        d.x.upload(ctx, x)
        d.wt.upload(ctx, wt)
        d.set_bias(bias)
        d.set_scales(scales)
        d.set_z(z)
        d.implicit_gemm(alpha1=alpha1, alpha2=0.5, activation=activation)
        got = d.y.download_raw(ctx)
        ref = o.conv2d_forward_int8(x, wt, bias, scales, z, alpha1=1.0 if alpha1 is None else alpha1, alpha2=0.5, activation=activation)
        if activation == "sigmoid":
            # expf on the device and exp in the oracle may differ by an ulp, which can move a value across a rounding boundary
            assert np.max(np.abs(got.astype(np.int32) - ref.astype(np.int32))) <= 1
        else:
            assert np.array_equal(got, ref), (alpha1, activation)


@pytest.mark.parametrize("shape", [(2, 14, 14, 64, 64), (2, 7, 9, 48, 16), (4, 12, 12, 16, 32), (1, 16, 8, 144, 80)])
def test_int8_tensor_core_small_and_partial_channel_blocks(ctx, shape):
    """small layers and channel counts that do not fill the kernel's 128-byte channel blocks (C = 64, 48, 16, 144) also run
    on the tensor-core kernel: the missing channels of a block arrive as zeros.  Bit exact like every int8 case."""
    n, h, w, c, k = shape
    got, ref = int8_case(ctx, n, h, w, c, k, (5e-5, 2e-4), activation="relu", with_z=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, n, h, w, c, k, None, int32_output=True)
    assert np.array_equal(got, ref)
    got, ref = int8_case(ctx, n, h, w, c, k, (5e-5, 2e-4), rotated=True)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 14, 14, 40, 64), (3, 10, 11, 72, 24), (2, 16, 16, 8, 16), (1, 20, 20, 200, 136)])
def test_implicit_gemm_16bit_partial_channel_blocks(ctx, dtype, shape):
    """16-bit layers whose channel count does not fill the kernel's 64-channel blocks (C = 40, 72, 8, 200): the filter map
    has the channels of one tap as its innermost dimension, so the columns past C arrive as zeros for filters and pixels
    alike and the layer stays on the tensor cores"""
    n, h, w, c, k = shape
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    d.implicit_gemm(activation="relu")
    ref = o.conv2d_forward(x, wt, bias=b, activation="relu")
    assert o.error_metrics(d.y.download(ctx), ref)["elem"] <= {"float16": 1.5e-3, "bfloat16": 1e-2}[dtype]
    assert ctx.last_device_status() == 0


@pytest.mark.parametrize("shape", [(4, 28, 28, 64, 64), (2, 9, 10, 24, 16), (3, 14, 15, 128, 72), (2, 8, 8, 16, 8)])
def test_implicit_gemm_float32_on_tensor_cores(ctx, shape):
    """float32 through cudaConvolutionImplicitGemmForward: lowered (im2row) onto the 3xTF32 tcgen05 GEMM, with the whole
    epilogue formula and with none; float32-level accuracy (1e-3 is the stated bound, the 3xTF32 scheme is well inside)"""
    n, h, w, c, k = shape
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "float32")
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    d.implicit_gemm()
    assert o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt))["elem"] <= 1e-4
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    z = d.set_z(common.uniform("z", d.y.shape))
    y0 = d.y.upload(ctx, common.uniform("y", d.y.shape))
    d.implicit_gemm(alpha1=1.1, alpha2=1.2, beta=0.1, activation="tanh")
    f = lambda v: float(np.float32(v))
    ref = o.conv2d_forward(x, wt, bias=b, z=z, y=y0, alpha1=f(1.1), alpha2=f(1.2), beta=f(0.1), activation="tanh")
    assert o.error_metrics(d.y.download(ctx), ref)["elem"] <= 1e-4


def test_implicit_gemm_float32_rotated_5x5_and_chunked(ctx):
    """CROSS_CORRELATION_MODE, a 5x5 kernel, and a batch large enough that the row matrix is built in several chunks"""
    n, h, w, c, k = 2, 12, 11, 16, 16
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "float32", kernel_size=5)
    d.conv = api.ConvolutionDescriptor(api.CROSS_CORRELATION_MODE, (-2, -2))
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 5, c))
    d.implicit_gemm(activation="relu")
    ref = o.conv2d_forward(x, wt, padding=(-2, -2), mode=1, activation="relu")
    assert o.error_metrics(d.y.download(ctx), ref)["elem"] <= 1e-4
    n, h, w, c, k = 24, 56, 56, 64, 32  # 24 * 3136 * 576 * 4 bytes = 1.7 GB of rows: two chunks
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "float32")
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    d.implicit_gemm()
    assert o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt))["elem"] <= 1e-4
