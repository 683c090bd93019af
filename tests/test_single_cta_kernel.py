"""The single-CTA (tcgen05 cta_group::1) implicit-GEMM kernel against the oracle.

Layers of at least 256 output pixels run on the CTA-pair kernel (cta_group::2), which is what every other test of the
implicit GEMM exercises; the single-CTA kernel then only sees layers of 129 to 255 pixels.  AVOCADO_B200_CONV=single
(read once when the library first dispatches a convolution) keeps every layer on it, so these cases run in a process of
their own with that variable set: a pixel count that is not a multiple of the 128-pixel tile, filter counts that end
inside a 256-filter block and 64- and 128-filter tiles, more tiles than CTAs, and the 16-bit floating path.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = r"""
import numpy as np
from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from tests import common
from tests.test_conv_pipeline import int8_case

api.load()
ctx = api.Context(0)
for shape in [(8, 14, 14, 256, 256), (16, 7, 9, 384, 272), (32, 28, 28, 128, 256), (8, 14, 14, 128, 64), (4, 9, 9, 64, 128)]:
    got, ref = int8_case(ctx, *shape, (5e-5, 2e-4), activation="relu", with_z=True)
    assert np.array_equal(got, ref), ("int8", shape)
    got, ref = int8_case(ctx, *shape, (1e-3, 1e-2))
    assert np.array_equal(got, ref), ("int8 saturating", shape)
    got, ref = int8_case(ctx, *shape, None, int32_output=True)
    assert np.array_equal(got, ref), ("int32", shape)
for dtype, bound in (("float16", 1.5e-3), ("bfloat16", 1e-2)):
    n, h, w, c, k = 2, 30, 31, 192, 320
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, dtype)
    x = d.x.upload(ctx, common.uniform("x", d.x.shape))
    wt = d.wt.upload(ctx, common.he_normal_weights(k, 3, c))
    b = d.set_bias(common.uniform("b", (k,), -0.1, 0.1))
    d.implicit_gemm(activation="relu")
    err = o.error_metrics(d.y.download(ctx), o.conv2d_forward(x, wt, bias=b, activation="relu"))["elem"]
    assert err <= bound, (dtype, err)
ctx.synchronize()
assert ctx.last_device_status() == 0
print("single-CTA kernel cases passed")
"""


def test_single_cta_kernel_matches_the_oracle(library, device_count):
    if device_count == 0:
        pytest.skip("no CUDA device visible")
    env = dict(os.environ, AVOCADO_B200_CONV="single")
    result = subprocess.run([sys.executable, "-c", CASES], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, (result.stdout[-1000:], result.stderr[-3000:])
    assert "single-CTA kernel cases passed" in result.stdout
