"""GPU tests against the reference's own kernels, run live.

oracle/_ref/libref_winograd.so is the reference's src/winograd_nonfused.cu, src/gemm.cpp and src/im2row.cu compiled unmodified (as
compute_75 PTX, JIT-compiled on the B200) with oracle/build_ref.py.  It is run in a process of its own by
oracle/run_ref.py.  Two claims are checked on the same seeded inputs:
  1. the CPU oracle reproduces the reference's transforms (this pins the oracle);
  2. this library's result is no further from the exact float64 convolution than the reference's;
  3. the int32 accumulators of the reference's own quantised path (cudaIm2Row + int8 cudaGemm) equal the oracle's and
     this library's bit for bit (the reference has no requantisation, so this is as far as it can pin the int8 path).
The library is built where the reference sources are mounted; on a machine without it the test reports a skip.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from cudabackend_b200 import api, pipeline
from oracle import oracle as o
from oracle import run_ref

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def reference_outputs(tmp_path_factory):
    if not os.path.exists(run_ref.LIB):
        pytest.skip("reference comparator not built (oracle/build_ref.py needs the reference sources)")
    out = str(tmp_path_factory.mktemp("ref") / "ref.npz")
    result = subprocess.run([sys.executable, "-m", "oracle.run_ref", "--out", out], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    return np.load(out)


@pytest.mark.parametrize("name", list(run_ref.CASES))
def test_library_is_no_worse_than_the_reference(ctx, reference_outputs, name):
    dtype, ts, ks, n, h, w, c, k, _ = run_ref.CASES[name]
    g = lambda key: reference_outputs[name + "/" + key].astype(np.float64)
    pad = -(ks // 2)
    eps = 2.0 ** -23 if dtype == "float32" else 2.0 ** -10
    rel = lambda a, b: np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)

    # 1. oracle == reference, transform by transform
    u = o.winograd_weight_transform(g("w"), ts)
    v = o.winograd_input_transform(g("x"), ts, ks, padding=(pad, pad))
    assert rel(g("u"), u) <= 2 * eps and rel(g("v"), v) <= 2 * eps
    exact = o.conv2d_forward(g("x"), g("w"), bias=g("bias"), padding=(pad, pad), activation="relu")
    reference_error = o.error_metrics(g("y"), exact)

    # 2. this library on the same inputs
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, None, ts, ks, training=(dtype == "float32"))
    p.x.upload(ctx, g("x"))
    p.wt.upload(ctx, g("w"))
    p.set_bias(g("bias"))
    p.forward(activation="relu")
    ours = p.y.download(ctx)
    our_error = o.error_metrics(ours, exact)
    # "no worse": within the float32 noise floor both are a few roundings from exact, so a floor applies there
    floor = 2e-5 if dtype == "float32" else 2e-3
    assert our_error["elem"] <= max(1.05 * reference_error["elem"], floor), (our_error, reference_error)
    assert rel(p.u.download(ctx), g("u")) <= 4 * eps and rel(p.v.download(ctx), g("v")) <= 4 * eps
    if dtype == "float32":
        p.dy.upload(ctx, g("dy"))
        p.backward_weights()
        exact_dw = o.conv2d_backward_weights(g("x"), g("dy"), (ks, ks), (pad, pad))
        assert o.error_metrics(p.dw.download(ctx), exact_dw)["elem"] <= max(1.05 * o.error_metrics(g("dw"), exact_dw)["elem"], 2e-5)


@pytest.mark.parametrize("name", list(run_ref.INT8_CASES))
def test_int8_accumulators_equal_the_reference(ctx, reference_outputs, name):
    x = reference_outputs[name + "/x"]
    wt = reference_outputs[name + "/w"]
    reference_acc = reference_outputs[name + "/acc"]
    n, h, w, c = x.shape
    k = wt.shape[0]
    # the oracle's exact integer convolution (no bias, int32 out) against the reference's lowering + cuBLAS product
    assert np.array_equal(o.conv2d_forward_int8(x, wt, None, int32_output=True), reference_acc)
    # the oracle's im2row against the reference's row matrix
    assert np.array_equal(o.im2row(x, (3, 3), (-1, -1)).reshape(n * h * w, 9 * c), reference_outputs[name + "/rows"])
    # this library, int32 output: the raw accumulators of the implicit-GEMM entry point
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8", out_dtype="int32")
    d.x.upload(ctx, x)
    d.wt.upload(ctx, wt)
    d.implicit_gemm()
    assert np.array_equal(d.y.download_raw(ctx), reference_acc)
