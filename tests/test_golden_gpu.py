"""GPU parity against the committed golden vectors (tests/golden/, written by make_golden.py from the oracle):
every stage of the Winograd pipeline at the fixture sizes, in float64 and float32, and the int8 convolution bit for bit."""
import json
import os

import numpy as np
import pytest

from cudabackend_b200 import api, pipeline

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = json.load(open(os.path.join(GOLDEN, "index.json")))


@pytest.mark.parametrize("case", [c for c in CASES if c["kind"] == "winograd"], ids=lambda c: c["name"])
@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_winograd_stages_match_golden(ctx, case, dtype):
    gold = np.load(os.path.join(GOLDEN, case["file"]))
    n, h, w, c = case["shape"]
    k, ts, ks = case["filters"], case["ts"], case["ks"]
    p = pipeline.WinogradNonFused(ctx, n, h, w, c, k, dtype, None, ts, ks, training=True)
    tol = 1e-12 if dtype == "float64" else 2e-5
    p.x.upload(ctx, gold["x"])
    p.wt.upload(ctx, gold["w"])
    p.dy.upload(ctx, gold["dy"])
    p.set_bias(gold["bias"])
    p.weight_transform()
    p.input_transform()
    assert np.abs(p.u.download(ctx) - gold["u"]).max() <= tol * max(1.0, np.abs(gold["u"]).max())
    assert np.abs(p.v.download(ctx) - gold["v"]).max() <= tol * max(1.0, np.abs(gold["v"]).max())
    p.gemm(p.v, p.u, p.m, False, True)
    assert np.abs(p.m.download(ctx) - gold["m"]).max() <= tol * max(1.0, np.abs(gold["m"]).max())
    p.output_transform(activation="relu")
    y = p.y.download(ctx)
    assert np.abs(y - gold["y"]).max() <= tol * max(1.0, np.abs(gold["y"]).max()) * 10
    assert np.abs(y - gold["y_direct"]).max() <= tol * max(1.0, np.abs(gold["y_direct"]).max()) * 10
    p.gradient_transform()
    assert np.abs(p.g.download(ctx) - gold["g"]).max() <= tol * max(1.0, np.abs(gold["g"]).max())
    p.gemm(p.g, p.v, p.mw, True, False)
    p.update_transform()
    dw = p.dw.download(ctx)
    assert np.abs(dw - gold["dw_direct"]).max() <= tol * max(1.0, np.abs(gold["dw_direct"]).max()) * 10


def test_int8_matches_golden(ctx):
    case = [c for c in CASES if c["kind"] == "int8"][0]
    gold = np.load(os.path.join(GOLDEN, case["file"]))
    n, h, w, c = case["shape"]
    k = case["filters"]
    d = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8")
    d.x.upload(ctx, gold["x"])
    d.wt.upload(ctx, gold["w"])
    d.set_bias(gold["bias"])
    d.set_scales(gold["scales"])
    d.set_z(gold["z"])
    d.implicit_gemm(alpha2=0.5, activation="relu")
    assert np.array_equal(d.y.download_raw(ctx), gold["y"])
    d32 = pipeline.DirectConvolution(ctx, n, h, w, c, k, "int8", out_dtype="int32")
    d32.x.upload(ctx, gold["x"])
    d32.wt.upload(ctx, gold["w"])
    d32.set_bias(gold["bias"])
    d32.implicit_gemm()
    assert np.array_equal(d32.y.download_raw(ctx), gold["acc"])
