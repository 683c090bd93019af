"""CPU tests of the oracle itself (no GPU): the Winograd transforms, chained with an exact contraction, must
reproduce the direct convolution and its exact gradients for every tile configuration of the reference
(src/winograd_nonfused.cu:532-582), and the committed golden vectors must be reproduced bit for bit."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as o

CONFIGS = [(2, 3), (4, 3), (2, 5)]
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("ts,ks", CONFIGS)
@pytest.mark.parametrize("mode", [0, 1])
def test_forward_identity(ts, ks, mode):
    r = np.random.default_rng(ts * 10 + ks + mode)
    n, h, w, c, k = 2, 13, 14, 5, 7
    pad = -(ks // 2)
    x = r.uniform(-1, 1, (n, h, w, c))
    wt = r.normal(size=(k, ks, ks, c))
    ref = o.conv2d_forward(x, wt, padding=(pad, pad), mode=mode)
    u = o.winograd_weight_transform(wt, ts, invert=(mode == 1))
    v = o.winograd_input_transform(x, ts, ks, padding=(pad, pad))
    m = o.gemm_batched(v, u, trans_b=True)
    y = o.winograd_output_transform(m, (n, h, w, k), ts, ks)
    assert np.abs(y - ref).max() < 1e-12


@pytest.mark.parametrize("ts,ks", CONFIGS)
def test_weight_gradient_identity(ts, ks):
    r = np.random.default_rng(100 + ts * 10 + ks)
    n, h, w, c, k = 2, 13, 14, 5, 7
    pad = -(ks // 2)
    x = r.uniform(-1, 1, (n, h, w, c))
    dy = r.uniform(-1, 1, (n, h, w, k))
    ref = o.conv2d_backward_weights(x, dy, (ks, ks), (pad, pad))
    g = o.winograd_gradient_transform(dy, ts, ks)
    v = o.winograd_input_transform(x, ts, ks, padding=(pad, pad))
    mw = o.gemm_batched(g, v, trans_a=True)
    dw = o.winograd_update_transform(mw, ts, ks)
    assert np.abs(dw - ref).max() < 1e-11


@pytest.mark.parametrize("ts,ks", CONFIGS)
def test_data_gradient_identity(ts, ks):
    r = np.random.default_rng(200 + ts * 10 + ks)
    n, h, w, c, k = 2, 9, 10, 5, 7
    pad = -(ks // 2)
    wt = r.normal(size=(k, ks, ks, c))
    dy = r.uniform(-1, 1, (n, h, w, k))
    ref = o.conv2d_backward_data(dy, wt, (h, w), (pad, pad))
    u = o.winograd_weight_transform(wt, ts, invert=True)
    v = o.winograd_input_transform(dy, ts, ks, padding=(pad, pad))
    m = o.gemm_batched(v, u)
    dx = o.winograd_output_transform(m, (n, h, w, c), ts, ks)
    assert np.abs(dx - ref).max() < 1e-12


def test_backward_are_adjoints():
    """<conv(x, w), dy> = <x, dX(dy, w)> = <w, dW(x, dy)>"""
    r = np.random.default_rng(5)
    n, h, w, c, k = 2, 7, 6, 3, 4
    x = r.normal(size=(n, h, w, c))
    wt = r.normal(size=(k, 3, 3, c))
    dy = r.normal(size=(n, h, w, k))
    lhs = np.sum(o.conv2d_forward(x, wt) * dy)
    assert abs(lhs - np.sum(x * o.conv2d_backward_data(dy, wt, (h, w)))) < 1e-9
    assert abs(lhs - np.sum(wt * o.conv2d_backward_weights(x, dy))) < 1e-9


def test_epilogue_order():
    r = np.random.default_rng(6)
    x = r.normal(size=(1, 5, 5, 2))
    wt = r.normal(size=(3, 3, 3, 2))
    b = r.normal(size=3)
    z = r.normal(size=(1, 5, 5, 3))
    y0 = r.normal(size=(1, 5, 5, 3))
    conv = o.conv2d_forward(x, wt)
    got = o.conv2d_forward(x, wt, bias=b, z=z, y=y0, alpha1=1.1, alpha2=1.2, beta=0.1, activation="relu")
    expect = np.maximum(1.1 * conv + b + 1.2 * z, 0.0) + 0.1 * y0
    assert np.abs(got - expect).max() < 1e-13


def test_int8_requantisation_rule():
    r = np.random.default_rng(7)
    x = r.integers(-127, 128, (2, 6, 6, 16), dtype=np.int8)
    wt = r.integers(-127, 128, (8, 3, 3, 16), dtype=np.int8)
    b = r.integers(-1000, 1001, 8, dtype=np.int32)
    s = r.uniform(5e-5, 2e-4, 8).astype(np.float32)
    acc = o.conv2d_forward_int8(x, wt, b, int32_output=True)
    exact = o.conv2d_forward(x.astype(np.float64), wt.astype(np.float64), bias=b.astype(np.float64))
    assert np.array_equal(acc.astype(np.int64), np.rint(exact).astype(np.int64))
    q = o.conv2d_forward_int8(x, wt, b, s)
    expect = np.clip(np.rint((acc.astype(np.float32) * s).astype(np.float32)), -128, 127).astype(np.int8)
    assert np.array_equal(q, expect)


def test_int8_ties_round_to_even_and_saturate():
    # one input pixel, one channel: acc = x*w, so that r = acc * 0.5 hits exact .5 ties
    x = np.zeros((1, 1, 1, 4), dtype=np.int8)
    x[0, 0, 0, 0] = 1
    wt = np.zeros((6, 3, 3, 4), dtype=np.int8)
    values = [1, 3, 5, -1, -3, 127]
    for k, v in enumerate(values):
        wt[k, 1, 1, 0] = v
    s = np.full(6, 0.5, dtype=np.float32)
    q = o.conv2d_forward_int8(x, wt, None, s)
    assert q.reshape(-1).tolist() == [0, 2, 2, 0, -2, 64]
    big = o.conv2d_forward_int8(x, wt, np.full(6, 100000, dtype=np.int32), s)
    assert big.reshape(-1).tolist() == [127] * 6
    small = o.conv2d_forward_int8(x, wt, np.full(6, -100000, dtype=np.int32), s)
    assert small.reshape(-1).tolist() == [-128] * 6


def test_golden_vectors():
    """The fixtures under tests/golden were written by tests/golden/make_golden.py from this oracle; they pin it
    against silent changes and are what the GPU tests compare with at the small sizes."""
    index = os.path.join(GOLDEN, "index.json")
    if not os.path.exists(index):
        pytest.skip("golden fixtures not generated yet")
    from tests.golden import make_golden
    for case in json.load(open(index)):
        data = np.load(os.path.join(GOLDEN, case["file"]))
        fresh = make_golden.compute(case)
        for key in fresh:
            assert np.array_equal(np.asarray(fresh[key]), data[key]), (case["name"], key)


def test_oracle_matches_reference_kernel_outputs():
    """tests/golden/reference_small.npz holds what the REFERENCE's own kernels (src/winograd_nonfused.cu compiled
    unmodified into oracle/_ref, plus its cuBLAS GEMM wrapper) produced on a B200 for the seeded cases of
    oracle/run_ref.py.  The oracle must reproduce every tensor of the forward and dW chains to the rounding of the
    storage type; this is the pin of the oracle against the reference."""
    from oracle import run_ref
    data = np.load(os.path.join(GOLDEN, "reference_small.npz"))
    rel = lambda a, b: np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    for name in run_ref.SMALL:
        dtype, ts, ks, n, h, w, c, k, _ = run_ref.CASES[name]
        g = lambda key: data[name + "/" + key].astype(np.float64)
        x_expected, w_expected, _, _ = run_ref.make_inputs(name)
        assert np.array_equal(data[name + "/x"], x_expected) and np.array_equal(data[name + "/w"], w_expected)
        pad = -(ks // 2)
        eps = 2.0 ** -23 if dtype == "float32" else 2.0 ** -10
        u = o.winograd_weight_transform(g("w"), ts)
        v = o.winograd_input_transform(g("x"), ts, ks, padding=(pad, pad))
        m = o.gemm_batched(v, u, trans_b=True)
        assert rel(g("u"), u) <= 2 * eps, name
        assert rel(g("v"), v) <= 2 * eps, name
        assert rel(g("m"), m) <= 4 * eps, name
        y = o.conv2d_forward(g("x"), g("w"), bias=g("bias"), padding=(pad, pad), activation="relu")
        # the reference keeps fp16 matrices and fp16 arithmetic: F(4x4,3x3) in fp16 is only good to a few 1e-2
        assert o.error_metrics(g("y"), y)["elem"] <= (1e-4 if dtype == "float32" else 6e-2), name
        if dtype == "float32":
            gr = o.winograd_gradient_transform(g("dy"), ts, ks)
            mw = o.gemm_batched(gr, v, trans_a=True)
            assert rel(g("g"), gr) <= 2 * eps, name
            assert rel(g("mw"), mw) <= 8 * eps, name
            dw = o.conv2d_backward_weights(g("x"), g("dy"), (ks, ks), (pad, pad))
            assert o.error_metrics(g("dw"), dw)["elem"] <= 1e-4, name


def test_oracle_int8_accumulators_match_the_reference():
    """tests/golden/reference_int8.npz holds what the REFERENCE's own quantised path produced on a B200 for the inputs of
    tests/golden/int8_requant.npz: its cudaIm2Row (src/im2row.cu:83-121) followed by its int8 -> int32 cudaGemm
    (src/gemm.cpp:42-57), both compiled unmodified into oracle/_ref and driven by oracle/run_ref.py --int8-fixture.
    The reference has no requantisation, so its int32 accumulators are as far as it can pin the int8 path: the
    oracle's exact integer convolution, its im2row and the accumulators stored in the golden file must equal them
    bit for bit."""
    golden = np.load(os.path.join(GOLDEN, "int8_requant.npz"))
    reference = np.load(os.path.join(GOLDEN, "reference_int8.npz"))
    n, h, w, c = golden["x"].shape
    assert np.array_equal(o.conv2d_forward_int8(golden["x"], golden["w"], None, int32_output=True), reference["acc"])
    assert np.array_equal(golden["acc"] - golden["bias"][None, None, None, :], reference["acc"])
    assert np.array_equal(o.im2row(golden["x"], (3, 3), (-1, -1)).reshape(n * h * w, 9 * c), reference["rows"])
