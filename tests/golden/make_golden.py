"""Writes the golden vectors under tests/golden/ from the CPU oracle.

Run from the repository root:  python -m tests.golden.make_golden
Each case is a small seeded problem; the .npz holds its inputs and every intermediate of the Winograd pipeline
(U, V, M, y, dW ...) in float64, or the int8 convolution with its requantised output.  tests/test_oracle.py checks
that the oracle still reproduces them bit for bit; the GPU tests compare the library against them.
"""
import json
import os

import numpy as np

from oracle import oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    {"name": "f23_forward", "kind": "winograd", "ts": 2, "ks": 3, "shape": [2, 5, 6, 4], "filters": 3, "seed": 11},
    {"name": "f43_forward", "kind": "winograd", "ts": 4, "ks": 3, "shape": [2, 7, 9, 4], "filters": 3, "seed": 12},
    {"name": "f25_forward", "kind": "winograd", "ts": 2, "ks": 5, "shape": [1, 6, 5, 4], "filters": 2, "seed": 13},
    {"name": "int8_requant", "kind": "int8", "shape": [2, 5, 6, 16], "filters": 16, "seed": 14},
]


def compute(case):
    r = np.random.default_rng(case["seed"])
    n, h, w, c = case["shape"]
    k = case["filters"]
    if case["kind"] == "int8":
        x = r.integers(-127, 128, (n, h, w, c), dtype=np.int8)
        wt = r.integers(-127, 128, (k, 3, 3, c), dtype=np.int8)
        bias = r.integers(-1000, 1001, k, dtype=np.int32)
        scales = r.uniform(5e-4, 2e-3, k).astype(np.float32)
        z = r.integers(-127, 128, (n, h, w, k), dtype=np.int8)
        return {"x": x, "w": wt, "bias": bias, "scales": scales, "z": z,
                "acc": o.conv2d_forward_int8(x, wt, bias, int32_output=True),
                "y": o.conv2d_forward_int8(x, wt, bias, scales, z, alpha2=0.5, activation="relu")}
    ts, ks = case["ts"], case["ks"]
    pad = -(ks // 2)
    # values on a coarse binary grid: every transform is then exact in float32 as well, so the same file pins
    # float32 and float64 kernels without a tolerance on the transforms
    x = np.round(r.uniform(-1, 1, (n, h, w, c)) * 64) / 64
    wt = np.round(r.normal(0, 0.5, (k, ks, ks, c)) * 64) / 64
    dy = np.round(r.uniform(-1, 1, (n, h, w, k)) * 64) / 64
    bias = np.round(r.uniform(-1, 1, k) * 64) / 64
    u = o.winograd_weight_transform(wt, ts)
    v = o.winograd_input_transform(x, ts, ks, padding=(pad, pad))
    m = o.gemm_batched(v, u, trans_b=True)
    y = o.winograd_output_transform(m, (n, h, w, k), ts, ks, bias=bias, activation="relu")
    g = o.winograd_gradient_transform(dy, ts, ks)
    mw = o.gemm_batched(g, v, trans_a=True)
    dw = o.winograd_update_transform(mw, ts, ks)
    return {"x": x, "w": wt, "dy": dy, "bias": bias, "u": u, "v": v, "m": m, "y": y, "g": g, "mw": mw, "dw": dw,
            "y_direct": o.conv2d_forward(x, wt, bias=bias, padding=(pad, pad), activation="relu"),
            "dw_direct": o.conv2d_backward_weights(x, dy, (ks, ks), (pad, pad))}


def main():
    index = []
    for case in CASES:
        data = compute(case)
        name = case["name"] + ".npz"
        np.savez_compressed(os.path.join(HERE, name), **data)
        index.append(dict(case, file=name))
    with open(os.path.join(HERE, "index.json"), "w") as f:
        json.dump(index, f, indent=1)
    print("wrote", len(index), "cases")


if __name__ == "__main__":
    main()
