"""Runs the reference's own Winograd kernels (oracle/_ref/libref_winograd.so) on seeded inputs.  TEST INFRASTRUCTURE ONLY.

    python -m oracle.run_ref --out results.npz [--case NAME ...]

Runs in a process of its own: the comparator exports the same C symbol names as the product library, so the two are
never loaded together.  For every case the .npz holds the inputs (already rounded to the storage type) and every
tensor the reference produced: U, V, M, y and, for float32, the dW chain (G, Mw, dw).
"""
import argparse
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libref_winograd.so")
FLOAT16, FLOAT32 = 6, 8  # avDataType_t values of include/Avocado/backend_defs.h

# name: (dtype, transform size, kernel size, N, H, W, C, K, seed)
CASES = {
    "cfg1_f43_fp32": ("float32", 4, 3, 2, 16, 16, 32, 32, 21),
    "small_f43_fp32": ("float32", 4, 3, 2, 7, 9, 6, 4, 22),
    "small_f23_fp32": ("float32", 2, 3, 2, 5, 6, 6, 4, 23),
    "small_f25_fp32": ("float32", 2, 5, 1, 6, 5, 6, 4, 24),
    "small_f43_fp16": ("float16", 4, 3, 2, 7, 9, 8, 4, 25),
    "small_f23_fp16": ("float16", 2, 3, 2, 5, 6, 8, 4, 26),
    "refshape_f43_fp32": ("float32", 4, 3, 12, 13, 14, 135, 21, 27),
}
SMALL = [name for name in CASES if name.startswith("small_")]


def make_inputs(name):
    dtype, ts, ks, n, h, w, c, k, seed = CASES[name]
    r = np.random.default_rng(seed)
    np_dtype = np.float32 if dtype == "float32" else np.float16
    x = r.uniform(-1, 1, (n, h, w, c)).astype(np_dtype)
    wt = r.normal(0, np.sqrt(2.0 / (ks * ks * c)), (k, ks, ks, c)).astype(np_dtype)
    bias = r.uniform(-0.1, 0.1, k).astype(np.float32)
    dy = r.uniform(-1, 1, (n, h, w, k)).astype(np_dtype)
    return x, wt, bias, dy


def run_case(lib, name):
    dtype, ts, ks, n, h, w, c, k, _ = CASES[name]
    x, wt, bias, dy = make_inputs(name)
    np_dtype = x.dtype
    tile = ts + ks - 1
    planes = tile * tile
    tiles = n * ((h + ts - 1) // ts) * ((w + ts - 1) // ts)
    out = {"u": np.zeros((planes, k, c), np_dtype), "v": np.zeros((planes, tiles, c), np_dtype), "m": np.zeros((planes, tiles, k), np_dtype),
           "y": np.zeros((n, h, w, k), np_dtype), "g": np.zeros((planes, tiles, k), np_dtype), "mw": np.zeros((planes, k, c), np_dtype),
           "dw": np.zeros((k, ks, ks, c), np_dtype)}
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    status = lib.ref_winograd_chain(FLOAT32 if dtype == "float32" else FLOAT16, ts, ks, n, h, w, c, k, p(x), p(wt), p(bias), p(dy), p(out["u"]),
                                    p(out["v"]), p(out["m"]), p(out["y"]), p(out["g"]), p(out["mw"]), p(out["dw"]), 1)
    if status != 0:
        raise RuntimeError("reference chain failed for %s with code %d" % (name, status))
    result = {"x": x, "w": wt, "bias": bias, "dy": dy}
    result.update(out)
    return result


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--out", required=True)
    parser.add_argument("--case", action="append", default=None)
    args = parser.parse_args()
    if not os.path.exists(LIB):
        print("comparator library not built: run python oracle/build_ref.py where the reference sources are mounted", file=sys.stderr)
        return 2
    lib = ctypes.CDLL(LIB)
    lib.ref_winograd_chain.restype = ctypes.c_int
    lib.ref_winograd_chain.argtypes = [ctypes.c_int] * 8 + [ctypes.c_void_p] * 11 + [ctypes.c_int]
    flat = {}
    for name in (args.case or list(CASES)):
        for key, value in run_case(lib, name).items():
            flat[name + "/" + key] = value
    np.savez_compressed(args.out, **flat)
    return 0


if __name__ == "__main__":
    sys.exit(main())
