"""Runs the reference's own kernels (oracle/_ref/libref_winograd.so) on seeded inputs.  TEST INFRASTRUCTURE ONLY.

    python -m oracle.run_ref --out results.npz [--case NAME ...]
    python -m oracle.run_ref --int8-fixture tests/golden/reference_int8.npz      (writes the committed int8 fixture)

Runs in a process of its own: the comparator exports the same C symbol names as the product library, so the two are
never loaded together.  For every case the .npz holds the inputs (already rounded to the storage type) and every
tensor the reference produced: U, V, M, y and, for float32, the dW chain (G, Mw, dw).  The int8 cases hold the int32
accumulators of the reference's explicit lowering (cudaIm2Row + int8 cudaGemm): its quantised convolution without the
requantisation it never had.
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

# int8 cases: name -> (N, H, W, C, K, seed); "golden" takes x and w from tests/golden/int8_requant.npz instead
INT8_CASES = {
    "int8_golden": None,
    "int8_14x14_c64": (4, 14, 14, 64, 64, 31),
    "int8_ragged": (3, 9, 7, 32, 48, 32),
}
GOLDEN_INT8 = os.path.join(os.path.dirname(HERE), "tests", "golden", "int8_requant.npz")


def make_int8_inputs(name):
    if INT8_CASES[name] is None:
        golden = np.load(GOLDEN_INT8)
        return golden["x"], golden["w"]
    n, h, w, c, k, seed = INT8_CASES[name]
    r = np.random.default_rng(seed)
    return r.integers(-127, 128, (n, h, w, c), dtype=np.int8), r.integers(-127, 128, (k, 3, 3, c), dtype=np.int8)


def run_int8_case(lib, name):
    x, wt = make_int8_inputs(name)
    n, h, w, c = x.shape
    k = wt.shape[0]
    rows = np.zeros((n * h * w, 9 * c), np.int8)
    acc = np.zeros((n, h, w, k), np.int32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    status = lib.ref_im2row_gemm_int8(n, h, w, c, k, p(np.ascontiguousarray(x)), p(np.ascontiguousarray(wt)), p(rows), p(acc))
    if status != 0:
        raise RuntimeError("reference im2row + int8 gemm failed for %s with code %d" % (name, status))
    return {"x": x, "w": wt, "rows": rows, "acc": acc}


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
    parser.add_argument("--out", default=None)
    parser.add_argument("--case", action="append", default=None)
    parser.add_argument("--int8-fixture", default=None, help="write the reference's int32 accumulators of the golden int8 case to this file")
    args = parser.parse_args()
    if args.out is None and args.int8_fixture is None:
        parser.error("give --out and/or --int8-fixture")
    if not os.path.exists(LIB):
        print("comparator library not built: run python oracle/build_ref.py where the reference sources are mounted", file=sys.stderr)
        return 2
    lib = ctypes.CDLL(LIB)
    lib.ref_winograd_chain.restype = ctypes.c_int
    lib.ref_winograd_chain.argtypes = [ctypes.c_int] * 8 + [ctypes.c_void_p] * 11 + [ctypes.c_int]
    lib.ref_im2row_gemm_int8.restype = ctypes.c_int
    lib.ref_im2row_gemm_int8.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 4
    if args.int8_fixture is not None:
        result = run_int8_case(lib, "int8_golden")
        np.savez_compressed(args.int8_fixture, acc=result["acc"], rows=result["rows"])
    if args.out is None:
        return 0
    flat = {}
    for name in (args.case or (list(CASES) + list(INT8_CASES))):
        runner = run_int8_case if name in INT8_CASES else run_case
        for key, value in runner(lib, name).items():
            flat[name + "/" + key] = value
    np.savez_compressed(args.out, **flat)
    return 0


if __name__ == "__main__":
    sys.exit(main())
