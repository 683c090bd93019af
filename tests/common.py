"""Shared helpers of the parity tests: seeded inputs with the distributions of the benchmark configurations."""
import numpy as np

SEEDS = {"x": 0x1001, "w": 0x1002, "b": 0x1003, "dy": 0x1004, "scales": 0x1005, "z": 0x1006, "y": 0x1007}

# max |err| / max(|ref|, rms(ref)) allowed against the float64 oracle
TOLERANCE = {"float64": 1e-10, "float32": 1e-3, "float16": 1e-2, "bfloat16": 1e-2}
# storage rounding of one value (used where a kernel's only error is the final rounding)
EPS = {"float64": 2.0 ** -52, "float32": 2.0 ** -23, "float16": 2.0 ** -10, "bfloat16": 2.0 ** -7}


def rng(name, extra=0):
    return np.random.default_rng(SEEDS[name] + 7919 * extra)


def uniform(name, shape, lo=-1.0, hi=1.0, extra=0):
    return rng(name, extra).uniform(lo, hi, size=shape)


def he_normal_weights(k, ks, c, extra=0):
    """He-normal filters, std = sqrt(2 / (ks*ks*C))."""
    return rng("w", extra).normal(0.0, np.sqrt(2.0 / (ks * ks * c)), size=(k, ks, ks, c))


def int8_uniform(name, shape, extra=0):
    return rng(name, extra).integers(-127, 128, size=shape, dtype=np.int8)
