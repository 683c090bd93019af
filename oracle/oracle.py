"""numpy front end of the CPU oracle (oracle/conv_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py (its cpu_baseline / reference arm, and the comparison of a timed
step's output with this oracle outside the timed region) may import this module; the product (cudabackend_b200) never does.  Every function takes and returns numpy arrays in the layouts of the
reference: activations NHWC, filters [K, kh, kw, C], transform-domain matrices [tile*tile, nbTiles, channels].
"""
import ctypes
import os

import numpy as np

from . import build as _build

ACTIVATIONS = {"linear": 0, "sigmoid": 1, "tanh": 2, "relu": 3, "selu": 4, "elu": 5, "exponential": 6, "softplus": 7, "softsign": 8}

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB
        if os.path.exists(os.path.join(_build.HERE, "conv_oracle.c")) and _have_gcc():
            path = _build.build()
        _lib = ctypes.CDLL(path)
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def _have_gcc():
    import shutil
    return shutil.which("gcc") is not None


def max_threads():
    return int(lib().oracle_max_threads())


def use_all_host_threads():
    """Lets the OpenMP loops use every core the process may run on, whatever OMP_NUM_THREADS a launcher exported."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(int(cores))
    return max_threads()


def _p(a, ctype):
    if a is None:
        return ctypes.POINTER(ctype)()
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _f64(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float64)


def _act(activation):
    return ACTIVATIONS[activation] if isinstance(activation, str) else int(activation)


def conv2d_forward(x, w, bias=None, z=None, y=None, padding=(-1, -1), mode=0, padding_value=0.0, alpha1=1.0, alpha2=1.0, beta=0.0,
                   activation="linear", out_hw=None):
    """float64 direct convolution with the reference's epilogue; returns y[N,Ho,Wo,K]."""
    x, w, bias, z = _f64(x), _f64(w), _f64(bias), _f64(z)
    N, H, W, C = x.shape
    K, kh, kw, _ = w.shape
    Ho, Wo = out_hw if out_hw is not None else (H, W)
    out = np.zeros((N, Ho, Wo, K), dtype=np.float64) if y is None else np.array(y, dtype=np.float64, order="C")
    d = ctypes.c_double
    lib().oracle_conv2d_forward_f64(_p(x, d), _p(w, d), _p(bias, d), _p(z, d), _p(out, d), N, H, W, C, Ho, Wo, K, kh, kw, int(padding[0]),
                                    int(padding[1]), int(mode), d(padding_value), d(alpha1), d(alpha2), d(beta), _act(activation))
    return out


def conv2d_backward_data(dy, w, x_hw, padding=(-1, -1)):
    dy, w = _f64(dy), _f64(w)
    N, Ho, Wo, K = dy.shape
    _, kh, kw, C = w.shape
    H, W = x_hw
    dx = np.zeros((N, H, W, C), dtype=np.float64)
    d = ctypes.c_double
    lib().oracle_conv2d_backward_data_f64(_p(dy, d), _p(w, d), _p(dx, d), N, H, W, C, Ho, Wo, K, kh, kw, int(padding[0]), int(padding[1]))
    return dx


def conv2d_backward_weights(x, dy, kernel=(3, 3), padding=(-1, -1)):
    x, dy = _f64(x), _f64(dy)
    N, H, W, C = x.shape
    _, Ho, Wo, K = dy.shape
    kh, kw = kernel
    dw = np.zeros((K, kh, kw, C), dtype=np.float64)
    d = ctypes.c_double
    lib().oracle_conv2d_backward_weights_f64(_p(x, d), _p(dy, d), _p(dw, d), N, H, W, C, Ho, Wo, K, kh, kw, int(padding[0]), int(padding[1]))
    return dw


def conv2d_forward_f32_naive(x, w, bias=None, padding=(-1, -1), relu=False):
    """The float32 naive convolution used as the timed CPU baseline (not the correctness oracle)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    N, H, W, C = x.shape
    K, kh, kw, _ = w.shape
    y = np.empty((N, H, W, K), dtype=np.float32)
    f = ctypes.c_float
    lib().oracle_conv2d_forward_f32_naive(_p(x, f), _p(w, f), _p(bias, f), _p(y, f), N, H, W, C, K, kh, kw, int(padding[0]), int(padding[1]), int(relu))
    return y


def conv2d_forward_int8(x, w, bias=None, scale=None, z=None, padding=(-1, -1), alpha1=1.0, alpha2=1.0, activation="linear", int32_output=False):
    """Exact int8 convolution; returns int8 (requantised) or int32 (raw accumulator + bias)."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.int32)
    scale = None if scale is None else np.ascontiguousarray(scale, dtype=np.float32)
    z = None if z is None else np.ascontiguousarray(z, dtype=np.int8)
    N, H, W, C = x.shape
    K, kh, kw, _ = w.shape
    y8 = None if int32_output else np.empty((N, H, W, K), dtype=np.int8)
    y32 = np.empty((N, H, W, K), dtype=np.int32) if int32_output else None
    lib().oracle_conv2d_forward_int8(_p(x, ctypes.c_int8), _p(w, ctypes.c_int8), _p(bias, ctypes.c_int32), _p(scale, ctypes.c_float),
                                     _p(z, ctypes.c_int8), _p(y8, ctypes.c_int8), _p(y32, ctypes.c_int32), N, H, W, C, K, kh, kw, int(padding[0]),
                                     int(padding[1]), ctypes.c_float(alpha1), ctypes.c_float(alpha2), _act(activation))
    return y32 if int32_output else y8


TABLE_KINDS = {"weight": 0, "input": 1, "output": 2, "gradient": 3, "update": 4}


def winograd_table(transform_size, kernel_size, kind):
    buf = np.zeros(64, dtype=np.float64)
    rows, cols = ctypes.c_int(0), ctypes.c_int(0)
    n = lib().oracle_winograd_table(transform_size, kernel_size, TABLE_KINDS[kind], _p(buf, ctypes.c_double), ctypes.byref(rows), ctypes.byref(cols))
    if n == 0:
        raise ValueError("unsupported Winograd configuration")
    return buf[:n].reshape(rows.value, cols.value).copy()


def nb_tiles(N, H, W, transform_size):
    return N * ((H + transform_size - 1) // transform_size) * ((W + transform_size - 1) // transform_size)


def winograd_weight_transform(w, transform_size, invert=False):
    w = _f64(w)
    K, ks, _, C = w.shape
    tile = transform_size + ks - 1
    out = np.zeros((tile * tile, K, C), dtype=np.float64)
    d = ctypes.c_double
    if lib().oracle_winograd_weight_transform_f64(_p(w, d), _p(out, d), K, C, transform_size, ks, int(invert)) != 0:
        raise ValueError("unsupported Winograd configuration")
    return out


def winograd_input_transform(x, transform_size, kernel_size, padding=(-1, -1), padding_value=0.0):
    x = _f64(x)
    N, H, W, C = x.shape
    tile = transform_size + kernel_size - 1
    out = np.zeros((tile * tile, nb_tiles(N, H, W, transform_size), C), dtype=np.float64)
    d = ctypes.c_double
    if lib().oracle_winograd_input_transform_f64(_p(x, d), _p(out, d), N, H, W, C, transform_size, kernel_size, int(padding[0]), int(padding[1]),
                                                 d(padding_value)) != 0:
        raise ValueError("unsupported Winograd configuration")
    return out


def winograd_output_transform(matrices, shape, transform_size, kernel_size, bias=None, z=None, y=None, alpha1=1.0, alpha2=1.0, beta=0.0,
                              activation="linear"):
    matrices, bias, z = _f64(matrices), _f64(bias), _f64(z)
    N, H, W, K = shape
    out = np.zeros(shape, dtype=np.float64) if y is None else np.array(y, dtype=np.float64, order="C")
    d = ctypes.c_double
    if lib().oracle_winograd_output_transform_f64(_p(matrices, d), _p(out, d), _p(bias, d), _p(z, d), N, H, W, K, transform_size, kernel_size,
                                                  d(alpha1), d(alpha2), d(beta), _act(activation)) != 0:
        raise ValueError("unsupported Winograd configuration")
    return out


def winograd_gradient_transform(dy, transform_size, kernel_size):
    dy = _f64(dy)
    N, H, W, K = dy.shape
    tile = transform_size + kernel_size - 1
    out = np.zeros((tile * tile, nb_tiles(N, H, W, transform_size), K), dtype=np.float64)
    d = ctypes.c_double
    if lib().oracle_winograd_gradient_transform_f64(_p(dy, d), _p(out, d), N, H, W, K, transform_size, kernel_size) != 0:
        raise ValueError("unsupported Winograd configuration")
    return out


def winograd_update_transform(matrices, transform_size, kernel_size, dw=None, alpha=1.0, beta=0.0):
    matrices = _f64(matrices)
    _, K, C = matrices.shape
    out = np.zeros((K, kernel_size, kernel_size, C), dtype=np.float64) if dw is None else np.array(dw, dtype=np.float64, order="C")
    d = ctypes.c_double
    if lib().oracle_winograd_update_transform_f64(_p(matrices, d), _p(out, d), K, C, transform_size, kernel_size, d(alpha), d(beta)) != 0:
        raise ValueError("unsupported Winograd configuration")
    return out


def activation(x, name):
    """The nine activations of the reference (src/activations.cuh:202-425) in float64 numpy; same formulas as the C oracle."""
    x = np.asarray(x, dtype=np.float64)
    if name == "linear":
        return x
    if name == "sigmoid":
        return 1.0 / (1.0 + np.exp(-x))
    if name == "tanh":
        return np.tanh(x)
    if name == "relu":
        return np.maximum(x, 0.0)
    if name == "selu":
        return np.where(x >= 0, float(np.float32(1.05070098)) * x, float(np.float32(1.05070098)) * float(np.float32(1.67326324)) * np.expm1(x))
    if name == "elu":
        return np.where(x >= 0, x, np.expm1(x))
    if name == "exponential":
        return np.exp(x)
    if name == "softplus":
        return np.log1p(np.exp(x))
    if name == "softsign":
        return x / (np.abs(x) + 1.0)
    raise ValueError(name)


def add_bias(x, bias, z=None, y=None, alpha1=1.0, alpha2=1.0, beta1=0.0, beta2=0.0, beta3=0.0, act="linear"):
    """y = alpha1 * act(alpha2 * x + b + beta1 * z) + beta2 * z + beta3 * y  (reference src/tensor_op.cu:199-228), float64."""
    x = np.asarray(x, dtype=np.float64)
    t = alpha2 * x + np.asarray(bias, dtype=np.float64)
    if z is not None and (beta1 != 0.0 or beta2 != 0.0):
        z = np.asarray(z, dtype=np.float64)
        t = alpha1 * activation(t + beta1 * z, act) + beta2 * z
    else:
        t = alpha1 * activation(t, act)
    if beta3 != 0.0:
        t = t + beta3 * np.asarray(y, dtype=np.float64)
    return t


def im2row(x, kernel=(3, 3), padding=(-1, -1), rotate=False, padding_value=0):
    """rows[N*Ho*Wo, kh*kw*C] of the explicit lowering (reference src/im2row.cu:29-66, restated as a gather).

    Tap (i, j) of an output pixel (oh, ow) reads input pixel (oh + i + padding_h, ow + j + padding_w); pixels outside the
    image hold padding_value; rotate=True (CROSS_CORRELATION_MODE) stores the taps in the opposite order.  Works on any
    dtype: values are only moved.  Pure numpy, small cases only.
    """
    x = np.asarray(x)
    N, H, W, C = x.shape
    kh, kw = kernel
    Ho, Wo = H - 2 * padding[0] - (kh - 1), W - 2 * padding[1] - (kw - 1)
    rows = np.empty((N, Ho, Wo, kh * kw, C), dtype=x.dtype)
    for i in range(kh):
        for j in range(kw):
            tap = i * kw + j
            src = (kh * kw - 1 - tap) if rotate else tap
            si, sj = divmod(src, kw)
            plane = np.full((N, Ho, Wo, C), padding_value, dtype=x.dtype)
            h0, w0 = si + padding[0], sj + padding[1]          # input coordinate of output (0, 0)
            oh_lo, oh_hi = max(0, -h0), min(Ho, H - h0)
            ow_lo, ow_hi = max(0, -w0), min(Wo, W - w0)
            if oh_hi > oh_lo and ow_hi > ow_lo:
                plane[:, oh_lo:oh_hi, ow_lo:ow_hi, :] = x[:, oh_lo + h0:oh_hi + h0, ow_lo + w0:ow_hi + w0, :]
            rows[:, :, :, tap, :] = plane
    return rows.reshape(N * Ho * Wo, kh * kw * C)


def optimizer_learn(kind, w, dw, state, learning_rate, coef=(0.0, 0.0), momentum=False, nesterov=False, steps=0, alpha=1.0, beta=0.0, eps=None):
    """One weight update in float64 (reference src/optimizers.cu:34-70 and :111-160); returns (w, state).

    kind "sgd": state = momentum buffer or None; kind "adam": state = (m, v), bias correction at t = steps + 1.
    eps: the flush-to-zero threshold and Adam's epsilon (machine epsilon of the tensor dtype on the device).
    """
    w = np.asarray(w, dtype=np.float64)
    dw = np.asarray(dw, dtype=np.float64)
    eps = np.finfo(np.float32).eps if eps is None else eps
    if kind == "sgd":
        if momentum:
            m = coef[0] * state - learning_rate * dw
            step = coef[0] * m - learning_rate * dw if nesterov else m
            state = m
        else:
            step = -learning_rate * dw
    else:
        m, v = state
        m = m * coef[0] + dw * (1.0 - coef[0])
        v = v * coef[1] + dw * dw * (1.0 - coef[1])
        t = steps + 1
        lr = learning_rate
        if t < 10000:
            lr = lr * np.sqrt(1.0 - coef[1] ** t) / (1.0 - coef[0] ** t)
        step = -m * lr / np.sqrt(v + eps)
        state = (m, v)
    out = alpha * step + beta * w
    out = np.where(np.abs(out) < eps, 0.0, out)
    return out, state


def gemm_batched(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None):
    """C[i] = alpha * op(A[i]) * op(B[i]) + beta * C[i] in float64 (row-major 3-D arrays)."""
    a, b = _f64(a), _f64(b)
    opa = np.swapaxes(a, 1, 2) if trans_a else a
    opb = np.swapaxes(b, 1, 2) if trans_b else b
    out = alpha * np.matmul(opa, opb)
    if c is not None and beta != 0.0:
        out = out + beta * np.asarray(c, dtype=np.float64)
    return out


def error_metrics(result, reference):
    """The three error figures quoted for floating-point parity.

    elem: max |e| / max(|ref|, rms(ref))  (headline; plain relative error is meaningless where ref crosses zero)
    norm: max |e| / max |ref|
    rms:  rms(e) / rms(ref)
    """
    result = np.asarray(result, dtype=np.float64)
    reference = np.asarray(reference, dtype=np.float64)
    err = np.abs(result - reference)
    rms_ref = float(np.sqrt(np.mean(reference * reference)))
    if rms_ref == 0.0:
        rms_ref = 1.0
    elem = float(np.max(err / np.maximum(np.abs(reference), rms_ref))) if err.size else 0.0
    norm = float(np.max(err) / max(float(np.max(np.abs(reference))), 1e-300)) if err.size else 0.0
    rms = float(np.sqrt(np.mean(err * err)) / rms_ref) if err.size else 0.0
    return {"elem": elem, "norm": norm, "rms": rms}
