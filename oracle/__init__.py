"""CPU oracle for the dense-contraction path (TEST INFRASTRUCTURE, not product code).

A ctypes front end for ``oracle.c``, the plain-C restatement of the reference's
host algorithms.  Only the test-suite, the smoke check and the CPU-baseline /
reference arm of the benchmark may import this package; the shipped library
never does.

Parity status: pinned on the generator-defined integer vectors of the
reference's own tests (exact in f32) and cross-checked against numpy/torch
f64; otherwise "parity unpinned" (the reference is Rust and cannot be built
where this was developed; its host GEMM lives in un-vendored ndarray 0.15.6 /
matrixmultiply).

Tensors are numpy float32 arrays.  A bf16 tensor is a float32 array whose
values are exactly representable in bf16 (see :func:`round_bf16`).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "liboracle.so"
_SRC = _HERE / "oracle.c"


def build(force: bool = False) -> Path:
    """Compile oracle.c into liboracle.so with gcc (skipped when up to date)."""
    if not force and _SO.exists() and _SO.stat().st_mtime >= _SRC.stat().st_mtime:
        return _SO
    cmd = [
        "gcc", "-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
        "-fvisibility=hidden", "-std=c11", str(_SRC), "-o", str(_SO), "-lm",
    ]
    subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists() or (_SRC.exists() and _SO.stat().st_mtime < _SRC.stat().st_mtime):
            build()
        _lib = ctypes.CDLL(str(_SO))
        _lib.orc_cross_entropy_loss.restype = ctypes.c_float
        _lib.orc_accuracy.restype = ctypes.c_int64
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _f(a: np.ndarray):
    assert a.dtype == np.float32
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _u32(a: np.ndarray):
    assert a.dtype == np.uint32 and a.flags.c_contiguous
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))


def _opts(filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    arr = (ctypes.c_int * 8)(filter[0], filter[1], padding[0], padding[1], stride[0], stride[1],
                             dilation[0], dilation[1])
    return arr


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Use every core this process may run on, whatever OMP_NUM_THREADS says."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(int(n))
    return num_threads()


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bf16 (ties to even), kept as float32."""
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    lib().orc_round_bf16(_f(y), ctypes.c_int64(y.size))
    return y


def scaled_cast_u8(x: np.ndarray, alpha: float, bf16=False) -> np.ndarray:
    """Tensor::scaled_cast for u8 input (src/tensor/ops.rs:209-218): alpha * x in the output type."""
    x = np.ascontiguousarray(x, dtype=np.uint8)
    y = np.empty(x.shape, np.float32)
    lib().orc_scaled_cast_u8(x.ctypes.data_as(ctypes.c_void_p), _f(y), ctypes.c_int64(x.size),
                             ctypes.c_float(alpha), int(bf16))
    return y


def conv2_output_shape(ih, iw, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    oh = (ih + 2 * padding[0] - dilation[0] * (filter[0] - 1) - 1) // stride[0] + 1
    ow = (iw + 2 * padding[1] - dilation[1] * (filter[1] - 1) - 1) // stride[1] + 1
    return oh, ow


def conv2_input_shape(oh, ow, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    """ConvOptions::input_shape of the reference (layer.rs:70-98); None when not positive."""
    ih = dilation[0] * (filter[0] - 1) + 1 + stride[0] * (oh - 1) - 2 * padding[0]
    iw = dilation[1] * (filter[1] - 1) + 1 + stride[1] * (ow - 1) - 2 * padding[1]
    if ih <= 0 or iw <= 0:
        return None
    return ih, iw


def gemm(a: np.ndarray, b: np.ndarray, c: np.ndarray | None = None, alpha=1.0, beta=0.0,
         acc="f32", bf16=False) -> np.ndarray:
    """C = alpha*A.B + beta*C on (possibly transposed / strided) 2-D float32 views.

    acc: "f32" (sequential f32), "f64" (f64 accumulation: tolerance checker),
    "bf16" (every operation rounded to bf16, the reference's host bf16 loop).
    """
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    if c is None:
        c = np.zeros((m, n), dtype=np.float32)
    assert c.shape == (m, n)
    mode = {"f32": 0, "f64": 1, "bf16": 2}[acc]
    es = 4
    lib().orc_gemm(
        ctypes.c_int64(m), ctypes.c_int64(k), ctypes.c_int64(n), ctypes.c_float(alpha),
        _f(a), ctypes.c_int64(a.strides[0] // es), ctypes.c_int64(a.strides[1] // es),
        _f(b), ctypes.c_int64(b.strides[0] // es), ctypes.c_int64(b.strides[1] // es),
        ctypes.c_float(beta),
        _f(c), ctypes.c_int64(c.strides[0] // es), ctypes.c_int64(c.strides[1] // es),
        ctypes.c_int(mode), ctypes.c_int(int(bf16)))
    return c


def gemm_f32_fast(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Threaded blocked f32 GEMM used for the timed CPU baseline."""
    m, k = a.shape
    _, n = b.shape
    c = np.empty((m, n), dtype=np.float32)
    es = 4
    lib().orc_gemm_f32_fast(
        ctypes.c_int64(m), ctypes.c_int64(k), ctypes.c_int64(n),
        _f(a), ctypes.c_int64(a.strides[0] // es), ctypes.c_int64(a.strides[1] // es),
        _f(b), ctypes.c_int64(b.strides[0] // es), ctypes.c_int64(b.strides[1] // es), _f(c))
    return c


def conv2_naive(x, w, padding=(0, 0), stride=(1, 1), dilation=(1, 1), acc64=False, bf16=False):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bs, ic, ih, iw = x.shape
    oc, ic2, fh, fw = w.shape
    assert ic == ic2
    oh, ow = conv2_output_shape(ih, iw, (fh, fw), padding, stride, dilation)
    y = np.empty((bs, oc, oh, ow), np.float32)
    lib().orc_conv2_naive(_f(x), _f(w), _f(y), bs, ic, ih, iw, oc,
                          _opts((fh, fw), padding, stride, dilation), int(acc64), int(bf16))
    return y


def conv2_backward_input_naive(w, dy, input_hw, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                               acc64=False, bf16=False):
    w = np.ascontiguousarray(w, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    oc, ic, fh, fw = w.shape
    bs = dy.shape[0]
    ih, iw = input_hw
    assert dy.shape == (bs, oc) + conv2_output_shape(ih, iw, (fh, fw), padding, stride, dilation)
    dx = np.empty((bs, ic, ih, iw), np.float32)
    lib().orc_conv2_backward_input_naive(_f(w), _f(dy), _f(dx), bs, ic, ih, iw, oc,
                                         _opts((fh, fw), padding, stride, dilation), int(acc64),
                                         int(bf16))
    return dx


def conv2_backward_weight_naive(x, dy, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                                acc64=False, bf16=False):
    x = np.ascontiguousarray(x, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    bs, ic, ih, iw = x.shape
    oc = dy.shape[1]
    fh, fw = filter
    dw = np.empty((oc, ic, fh, fw), np.float32)
    lib().orc_conv2_backward_weight_naive(_f(x), _f(dy), _f(dw), bs, ic, ih, iw, oc,
                                          _opts((fh, fw), padding, stride, dilation), int(acc64),
                                          int(bf16))
    return dw


def conv2_direct_f32(x, w):
    """The reference's host f32 production path for default options (conv_direct.rs)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    bs, ic, ih, iw = x.shape
    oc, _, fh, fw = w.shape
    y = np.empty((bs, oc, ih - fh + 1, iw - fw + 1), np.float32)
    lib().orc_conv2_direct_f32(_f(x), _f(w), _f(y), bs, ic, ih, iw, oc, fh, fw)
    return y


def conv2_direct_backward_input_f32(w, dy, input_hw):
    """Input gradient of the reference's host f32 direct convolution, in its accumulation
    order (conv_direct.rs:948-1156); default options."""
    w = np.ascontiguousarray(w, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    oc, ic, fh, fw = w.shape
    bs = dy.shape[0]
    ih, iw = input_hw
    dx = np.empty((bs, ic, ih, iw), np.float32)
    lib().orc_conv2_direct_backward_input_f32(_f(w), _f(dy), _f(dx), bs, ic, ih, iw, oc, fh, fw)
    return dx


def conv2_direct_backward_weight_f32(x, dy, filter, threads=None):
    """Weight gradient of the reference's host f32 direct convolution (conv_direct.rs:1158-1346).
    The reference's summation order depends on its thread count: `threads` stands for
    rayon::current_num_threads() (default: the oracle's own thread count)."""
    x = np.ascontiguousarray(x, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    bs, ic, ih, iw = x.shape
    oc = dy.shape[1]
    fh, fw = filter
    dw = np.empty((oc, ic, fh, fw), np.float32)
    lib().orc_conv2_direct_backward_weight_f32(_f(x), _f(dy), _f(dw), bs, ic, ih, iw, oc, fh, fw,
                                               int(threads or num_threads()))
    return dw


def im2col_conv2(x, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    x = np.ascontiguousarray(x, np.float32)
    bs, c, ih, iw = x.shape
    oh, ow = conv2_output_shape(ih, iw, filter, padding, stride, dilation)
    y = np.empty((bs * oh * ow, c * filter[0] * filter[1]), np.float32)
    lib().orc_im2col_conv2(_f(x), _f(y), bs, c, ih, iw, _opts(filter, padding, stride, dilation))
    return y


def col2im_conv2(x, shape, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1), bf16=False,
                 device_acc=False):
    """shape = patch grid [gh, gw]; returns the image [bs, c, oh, ow]."""
    x = np.ascontiguousarray(x, np.float32)
    gh, gw = shape
    fh, fw = filter
    rows, cols = x.shape
    bs = rows // (gh * gw)
    c = cols // (fh * fw)
    oh = (gh - 1) * stride[0] + dilation[0] * (fh - 1) + 1 - 2 * padding[0]
    ow = (gw - 1) * stride[1] + dilation[1] * (fw - 1) + 1 - 2 * padding[1]
    y = np.empty((bs, c, oh, ow), np.float32)
    lib().orc_col2im_conv2(_f(x), _f(y), bs, c, gh, gw, _opts(filter, padding, stride, dilation),
                           int(bf16), int(device_acc))
    return y


def max_pool2(x, size=(2, 2), strides=None):
    strides = strides or size
    x = np.ascontiguousarray(x, np.float32)
    bs, c, ih, iw = x.shape
    oh, ow = (ih - size[0]) // strides[0] + 1, (iw - size[1]) // strides[1] + 1
    y = np.empty((bs, c, oh, ow), np.float32)
    lib().orc_max_pool2(_f(x), _f(y), bs, c, ih, iw, size[0], size[1], strides[0], strides[1])
    return y


def max_pool2_backward(x, dy, size=(2, 2), strides=None):
    """Returns dx; x is the forward input (dx starts as a copy of it, as in the reference)."""
    strides = strides or size
    dx = np.ascontiguousarray(x, np.float32).copy()
    dy = np.ascontiguousarray(dy, np.float32)
    bs, c, ih, iw = dx.shape
    lib().orc_max_pool2_backward(_f(dx), _f(dy), bs, c, ih, iw, size[0], size[1], strides[0],
                                 strides[1])
    return dx


def relu(x):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_relu(_f(x), _f(y), ctypes.c_int64(x.size))
    return y


def relu_backward(x, dy):
    x = np.ascontiguousarray(x, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    dx = np.empty_like(x)
    lib().orc_relu_backward(_f(x), _f(dy), _f(dx), ctypes.c_int64(x.size))
    return dx


def scaled_add(alpha, x, y, bf16=False):
    """Returns alpha*x + y (y is not modified)."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.ascontiguousarray(y, np.float32).copy()
    lib().orc_scaled_add(ctypes.c_float(alpha), _f(x), _f(out), ctypes.c_int64(x.size), int(bf16))
    return out


def bias_add(y, bias, bf16=False):
    """y [rows, cols, *inner] + bias[cols] broadcast (Dense: inner empty; Conv2: oh, ow)."""
    out = np.ascontiguousarray(y, np.float32).copy()
    bias = np.ascontiguousarray(bias, np.float32)
    rows, cols = out.shape[0], out.shape[1]
    inner = int(np.prod(out.shape[2:])) if out.ndim > 2 else 1
    lib().orc_bias_add(_f(out), _f(bias), ctypes.c_int64(rows), ctypes.c_int64(cols),
                       ctypes.c_int64(inner), int(bf16))
    return out


def bias_grad(dy, acc64=False, bf16=False, beta=0.0, y=None):
    """Sum over every axis except axis 1 (the bias gradient)."""
    dy = np.ascontiguousarray(dy, np.float32)
    rows, cols = dy.shape[0], dy.shape[1]
    inner = int(np.prod(dy.shape[2:])) if dy.ndim > 2 else 1
    out = np.zeros(cols, np.float32) if y is None else np.ascontiguousarray(y, np.float32).copy()
    lib().orc_sum_axis_keep_mid(_f(dy), _f(out), ctypes.c_int64(rows), ctypes.c_int64(cols),
                                ctypes.c_int64(inner), ctypes.c_float(beta), int(acc64), int(bf16))
    return out


def cross_entropy_loss(x, t) -> float:
    x = np.ascontiguousarray(x, np.float32)
    t = np.ascontiguousarray(t, np.uint32)
    bs, classes = x.shape
    return float(lib().orc_cross_entropy_loss(_f(x), _u32(t), ctypes.c_int64(bs),
                                              ctypes.c_int64(classes)))


def cross_entropy_loss_backward(x, t, dy=1.0, bf16=False):
    x = np.ascontiguousarray(x, np.float32)
    t = np.ascontiguousarray(t, np.uint32)
    bs, classes = x.shape
    dx = np.empty_like(x)
    lib().orc_cross_entropy_loss_backward(_f(x), _u32(t), ctypes.c_float(dy), _f(dx),
                                          ctypes.c_int64(bs), ctypes.c_int64(classes), int(bf16))
    return dx


def accuracy(x, t) -> int:
    x = np.ascontiguousarray(x, np.float32)
    t = np.ascontiguousarray(t, np.uint32)
    bs, classes = x.shape
    return int(lib().orc_accuracy(_f(x), _u32(t), ctypes.c_int64(bs), ctypes.c_int64(classes)))


def sgd_update(w, g, lr, bf16=False):
    out = np.ascontiguousarray(w, np.float32).copy()
    g = np.ascontiguousarray(g, np.float32)
    lib().orc_sgd_update(_f(out), _f(g), ctypes.c_int64(out.size), ctypes.c_float(lr), int(bf16))
    return out


def sgd_update_momentum(w, g, v, lr, momentum, bf16=False):
    w2 = np.ascontiguousarray(w, np.float32).copy()
    v2 = np.ascontiguousarray(v, np.float32).copy()
    g = np.ascontiguousarray(g, np.float32)
    lib().orc_sgd_update_momentum(_f(w2), _f(g), _f(v2), ctypes.c_int64(w2.size),
                                  ctypes.c_float(lr), ctypes.c_float(momentum), int(bf16))
    return w2, v2
