"""autograph_b200 — B200 (sm_100a) backend for autograph's dense-contraction path.

The product is the C-ABI shared library ``libautograph_b200.so`` (declared in
``include/autograph_b200.h``).  This package is a thin ctypes front end over it
that mirrors the reference's operator interface (``dot``, ``Conv2`` / ``Dense`` /
``MaxPool2`` / ``Relu`` forward and backward, cross-entropy, SGD, and the
LeNet5-style model object) so that tests and benchmarks read like the
reference's own.  PyTorch is used only to hold device memory, streams and for
``torch.distributed``.

There is no CPU fallback: if the library is missing, importing this package
fails; if there is no B200, creating a :class:`Device` fails.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

from . import _capi
from ._capi import AgError, lib, lib_path  # noqa: F401

__all__ = ["AgError", "Device", "Model", "lib", "lib_path", "LENET5_SPEC", "WIDE_STACK_SPEC"]

_HERE = Path(__file__).resolve().parent


def _torch():
    import torch
    return torch


_DTYPE_CODES = {}


def _dtype_code(t) -> int:
    if not _DTYPE_CODES:
        torch = _torch()
        _DTYPE_CODES.update({torch.float32: _capi.AG_F32, torch.bfloat16: _capi.AG_BF16,
                             torch.uint8: _capi.AG_U8, torch.uint16: _capi.AG_U16,
                             torch.uint32: _capi.AG_U32})
    try:
        return _DTYPE_CODES[t]
    except KeyError:
        raise AgError(_capi.AG_ERR_DTYPE, f"dtype {t} unimplemented") from None


def _ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _conv_options(filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    o = _capi.ConvOptions()
    o.filter[0], o.filter[1] = filter
    o.padding[0], o.padding[1] = padding
    o.stride[0], o.stride[1] = stride
    o.dilation[0], o.dilation[1] = dilation
    return o


def kernel_launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    n = ctypes.c_uint64()
    _capi.check(lib().ag_kernel_launch_count(ctypes.byref(n)))
    return n.value


class Device:
    """≙ ``Device::builder().index(i).build()``.  Work is submitted to a CUDA
    stream: by default a torch stream created here, which also becomes torch's
    current stream for the GPU, so that torch allocations, copies and events are
    ordered with the library's kernels.  A second Device on the same GPU makes ITS stream
    current: torch operations on tensors of the first must then be ordered by the caller
    (``torch.cuda.set_stream(first.stream)`` or an event)."""

    def __init__(self, index: int = 0, stream=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise AgError(_capi.AG_ERR_CUDA, "no CUDA device is visible (there is no CPU fallback)")
        self.index = index
        self.torch_device = torch.device("cuda", index)
        with torch.cuda.device(index):
            self.stream = stream if stream is not None else torch.cuda.Stream(device=index)
            torch.cuda.set_stream(self.stream)
        self._stream_ptr = self.stream.cuda_stream
        handle = ctypes.c_void_p()
        _capi.check(lib().ag_device_create_on_stream(index, ctypes.c_void_p(self.stream.cuda_stream),
                                                     ctypes.byref(handle)))
        self._h = handle

    def close(self):
        if getattr(self, "_h", None):
            lib().ag_device_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ≙ device.wait()
    def wait(self):
        _capi.check(lib().ag_device_wait(self._h))

    # -- tensors -------------------------------------------------------------
    def empty(self, shape, dtype):
        torch = _torch()
        return torch.empty(shape, dtype=dtype, device=self.torch_device)

    # Memory-safety net for tests (compute-sanitizer's place where it cannot run): with guards
    # on, every output an operator allocates sits between two red zones and is pre-filled
    # with a poison pattern (all bits set: a NaN no kernel produces).  check_guards() then
    # reports an operator that wrote outside its output (a damaged red zone) or left part of
    # it unwritten (surviving poison).  Off by default; costs two fills per output.
    GUARD_BYTES = 512

    def set_guards(self, on: bool):
        self._guarded = [] if on else None
        self._guard_mark = 0

    def _out(self, shape, dtype):
        """Output buffer of an operator (guarded and poisoned when guards are on)."""
        torch = _torch()
        if getattr(self, "_guarded", None) is None:
            return torch.empty(shape, dtype=dtype, device=self.torch_device)
        import weakref
        n = 1
        for d in shape:
            n *= int(d)
        es = torch.empty((), dtype=dtype).element_size()
        pad = self.GUARD_BYTES // es
        raw = torch.empty((n + 2 * pad,), dtype=dtype, device=self.torch_device)
        raw.view(torch.uint8).fill_(0xFF)
        out = raw[pad:pad + n].view(tuple(shape))
        self._guarded.append((weakref.ref(out), raw, pad, n, tuple(shape)))
        return out

    def _check(self, status):
        """_capi.check for operator calls: outputs allocated for a call that failed are not
        expected to have been written."""
        guarded = getattr(self, "_guarded", None)
        if status != _capi.AG_OK and guarded is not None:
            del guarded[getattr(self, "_guard_mark", 0):]
        _capi.check(status)
        if guarded is not None:
            self._guard_mark = len(guarded)

    def check_guards(self):
        """Raises AssertionError for the first damaged red zone or unwritten output among the
        outputs that are still alive; forgets all of them."""
        torch = _torch()
        entries, self._guarded = (self._guarded or []), ([] if self._guarded is not None else None)
        self._guard_mark = 0
        torch.cuda.current_stream(self.index).synchronize()
        self.stream.synchronize()
        for ref, raw, pad, n, shape in entries:
            bytes_ = raw.view(torch.uint8)
            es = raw.element_size()
            lo, hi = bytes_[:pad * es], bytes_[(pad + n) * es:]
            assert bool((lo == 0xFF).all()) and bool((hi == 0xFF).all()), \
                f"an operator wrote outside its output of shape {shape}"
            if ref() is None or n == 0:
                continue   # the caller dropped it (e.g. the call raised): nothing to say
            body = bytes_[pad * es:(pad + n) * es].view(-1, es)
            unwritten = int((body == 0xFF).all(dim=1).sum())
            assert unwritten == 0, f"{unwritten} of {n} elements of an output of shape {shape} were never written"

    def tensor(self, array, dtype=None):
        """Host numpy array -> device tensor (≙ Tensor::from(array).into_device(device))."""
        torch = _torch()
        t = torch.from_numpy(array)
        if dtype is not None:
            t = t.to(dtype)
        out = t.to(self.torch_device)
        torch.cuda.current_stream(self.index).synchronize()
        return out

    def _sync_in(self):
        # Inputs were produced on torch's current stream; order this stream after it (nothing
        # to do when that stream is this device's own, which is the case unless the caller
        # changed torch's current stream after creating the device).
        cur = _torch().cuda.current_stream(self.index)
        if cur.cuda_stream != self._stream_ptr:
            self.stream.wait_stream(cur)

    # -- linalg ----------------------------------------------------------------
    def gemm(self, alpha, a, b, beta, c):
        """C = alpha*A.B + beta*C on 2-D (possibly transposed) views; ≙ fn gemm."""
        if a.dtype != b.dtype:
            raise AgError(_capi.AG_ERR_DTYPE, "a_scalar_type != b_scalar_type")
        if a.dtype != c.dtype:
            raise AgError(_capi.AG_ERR_DTYPE, "a_scalar_type != c_scalar_type")
        m, k = a.shape
        k2, n = b.shape
        m2, n2 = c.shape
        if m != m2:
            raise AgError(_capi.AG_ERR_SHAPE, f"a_rows != c_rows, {m} != {m2}")
        if k != k2:
            raise AgError(_capi.AG_ERR_SHAPE, f"a_cols != b_rows, {k} != {k2}")
        if n != n2:
            raise AgError(_capi.AG_ERR_SHAPE, f"b_cols != c_rows, {n} != {n2}")
        self._sync_in()
        self._check(lib().ag_gemm(
            self._h, _dtype_code(a.dtype), m, k, n, ctypes.c_float(alpha),
            _ptr(a), 0, a.stride(0), a.stride(1), _ptr(b), 0, b.stride(0), b.stride(1),
            ctypes.c_float(beta), _ptr(c), 0, c.stride(0), c.stride(1)))
        return c

    def dot(self, a, b):
        """≙ ``a.dot(&b)`` (Dot for TensorBase / ScalarTensorBase): fresh [m, n] output."""
        if a.dtype != b.dtype:
            raise AgError(_capi.AG_ERR_DTYPE,
                          f"Can not dot tensors of different types {a.dtype} != {b.dtype}!")
        if a.shape[1] != b.shape[0]:
            raise AgError(_capi.AG_ERR_SHAPE, f"a_cols != b_rows, {a.shape[1]} != {b.shape[0]}")
        c = self._out((a.shape[0], b.shape[1]), a.dtype)
        return self.gemm(1.0, a, b, 0.0, c)

    # -- convolution -----------------------------------------------------------
    def conv2_output_shape(self, ih, iw, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
        oh, ow = ctypes.c_int64(), ctypes.c_int64()
        o = _conv_options(filter, padding, stride, dilation)
        self._check(lib().ag_conv2_output_shape(ih, iw, ctypes.byref(o), ctypes.byref(oh),
                                                ctypes.byref(ow)))
        return oh.value, ow.value

    def conv2_forward(self, x, w, bias=None, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                      relu=False):
        bs, ic, ih, iw = x.shape
        oc, ic2, fh, fw = w.shape
        if ic != ic2:
            raise AgError(_capi.AG_ERR_SHAPE, "input channels do not match the weight")
        o = _conv_options((fh, fw), padding, stride, dilation)
        oh, ow = self.conv2_output_shape(ih, iw, (fh, fw), padding, stride, dilation)
        y = self._out((bs, oc, oh, ow), x.dtype)
        self._sync_in()
        self._check(lib().ag_conv2_forward(self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs,
                                           ic, ih, iw, _ptr(w.contiguous()), oc, _ptr(bias),
                                           ctypes.byref(o), int(relu), _ptr(y)))
        return y

    def conv2_relu_max_pool2(self, x, w, bias=None, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                             relu=True, pool=(2, 2)):
        """Conv2 -> Relu -> MaxPool2 (window = stride) in one call (inference fusion)."""
        bs, ic, ih, iw = x.shape
        oc, ic2, fh, fw = w.shape
        if ic != ic2:
            raise AgError(_capi.AG_ERR_SHAPE, "input channels do not match the weight")
        o = _conv_options((fh, fw), padding, stride, dilation)
        oh, ow = self.conv2_output_shape(ih, iw, (fh, fw), padding, stride, dilation)
        if oh < pool[0] or ow < pool[1]:
            raise AgError(_capi.AG_ERR_SHAPE, "pool window does not fit the convolution output")
        y = self._out((bs, oc, (oh - pool[0]) // pool[0] + 1, (ow - pool[1]) // pool[1] + 1),
                       x.dtype)
        self._sync_in()
        self._check(lib().ag_conv2_relu_max_pool2_forward(
            self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs, ic, ih, iw,
            _ptr(w.contiguous()), oc, _ptr(bias), ctypes.byref(o), int(relu), pool[0], pool[1],
            _ptr(y)))
        return y

    def conv2_relu_max_pool2_keep(self, x, w, bias=None, padding=(0, 0), stride=(1, 1),
                                  dilation=(1, 1)):
        """Conv2 -> Relu -> 2x2 MaxPool2 for a gradient-recording pass: returns (the
        convolution's output, the pooled activations)."""
        bs, ic, ih, iw = x.shape
        oc, ic2, fh, fw = w.shape
        if ic != ic2:
            raise AgError(_capi.AG_ERR_SHAPE, "input channels do not match the weight")
        o = _conv_options((fh, fw), padding, stride, dilation)
        oh, ow = self.conv2_output_shape(ih, iw, (fh, fw), padding, stride, dilation)
        pre = self._out((bs, oc, oh, ow), x.dtype)
        y = self._out((bs, oc, oh // 2, ow // 2), x.dtype)
        self._sync_in()
        self._check(lib().ag_conv2_relu_max_pool2_forward_keep(
            self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs, ic, ih, iw,
            _ptr(w.contiguous()), oc, _ptr(bias), ctypes.byref(o), _ptr(pre), _ptr(y)))
        return pre, y

    def dense_forward(self, x, w, bias=None, relu=False):
        """≙ Dense::forward (x.dot(w) + bias) with an optional following Relu folded in."""
        if x.dtype != w.dtype:
            raise AgError(_capi.AG_ERR_DTYPE, "Can not dot tensors of different types")
        if x.shape[1] != w.shape[0]:
            raise AgError(_capi.AG_ERR_SHAPE, f"a_cols != b_rows, {x.shape[1]} != {w.shape[0]}")
        y = self._out((x.shape[0], w.shape[1]), x.dtype)
        self._sync_in()
        self._check(lib().ag_dense_forward(self._h, _dtype_code(x.dtype), _ptr(x.contiguous()),
                                           x.shape[0], x.shape[1], _ptr(w.contiguous()),
                                           w.shape[1], _ptr(bias), int(relu), _ptr(y)))
        return y

    def dense_chain_forward(self, x, weights, biases=None, relus=None):
        """A run of Dense (+ Relu) layers in one call; weights[i] is [in_i, out_i]."""
        n = len(weights)
        biases = biases or [None] * n
        relus = relus or [False] * n
        dims = (ctypes.c_int64 * (n + 1))(x.shape[1], *[w.shape[1] for w in weights])
        ws = (ctypes.c_void_p * n)(*[w.contiguous().data_ptr() for w in weights])
        bs = (ctypes.c_void_p * n)(*[(b.data_ptr() if b is not None else None) for b in biases])
        rl = (ctypes.c_int32 * n)(*[int(r) for r in relus])
        y = self._out((x.shape[0], weights[-1].shape[1]), x.dtype)
        self._sync_in()
        self._check(lib().ag_dense_chain_forward(self._h, _dtype_code(x.dtype),
                                                 _ptr(x.contiguous()), x.shape[0], n, dims, ws, bs,
                                                 rl, _ptr(y)))
        return y

    def dense_chain_forward_keep(self, x, weights, biases=None, relus=None):
        """The same run for a pass that records gradients: returns (pre, act), the outputs of
        every Dense and (where relus[i]) of the Relu after it; act[i] is None without a Relu."""
        n = len(weights)
        biases = biases or [None] * n
        relus = relus or [False] * n
        dims = (ctypes.c_int64 * (n + 1))(x.shape[1], *[w.shape[1] for w in weights])
        ws = (ctypes.c_void_p * n)(*[w.contiguous().data_ptr() for w in weights])
        bs = (ctypes.c_void_p * n)(*[(b.data_ptr() if b is not None else None) for b in biases])
        rl = (ctypes.c_int32 * n)(*[int(r) for r in relus])
        pre = [self._out((x.shape[0], w.shape[1]), x.dtype) for w in weights]
        act = [self._out((x.shape[0], w.shape[1]), x.dtype) if r else None
               for w, r in zip(weights, relus)]
        pp = (ctypes.c_void_p * n)(*[_ptr(t) for t in pre])
        ap = (ctypes.c_void_p * n)(*[(_ptr(t) if t is not None else None) for t in act])
        self._sync_in()
        self._check(lib().ag_dense_chain_forward_keep(self._h, _dtype_code(x.dtype),
                                                      _ptr(x.contiguous()), x.shape[0], n, dims, ws,
                                                      bs, rl, pp, ap))
        return pre, act

    def dense_chain_backward(self, x, weights, relus, pre, act, dy, has_bias=None, want_dx=True):
        """Every gradient of a Dense (+ Relu) run from the values dense_chain_forward_keep kept.
        Returns (dx or None, [dw], [db or None], [gradient at each Dense's output])."""
        n = len(weights)
        has_bias = has_bias or [False] * n
        dt = x.dtype
        dims = (ctypes.c_int64 * (n + 1))(x.shape[1], *[w.shape[1] for w in weights])
        ins = [x.contiguous()] + [(act[i] if relus[i] else pre[i]) for i in range(n - 1)]
        g = [self._out(p.shape, dt) for p in pre]
        dw = [self._out(w.shape, dt) for w in weights]
        db = [self._out((w.shape[1],), dt) if b else None for w, b in zip(weights, has_bias)]
        dx = self._out(x.shape, dt) if want_dx else None
        dy = dy.contiguous()
        if not relus[-1]:
            g[-1] = dy
        arr = lambda ts: (ctypes.c_void_p * n)(*[(_ptr(t) if t is not None else None) for t in ts])
        self._sync_in()
        self._check(lib().ag_dense_chain_backward(
            self._h, _dtype_code(dt), x.shape[0], n, dims, arr(ins),
            arr([w.contiguous() for w in weights]), arr([pre[i] if relus[i] else None for i in range(n)]),
            _ptr(dy), arr([g[i] if (i < n - 1 or relus[i]) else None for i in range(n)]),
            _ptr(dx) if dx is not None else None, arr(dw), arr(db)))
        return dx, dw, db, g

    # ---- 1-D wrappers: ≙ Conv1 / MaxPool1 (layer.rs:1007-1033, 1173-1191), which reshape
    # [n, c, l] to [n, c, l, 1] and call the 2-D operators
    def conv1_forward(self, x, w, bias=None, padding=0, stride=1, dilation=1, relu=False):
        n, c, l = x.shape
        oc, ic, f = w.shape
        y = self.conv2_forward(x.reshape(n, c, l, 1), w.reshape(oc, ic, f, 1), bias=bias,
                               padding=(padding, 0), stride=(stride, 1), dilation=(dilation, 1),
                               relu=relu)
        return y.reshape(n, oc, y.shape[2])

    def conv1_backward_input(self, w, dy, length, padding=0, stride=1, dilation=1):
        oc, ic, f = w.shape
        n = dy.shape[0]
        dx = self.conv2_backward_input(w.reshape(oc, ic, f, 1), dy.reshape(n, oc, dy.shape[2], 1),
                                       (length, 1), padding=(padding, 0), stride=(stride, 1),
                                       dilation=(dilation, 1))
        return dx.reshape(n, ic, length)

    def conv1_backward_weight(self, x, dy, filter, padding=0, stride=1, dilation=1):
        n, c, l = x.shape
        oc = dy.shape[1]
        dw = self.conv2_backward_weight(x.reshape(n, c, l, 1), dy.reshape(n, oc, dy.shape[2], 1),
                                        (filter, 1), padding=(padding, 0), stride=(stride, 1),
                                        dilation=(dilation, 1))
        return dw.reshape(oc, c, filter)

    def max_pool1(self, x, size=2, stride=None):
        n, c, l = x.shape
        y = self.max_pool2(x.reshape(n, c, l, 1), (size, 1), (stride or size, 1))
        return y.reshape(n, c, y.shape[2])

    def scaled_cast_u8(self, x_u8, alpha, dtype):
        """≙ Tensor::scaled_cast for u8 input: alpha * x in `dtype` (f32 or bf16)."""
        y = self._out(tuple(x_u8.shape), dtype)
        self._sync_in()
        self._check(lib().ag_scaled_cast_u8(self._h, _dtype_code(dtype), ctypes.c_float(alpha),
                                            _ptr(x_u8.contiguous()), _ptr(y), x_u8.numel()))
        return y

    def conv_dense_chain_forward(self, x, convs, weights, biases=None, relus=None, u8_alpha=None):
        """A small network in one kernel.  convs: list of (w, bias, relu, pool) with pool a
        (ph, pw) window or None; then Flatten and the Dense (+ Relu) layers of
        dense_chain_forward.  With u8_alpha, x is a u8 tensor that the kernel scales by
        u8_alpha into the weights' dtype while staging it.  Raises AgError(AG_ERR_UNSUPPORTED)
        when the network does not fit the fused kernel."""
        bs, ic, ih, iw = x.shape
        stages = (_capi.ConvStage * len(convs))()
        keep = []
        for st, (w, b, relu, pool) in zip(stages, convs):
            w = w.contiguous()
            keep.append(w)
            st.w = w.data_ptr()
            st.bias = b.data_ptr() if b is not None else None
            st.oc = w.shape[0]
            st.options = _conv_options(tuple(w.shape[2:]))
            st.relu = int(relu)
            st.pool[0], st.pool[1] = pool if pool else (0, 0)
        n = len(weights)
        biases = biases or [None] * n
        relus = relus or [False] * n
        weights = [w.contiguous() for w in weights]
        dims = (ctypes.c_int64 * (n + 1))(weights[0].shape[0], *[w.shape[1] for w in weights])
        ws = (ctypes.c_void_p * n)(*[w.data_ptr() for w in weights])
        bp = (ctypes.c_void_p * n)(*[(b.data_ptr() if b is not None else None) for b in biases])
        rl = (ctypes.c_int32 * n)(*[int(r) for r in relus])
        out_dtype = weights[0].dtype
        y = self._out((bs, weights[-1].shape[1]), out_dtype)
        self._sync_in()
        if u8_alpha is not None:
            self._check(lib().ag_conv_dense_chain_forward_u8(
                self._h, _dtype_code(out_dtype), _ptr(x.contiguous()), ctypes.c_float(u8_alpha), bs,
                ic, ih, iw, len(convs), stages, n, dims, ws, bp, rl, _ptr(y)))
        else:
            self._check(lib().ag_conv_dense_chain_forward(
                self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs, ic, ih, iw, len(convs),
                stages, n, dims, ws, bp, rl, _ptr(y)))
        return y

    def conv2_backward_input(self, w, dy, input_hw, padding=(0, 0), stride=(1, 1),
                             dilation=(1, 1)):
        oc, ic, fh, fw = w.shape
        bs = dy.shape[0]
        ih, iw = input_hw
        o = _conv_options((fh, fw), padding, stride, dilation)
        dx = self._out((bs, ic, ih, iw), dy.dtype)
        self._sync_in()
        self._check(lib().ag_conv2_backward_input(self._h, _dtype_code(dy.dtype),
                                                  _ptr(w.contiguous()), oc, ic,
                                                  _ptr(dy.contiguous()), bs, ih, iw,
                                                  ctypes.byref(o), _ptr(dx)))
        return dx

    def conv2_backward_weight(self, x, dy, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1),
                              beta=0.0, dw=None):
        bs, ic, ih, iw = x.shape
        oc = dy.shape[1]
        o = _conv_options(filter, padding, stride, dilation)
        if dw is None:
            dw = self._out((oc, ic, filter[0], filter[1]), x.dtype)
        self._sync_in()
        self._check(lib().ag_conv2_backward_weight(self._h, _dtype_code(x.dtype),
                                                   _ptr(x.contiguous()), bs, ic, ih, iw,
                                                   _ptr(dy.contiguous()), oc, ctypes.byref(o),
                                                   ctypes.c_float(beta), _ptr(dw)))
        return dw

    def im2col_conv2(self, x, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
        bs, c, ih, iw = x.shape
        o = _conv_options(filter, padding, stride, dilation)
        oh, ow = self.conv2_output_shape(ih, iw, filter, padding, stride, dilation)
        y = self._out((bs * oh * ow, c * filter[0] * filter[1]), x.dtype)
        self._sync_in()
        self._check(lib().ag_im2col_conv2(self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs,
                                          c, ih, iw, ctypes.byref(o), _ptr(y)))
        return y

    def col2im_conv2(self, x, shape, filter, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
        gh, gw = shape
        fh, fw = filter
        rows, cols = x.shape
        bs, c = rows // (gh * gw), cols // (fh * fw)
        oh = (gh - 1) * stride[0] + dilation[0] * (fh - 1) + 1 - 2 * padding[0]
        ow = (gw - 1) * stride[1] + dilation[1] * (fw - 1) + 1 - 2 * padding[1]
        o = _conv_options(filter, padding, stride, dilation)
        y = self._out((bs, c, oh, ow), x.dtype)
        self._sync_in()
        self._check(lib().ag_col2im_conv2(self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs,
                                          c, gh, gw, ctypes.byref(o), _ptr(y)))
        return y

    # -- pooling / relu ----------------------------------------------------------
    def max_pool2(self, x, size=(2, 2), strides=None):
        strides = strides or size
        bs, c, ih, iw = x.shape
        if ih < size[0] or iw < size[1]:
            raise AgError(_capi.AG_ERR_SHAPE, "pool window does not fit input")
        oh, ow = (ih - size[0]) // strides[0] + 1, (iw - size[1]) // strides[1] + 1
        y = self._out((bs, c, oh, ow), x.dtype)
        self._sync_in()
        self._check(lib().ag_max_pool2(self._h, _dtype_code(x.dtype), _ptr(x.contiguous()), bs, c,
                                       ih, iw, size[0], size[1], strides[0], strides[1], _ptr(y)))
        return y

    def max_pool2_backward_inplace(self, dx, dy, size=(2, 2), strides=None):
        """The reference's kernel form: dx holds the pool's input on entry and its gradient on
        return (cells no window covers keep the input's value)."""
        strides = strides or size
        if not dx.is_contiguous():
            raise AgError(_capi.AG_ERR_INVALID, "dx must be contiguous")
        bs, c, ih, iw = dx.shape
        self._sync_in()
        self._check(lib().ag_max_pool2_backward(self._h, _dtype_code(dx.dtype), _ptr(dx), bs, c, ih,
                                                iw, size[0], size[1], strides[0], strides[1],
                                                _ptr(dy.contiguous())))
        return dx

    def max_pool2_backward(self, x, dy, size=(2, 2), strides=None):
        """≙ the MaxPool2 backward edge: clone the input, run max_pool2_backward in place."""
        return self.max_pool2_backward_inplace(x.contiguous().clone(), dy, size, strides)

    def max_pool2_backward_from_input(self, x, dy, size=(2, 2), strides=None):
        """The same result in one pass: x is read, the gradient written (no clone)."""
        strides = strides or size
        x = x.contiguous()
        dx = self._out(x.shape, x.dtype)
        bs, c, ih, iw = x.shape
        self._sync_in()
        self._check(lib().ag_max_pool2_backward_from_input(
            self._h, _dtype_code(x.dtype), _ptr(x), bs, c, ih, iw, size[0], size[1], strides[0],
            strides[1], _ptr(dy.contiguous()), _ptr(dx)))
        return dx

    def relu_max_pool2(self, x):
        """max_pool2(relu(x)) with a 2x2 window and stride in one pass (even planes)."""
        x = x.contiguous()
        bs, c, ih, iw = x.shape
        y = self._out((bs, c, ih // 2, iw // 2), x.dtype)
        self._sync_in()
        self._check(lib().ag_relu_max_pool2_forward(self._h, _dtype_code(x.dtype), _ptr(x), bs, c,
                                                    ih, iw, _ptr(y)))
        return y

    def relu_max_pool2_backward(self, x, dy):
        """Gradient of relu_max_pool2 at x: the pool's and the Relu's backward in one pass."""
        x = x.contiguous()
        bs, c, ih, iw = x.shape
        dx = self._out(x.shape, x.dtype)
        self._sync_in()
        self._check(lib().ag_relu_max_pool2_backward(self._h, _dtype_code(x.dtype), _ptr(x), bs, c,
                                                     ih, iw, _ptr(dy.contiguous()), _ptr(dx)))
        return dx

    def relu(self, x, inplace=False):
        x = x.contiguous()
        y = x if inplace else self._out(x.shape, x.dtype)
        self._sync_in()
        self._check(lib().ag_relu(self._h, _dtype_code(x.dtype), _ptr(x), _ptr(y), x.numel()))
        return y

    def relu_backward(self, x, dy, inplace=False):
        x, dy = x.contiguous(), dy.contiguous()
        dx = dy if inplace else self._out(dy.shape, dy.dtype)
        self._sync_in()
        self._check(lib().ag_relu_backward(self._h, _dtype_code(x.dtype), _ptr(x), _ptr(dy),
                                           _ptr(dx), x.numel()))
        return dx

    # -- elementwise ---------------------------------------------------------------
    def scaled_add(self, y, alpha, x):
        """≙ ``y.scaled_add(alpha, &x)`` (in place on y)."""
        assert y.is_contiguous() and x.is_contiguous() and x.shape == y.shape
        self._sync_in()
        self._check(lib().ag_scaled_add(self._h, _dtype_code(y.dtype), ctypes.c_float(alpha),
                                        _ptr(x), _ptr(y), y.numel()))
        return y

    def bias_add(self, y, bias):
        rows, cols = y.shape[0], y.shape[1]
        inner = y[0, 0].numel() if y.dim() > 2 else 1
        self._sync_in()
        self._check(lib().ag_bias_add(self._h, _dtype_code(y.dtype), _ptr(y), _ptr(bias), rows,
                                      cols, inner))
        return y

    def bias_grad(self, dy, beta=0.0, out=None):
        rows, cols = dy.shape[0], dy.shape[1]
        inner = dy[0, 0].numel() if dy.dim() > 2 else 1
        if out is None:
            out = self._out((cols,), dy.dtype)
        self._sync_in()
        self._check(lib().ag_bias_grad(self._h, _dtype_code(dy.dtype), _ptr(dy.contiguous()), rows,
                                       cols, inner, ctypes.c_float(beta), _ptr(out)))
        return out

    # -- criterion -------------------------------------------------------------------
    def cross_entropy_loss(self, x, t) -> float:
        bs, classes = x.shape
        if t.shape[0] != bs:
            raise AgError(_capi.AG_ERR_SHAPE, f"Expected target with shape [{bs}], found "
                                              f"[{t.shape[0]}]")
        loss = ctypes.c_float()
        self._sync_in()
        self._check(lib().ag_cross_entropy_loss(self._h, _dtype_code(x.dtype), _dtype_code(t.dtype),
                                                _ptr(x.contiguous()), _ptr(t), bs, classes,
                                                ctypes.byref(loss)))
        return loss.value

    def cross_entropy_loss_with_grad(self, x, t, dy=1.0):
        """(loss as a one-element device tensor, dx) from one call; nothing synchronises."""
        torch = _torch()
        x, t = x.contiguous(), t.contiguous()
        loss = torch.empty((1,), dtype=torch.float32, device=self.torch_device)
        dx = self._out(x.shape, x.dtype)
        self._sync_in()
        self._check(lib().ag_cross_entropy_loss_device_grad(
            self._h, _dtype_code(x.dtype), _dtype_code(t.dtype), _ptr(x), _ptr(t), x.shape[0],
            x.shape[1], _ptr(loss), ctypes.c_float(dy), _ptr(dx)))
        return loss, dx

    def cross_entropy_loss_backward(self, x, t, dy=1.0):
        bs, classes = x.shape
        dx = self._out(x.shape, x.dtype)
        self._sync_in()
        self._check(lib().ag_cross_entropy_loss_backward(
            self._h, _dtype_code(x.dtype), _dtype_code(t.dtype), _ptr(x.contiguous()), _ptr(t), bs,
            classes, ctypes.c_float(dy), _ptr(dx)))
        return dx

    def accuracy(self, x, t) -> int:
        bs, classes = x.shape
        out = ctypes.c_uint64()
        self._sync_in()
        self._check(lib().ag_accuracy(self._h, _dtype_code(x.dtype), _dtype_code(t.dtype),
                                      _ptr(x.contiguous()), _ptr(t), bs, classes,
                                      ctypes.byref(out)))
        return out.value

    # -- optimizer ----------------------------------------------------------------------
    def sgd_update(self, w, g, lr):
        self._sync_in()
        self._check(lib().ag_sgd_update(self._h, _dtype_code(w.dtype), _ptr(w), _ptr(g), w.numel(),
                                        ctypes.c_float(lr)))
        return w

    def sgd_update_momentum(self, w, g, v, lr, momentum):
        self._sync_in()
        self._check(lib().ag_sgd_update_momentum(self._h, _dtype_code(w.dtype), _ptr(w), _ptr(g),
                                                 _ptr(v), w.numel(), ctypes.c_float(lr),
                                                 ctypes.c_float(momentum)))
        return w, v


# Layer specs shared with the oracle's composition (kind, a, b, c, d, bias).
LENET5_SPEC = [
    ("conv", 1, 6, (5, 5), False), ("relu",), ("pool", (2, 2)),
    ("conv", 6, 16, (5, 5), False), ("relu",), ("pool", (2, 2)),
    ("flatten",),
    ("dense", 256, 128, False), ("relu",),
    ("dense", 128, 84, False), ("relu",),
    ("dense", 84, 10, True),
]

WIDE_STACK_SPEC = [
    ("conv", 3, 64, (3, 3), False), ("relu",), ("pool", (2, 2)),
    ("conv", 64, 128, (3, 3), False), ("relu",), ("pool", (2, 2)),
    ("flatten",),
    ("dense", 128 * 14 * 14, 512, False), ("relu",),
    ("dense", 512, 10, True),
]


def _c_specs(spec):
    arr = (_capi.LayerSpec * len(spec))()
    for i, layer in enumerate(spec):
        kind = layer[0]
        s = arr[i]
        if kind == "conv":
            s.kind, s.a, s.b, s.c, s.d, s.bias = (_capi.AG_LAYER_CONV2, layer[1], layer[2],
                                                  layer[3][0], layer[3][1], int(layer[4]))
        elif kind == "dense":
            s.kind, s.a, s.b, s.bias = _capi.AG_LAYER_DENSE, layer[1], layer[2], int(layer[3])
            if len(layer) > 4:   # shares the parameters of the dense layer at spec index layer[4]
                s.c = layer[4] + 1
        elif kind == "relu":
            s.kind = _capi.AG_LAYER_RELU
        elif kind == "pool":
            s.kind, s.c, s.d = _capi.AG_LAYER_MAXPOOL2, layer[1][0], layer[1][1]
        elif kind == "flatten":
            s.kind = _capi.AG_LAYER_FLATTEN
        else:
            raise ValueError(kind)
    return arr


class Model:
    """≙ ``LeNet5Classifier`` of the reference's bench crate: a chain of layers with
    resident parameters, ``infer`` and ``train`` steps."""

    def __init__(self, device: Device, spec=None, dtype=None, seed: int = 0):
        torch = _torch()
        self.device = device
        self.spec = spec or LENET5_SPEC
        self.dtype = dtype or torch.float32
        arr = _c_specs(self.spec)
        h = ctypes.c_void_p()
        _capi.check(lib().ag_model_create(device._h, _dtype_code(self.dtype), arr, len(arr),
                                          ctypes.c_uint64(seed), ctypes.byref(h)))
        self._h = h
        n = ctypes.c_int32()
        _capi.check(lib().ag_model_parameter_count(self._h, ctypes.byref(n)))
        self.parameter_lens = []
        for i in range(n.value):
            ln = ctypes.c_int64()
            _capi.check(lib().ag_model_parameter_len(self._h, i, ctypes.byref(ln)))
            self.parameter_lens.append(ln.value)
        self.out_features = [l for l in self.spec if l[0] == "dense"][-1][2]

    def close(self):
        if getattr(self, "_h", None):
            lib().ag_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _host(self, array):
        """numpy float32 array -> contiguous host torch tensor of the model dtype."""
        torch = _torch()
        return torch.from_numpy(array).to(self.dtype).contiguous()

    def set_parameters(self, arrays):
        for i, a in enumerate(arrays):
            h = self._host(a)
            assert h.numel() == self.parameter_lens[i]
            _capi.check(lib().ag_model_set_parameter(self._h, i, _ptr(h)))

    def _fetch(self, fn, index):
        torch = _torch()
        h = torch.empty(self.parameter_lens[index], dtype=self.dtype)
        _capi.check(fn(self._h, index, _ptr(h)))
        return h.float().numpy()

    def get_parameter(self, index):
        return self._fetch(lib().ag_model_get_parameter, index)

    def get_gradient(self, index):
        return self._fetch(lib().ag_model_get_gradient, index)

    def set_sgd(self, momentum=None):
        """≙ SGD::builder().momentum(m).build(); clears the velocity state."""
        _capi.check(lib().ag_model_set_sgd(self._h,
                                           ctypes.c_float(-1.0 if momentum is None else momentum)))
        self.momentum = momentum

    def get_velocity(self, index):
        return self._fetch(lib().ag_model_get_velocity, index)

    def set_velocities(self, arrays):
        for i, a in enumerate(arrays):
            h = self._host(np.asarray(a, dtype="float32").ravel())
            assert h.numel() == self.parameter_lens[i]
            _capi.check(lib().ag_model_set_velocity(self._h, i, _ptr(h)))

    def set_grad_scale(self, scale: float):
        _capi.check(lib().ag_model_set_grad_scale(self._h, ctypes.c_float(scale)))

    def _check(self, t, what, dtype, cuda, shape=None):
        """The library reads raw pointers: refuse tensors it would read past or misread."""
        if t.dtype != dtype:
            raise AgError(_capi.AG_ERR_DTYPE, f"{what}: expected {dtype}, found {t.dtype}")
        if not t.is_contiguous():
            raise AgError(_capi.AG_ERR_INVALID, f"{what} must be contiguous")
        if t.is_cuda != cuda:
            raise AgError(_capi.AG_ERR_INVALID,
                          f"{what} must be in {'device' if cuda else 'host'} memory")
        if cuda and t.device.index != self.device.index:
            raise AgError(_capi.AG_ERR_INVALID, f"{what} is on another GPU")
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise AgError(_capi.AG_ERR_SHAPE, f"{what}: expected shape {tuple(shape)}, found "
                                              f"{tuple(t.shape)}")

    def infer(self, x_host, out_host=None):
        """Host tensor [bs,c,h,w] (model dtype, ideally pinned) -> host logits (blocking)."""
        torch = _torch()
        bs, c, h, w = x_host.shape
        self._check(x_host, "x_host", self.dtype, False)
        if out_host is None:
            out_host = torch.empty((bs, self.out_features), dtype=self.dtype)
        self._check(out_host, "out_host", self.dtype, False, (bs, self.out_features))
        _capi.check(lib().ag_model_infer(self._h, _ptr(x_host), bs, c, h, w, _ptr(out_host)))
        return out_host

    def infer_enqueue(self, x_host, out_host) -> int:
        """Pipelined form of infer for two batches in flight: starts the copy of the pinned batch
        and the network behind it, returns a ticket at once; infer_wait(ticket) blocks until
        out_host (pinned) holds the logits."""
        bs, c, h, w = x_host.shape
        self._check(x_host, "x_host", self.dtype, False)
        self._check(out_host, "out_host", self.dtype, False, (bs, self.out_features))
        ticket = ctypes.c_int32(-1)
        _capi.check(lib().ag_model_infer_enqueue(self._h, _ptr(x_host), bs, c, h, w, _ptr(out_host),
                                                 ctypes.byref(ticket)))
        return ticket.value

    def infer_wait(self, ticket: int):
        _capi.check(lib().ag_model_infer_wait(self._h, ticket))

    def infer_u8(self, x_host_u8, alpha=1.0 / 255.0, out_host=None):
        """u8 host images [bs,c,h,w] -> alpha * x in the model dtype -> host logits (blocking);
        ≙ images_to_device_and_scale + forward of the reference's MNIST example."""
        torch = _torch()
        bs, c, h, w = x_host_u8.shape
        self._check(x_host_u8, "x_host_u8", torch.uint8, False)
        if out_host is None:
            out_host = torch.empty((bs, self.out_features), dtype=self.dtype)
        self._check(out_host, "out_host", self.dtype, False, (bs, self.out_features))
        _capi.check(lib().ag_model_infer_u8(self._h, _ptr(x_host_u8), bs, c, h, w,
                                            ctypes.c_float(alpha), _ptr(out_host)))
        return out_host

    def to_serde_json(self, field_names) -> str:
        """The model as serde_json text in the reference's layout (one field name per layer,
        as in the user's model struct); see serde_format."""
        from . import serde_format as sf
        n = len(self.parameter_lens)
        params = [self.get_parameter(i) for i in range(n)]
        bf16 = self.dtype == _torch().bfloat16
        # optimizer state travels with the parameters when there is one (SGD with momentum)
        vel = [self.get_velocity(i) for i in range(n)] if getattr(self, "momentum", None) else None
        return sf.dumps(sf.model_to_value(self.spec, params, field_names, bf16=bf16, velocities=vel))

    def load_serde_json(self, text: str):
        """Loads the parameters of a stack written by to_serde_json or by the reference."""
        from . import serde_format as sf
        params, states = sf.model_from_value(sf.loads(text), with_state=True)
        if [p.size for p in params] != list(self.parameter_lens):
            raise AgError(_capi.AG_ERR_SHAPE, "checkpoint does not match the model's parameters")
        self.set_parameters(params)
        if all(v is not None for v in states) and getattr(self, "momentum", None):
            self.set_velocities(states)   # a momentum run continues where it stopped

    def forward_device(self, x_dev, out_dev=None):
        bs, c, h, w = x_dev.shape
        self._check(x_dev, "x_dev", self.dtype, True)
        if out_dev is None:
            out_dev = self.device.empty((bs, self.out_features), self.dtype)
        self._check(out_dev, "out_dev", self.dtype, True, (bs, self.out_features))
        _capi.check(lib().ag_model_forward_device(self._h, _ptr(x_dev), bs, c, h, w, _ptr(out_dev)))
        return out_dev

    def train_step(self, x_host, t_host, lr) -> float:
        bs, c, h, w = x_host.shape
        self._check(x_host, "x_host", self.dtype, False)
        self._check(t_host, "t_host", _torch().uint8, False, (bs,))
        loss = ctypes.c_float()
        _capi.check(lib().ag_model_train_step(self._h, _ptr(x_host), _ptr(t_host), bs, c, h, w,
                                              ctypes.c_float(lr), ctypes.byref(loss)))
        return loss.value

    def train_forward_backward(self, x_dev, t_dev, sync=True):
        """Returns (loss, grad bucket pointer, bucket length); the bucket can be all-reduced.
        sync=False only enqueues the step (loss is None; read it with last_loss())."""
        bs, c, h, w = x_dev.shape
        self._check(x_dev, "x_dev", self.dtype, True)
        self._check(t_dev, "t_dev", _torch().uint8, True, (bs,))
        loss = ctypes.c_float()
        bucket = ctypes.c_void_p()
        length = ctypes.c_int64()
        _capi.check(lib().ag_model_train_forward_backward(
            self._h, _ptr(x_dev), _ptr(t_dev), bs, c, h, w, ctypes.byref(loss) if sync else None,
            ctypes.byref(bucket), ctypes.byref(length)))
        return (loss.value if sync else None), bucket.value, length.value

    def last_loss(self) -> float:
        """Waits for the stream and returns the loss of the last enqueued step."""
        loss = ctypes.c_float()
        _capi.check(lib().ag_model_last_loss(self._h, ctypes.byref(loss)))
        return loss.value

    def apply_update(self, lr):
        _capi.check(lib().ag_model_apply_update(self._h, ctypes.c_float(lr)))
