"""GPU: the C ABI's own device and buffer management, with no torch memory anywhere.

This is the path a Rust `Buffer` would sit on (Tensor::into_device / into_array,
src/tensor.rs:1819-1833, 1923-1945): ag_device_create (a stream the library owns) ->
ag_host_alloc / plain host memory -> ag_alloc -> ag_upload -> operators -> ag_download ->
ag_free, everything through ctypes and numpy only, compared with the oracle.
"""
import ctypes

import numpy as np
import pytest

import oracle
from autograph_b200 import _capi

pytestmark = pytest.mark.gpu


def _np_view(ptr, shape, dtype=np.float32):
    n = int(np.prod(shape))
    buf = (ctypes.c_byte * (n * np.dtype(dtype).itemsize)).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype).reshape(shape)


class _Abi:
    def __init__(self):
        self.lib = _capi.lib()
        h = ctypes.c_void_p()
        _capi.check(self.lib.ag_device_create(0, ctypes.byref(h)))
        self.dev = h
        self.blocks = []

    def alloc(self, nbytes):
        p = ctypes.c_void_p()
        _capi.check(self.lib.ag_alloc(self.dev, nbytes, ctypes.byref(p)))
        self.blocks.append(p)
        return p

    def upload(self, array):
        array = np.ascontiguousarray(array)
        p = self.alloc(array.nbytes)
        _capi.check(self.lib.ag_upload(self.dev, p, array.ctypes.data_as(ctypes.c_void_p),
                                       array.nbytes))
        return p

    def download(self, p, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        _capi.check(self.lib.ag_download(self.dev, out.ctypes.data_as(ctypes.c_void_p), p,
                                         out.nbytes))
        return out

    def close(self):
        for p in self.blocks:
            _capi.check(self.lib.ag_free(self.dev, p))
        _capi.check(self.lib.ag_device_wait(self.dev))
        _capi.check(self.lib.ag_device_destroy(self.dev))


@pytest.fixture()
def abi():
    a = _Abi()
    yield a
    a.close()


def test_device_object(abi):
    lib = abi.lib
    n = ctypes.c_int()
    _capi.check(lib.ag_device_count(ctypes.byref(n)))
    assert n.value >= 1
    assert lib.ag_device_ordinal(abi.dev) == 0
    assert lib.ag_device_stream(abi.dev)            # a stream of its own
    bad = ctypes.c_void_p()
    assert lib.ag_device_create(n.value, ctypes.byref(bad)) == _capi.AG_ERR_INVALID
    assert lib.ag_device_wait(abi.dev) == _capi.AG_OK


def test_upload_copy_fill_download_round_trip(abi):
    lib = abi.lib
    rng = np.random.default_rng(1)
    # pageable host memory (what a Vec hands over) and pinned host memory
    x = rng.standard_normal(100003).astype(np.float32)
    d = abi.upload(x)
    assert np.array_equal(abi.download(d, x.shape), x)
    hp = ctypes.c_void_p()
    _capi.check(lib.ag_host_alloc(x.nbytes, ctypes.byref(hp)))
    pinned = _np_view(hp.value, x.shape)
    pinned[:] = x[::-1]
    d2 = abi.alloc(x.nbytes)
    _capi.check(lib.ag_upload(abi.dev, d2, hp, x.nbytes))
    d3 = abi.alloc(x.nbytes)
    _capi.check(lib.ag_copy(abi.dev, d3, d2, x.nbytes))
    _capi.check(lib.ag_fill_zero(abi.dev, d2, 4 * 1000))          # first 1000 elements
    pinned[:] = 0
    _capi.check(lib.ag_download(abi.dev, hp, d3, x.nbytes))        # into pinned memory
    assert np.array_equal(pinned, x[::-1])
    back = abi.download(d2, x.shape)
    assert not back[:1000].any() and np.array_equal(back[1000:], x[::-1][1000:])
    _capi.check(lib.ag_host_free(hp))
    # degenerate calls
    p = ctypes.c_void_p(1)
    assert lib.ag_alloc(abi.dev, 0, ctypes.byref(p)) == _capi.AG_OK and not p.value
    assert lib.ag_free(abi.dev, None) == _capi.AG_OK
    assert lib.ag_upload(abi.dev, None, None, 0) == _capi.AG_OK
    assert lib.ag_upload(abi.dev, None, x.ctypes.data_as(ctypes.c_void_p), 4) == _capi.AG_ERR_INVALID
    assert lib.ag_host_free(None) == _capi.AG_OK


@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_gemm_on_abi_memory(abi, layout):
    """ag_gemm on buffers from ag_alloc: a transposed operand is a stride swap over the stored
    transpose, offsets are element offsets into a larger buffer."""
    rng = np.random.default_rng(2)
    m, k, n = 77, 130, 45
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    pad_a, pad_b, pad_c = 5, 11, 3                     # element offsets
    def stored(mat, t, pad):
        flat = np.ascontiguousarray(mat.T if t else mat).ravel()
        return np.concatenate([np.full(pad, 7.0, np.float32), flat])
    ta, tb = layout[0] == "t", layout[1] == "t"
    da = abi.upload(stored(a, ta, pad_a))
    db = abi.upload(stored(b, tb, pad_b))
    dc = abi.upload(np.concatenate([np.full(pad_c, 9.0, np.float32), c0.ravel()]))
    rsa, csa = (1, m) if ta else (k, 1)
    rsb, csb = (1, k) if tb else (n, 1)
    _capi.check(abi.lib.ag_gemm(abi.dev, _capi.AG_F32, m, k, n, 0.5, da, pad_a, rsa, csa, db, pad_b,
                                rsb, csb, -2.0, dc, pad_c, n, 1))
    got = abi.download(dc, (pad_c + m * n,))
    assert (got[:pad_c] == 9.0).all()
    ref = 0.5 * (a.astype(np.float64) @ b.astype(np.float64)) - 2.0 * c0
    assert np.abs(got[pad_c:].reshape(m, n) - ref).max() <= 1e-5 * np.sqrt(k) * np.abs(ref).max()


def test_conv_pool_relu_on_abi_memory(abi):
    """Conv2 (+ bias, ReLU) -> MaxPool2 on ag_alloc'd buffers against the oracle."""
    lib = abi.lib
    rng = np.random.default_rng(3)
    bs, ic, ih, iw, oc, f = 9, 3, 14, 12, 8, 3
    x = rng.integers(-3, 4, (bs, ic, ih, iw)).astype(np.float32)
    w = rng.integers(-2, 3, (oc, ic, f, f)).astype(np.float32)
    bias = rng.integers(-5, 6, (oc,)).astype(np.float32)
    o = _capi.ConvOptions()
    o.filter[0] = o.filter[1] = f
    o.padding[0], o.padding[1] = 1, 0
    o.stride[0] = o.stride[1] = 1
    o.dilation[0] = o.dilation[1] = 1
    oh, ow = ctypes.c_int64(), ctypes.c_int64()
    _capi.check(lib.ag_conv2_output_shape(ih, iw, ctypes.byref(o), ctypes.byref(oh), ctypes.byref(ow)))
    oh, ow = oh.value, ow.value
    dx, dw, dbias = abi.upload(x), abi.upload(w), abi.upload(bias)
    dy = abi.alloc(4 * bs * oc * oh * ow)
    _capi.check(lib.ag_conv2_forward(abi.dev, _capi.AG_F32, dx, bs, ic, ih, iw, dw, oc, dbias,
                                     ctypes.byref(o), 1, dy))
    want = oracle.relu(oracle.bias_add(oracle.conv2_naive(x, w, padding=(1, 0)), bias))
    assert np.array_equal(abi.download(dy, want.shape), want)       # integer-valued: exact
    dp = abi.alloc(4 * bs * oc * (oh // 2) * (ow // 2))
    _capi.check(lib.ag_max_pool2(abi.dev, _capi.AG_F32, dy, bs, oc, oh, ow, 2, 2, 2, 2, dp))
    pooled = oracle.max_pool2(want, (2, 2))
    assert np.array_equal(abi.download(dp, pooled.shape), pooled)
    # in-place relu_backward and an axpy, still on the library's own stream
    g = rng.integers(-4, 5, pooled.shape).astype(np.float32)
    dg = abi.upload(g)
    _capi.check(lib.ag_relu_backward(abi.dev, _capi.AG_F32, dp, dg, dg, g.size))
    _capi.check(lib.ag_scaled_add(abi.dev, _capi.AG_F32, 2.0, dp, dg, g.size))
    assert np.array_equal(abi.download(dg, g.shape), np.where(pooled >= 0, g, 0) + 2 * pooled)


def test_lenet5_model_on_abi_memory(abi):
    """ag_model_create_lenet5 / ag_model_infer from pageable numpy memory (no pinned buffers,
    no torch): the copying path of the layer object, against the oracle."""
    from oracle import models
    lib = abi.lib
    h = ctypes.c_void_p()
    _capi.check(lib.ag_model_create_lenet5(abi.dev, _capi.AG_F32, 5, ctypes.byref(h)))
    P = models.init_params(models.LENET5, 2000)
    for i, p in enumerate(P):
        _capi.check(lib.ag_model_set_parameter(h, i, np.ascontiguousarray(p).ctypes.data_as(ctypes.c_void_p)))
    x = np.random.default_rng(4).uniform(0, 1, (300, 1, 28, 28)).astype(np.float32)
    out = np.empty((300, 10), np.float32)
    for _ in range(3):
        out[:] = 0
        _capi.check(lib.ag_model_infer(h, x.ctypes.data_as(ctypes.c_void_p), 300, 1, 28, 28,
                                       out.ctypes.data_as(ctypes.c_void_p)))
        ref = models.forward(models.LENET5, P, x)
        assert np.abs(out - ref).max() <= 1e-5 * np.sqrt(256) * np.abs(ref).max()
        assert np.array_equal(out.argmax(1), ref.argmax(1))
    _capi.check(lib.ag_model_destroy(h))
