"""GPU: relu, max-pool, scaled_add, bias and SGD kernels; bit-exact against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from conftest import cycle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _prep(a, dtype):
    return oracle.round_bf16(a) if dtype == torch.bfloat16 else a.astype(np.float32)


def _np(t):
    return t.float().cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_relu_golden_and_random(dev, golden, dtype):
    for c in golden.meta["relu"]:
        shape = tuple(c["shape"])
        n = shape[0] * shape[1]
        x = dev.tensor(cycle(-10, 10, n).reshape(shape), dtype)
        assert np.array_equal(_np(dev.relu(x)), golden[c["name"] + "_y"])
        xb = dev.tensor(cycle(-1, 1, n).reshape(shape), dtype)
        dy = np.arange(n, dtype=np.float32).reshape(shape)
        if dtype == torch.bfloat16:
            dy = oracle.round_bf16(dy)
        want = np.where(cycle(-1, 1, n).reshape(shape) >= 0, dy, 0)
        dyd = dev.tensor(dy, dtype)
        assert np.array_equal(_np(dev.relu_backward(xb, dyd)), want)          # relu_backward
        assert np.array_equal(_np(dev.relu_backward(xb, dyd, inplace=True)), want)  # _mut
    rng = np.random.default_rng(1)
    for n in [1, 7, 1000, 100003]:
        x = _prep(rng.standard_normal(n), dtype)
        x[::5] = 0.0
        x[1::7] = -0.0
        dy = _prep(rng.standard_normal(n), dtype)
        xd = dev.tensor(x, dtype)
        y = dev.relu(xd)
        assert np.array_equal(_np(y).view(np.uint32), oracle.relu(x).view(np.uint32))
        dx = dev.relu_backward(xd, dev.tensor(dy, dtype))
        assert np.array_equal(_np(dx).view(np.uint32), oracle.relu_backward(x, dy).view(np.uint32))
        y2 = dev.relu(xd.clone(), inplace=True)
        assert torch.equal(y, y2)
    # NaN -> 0, like x >= 0 ? x : 0
    y = dev.relu(dev.tensor(np.array([np.nan, -np.inf, np.inf], np.float32), dtype))
    assert _np(y).tolist() == [0.0, 0.0, float("inf")]


@pytest.mark.parametrize("dtype", DTYPES)
def test_max_pool2_golden(dev, golden, dtype):
    for c in golden.meta["pool"]:
        shape = tuple(c["shape"])
        x = cycle(0, 10, int(np.prod(shape))).reshape(shape)
        xd = dev.tensor(x, dtype)
        y = dev.max_pool2(xd)
        assert np.array_equal(_np(y), golden[c["name"] + "_y"])
        dy = np.arange(y.numel(), dtype=np.float32).reshape(tuple(y.shape))
        want = golden[c["name"] + "_dx"]
        if dtype == torch.bfloat16:
            dy = oracle.round_bf16(dy)
            want = oracle.max_pool2_backward(x, dy)
        assert np.array_equal(_np(dev.max_pool2_backward(xd, dev.tensor(dy, dtype))), want)
        assert np.array_equal(_np(dev.max_pool2_backward_from_input(xd, dev.tensor(dy, dtype))), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [((3, 6, 24, 24), (2, 2), None), ((2, 16, 8, 8), (2, 2), None),
                                  ((2, 4, 62, 62), (2, 2), None), ((2, 3, 29, 29), (2, 2), None),
                                  ((2, 2, 13, 17), (3, 2), None), ((1, 2, 20, 21), (2, 3), (3, 4)),
                                  # a last row no window covers (keeps x), vector / staged paths
                                  ((2, 3, 9, 16), (2, 2), None), ((2, 3, 7, 10), (2, 2), None),
                                  ((2, 3, 10, 10), (2, 2), None), ((700, 5, 12, 14), (2, 2), None)])
def test_max_pool2_random(dev, dtype, case):
    shape, size, strides = case
    rng = np.random.default_rng(2)
    x = _prep(rng.integers(-4, 5, shape).astype(np.float32) * 0.5, dtype)  # many ties
    xd = dev.tensor(x, dtype)
    y = dev.max_pool2(xd, size, strides)
    want = oracle.max_pool2(x, size, strides)
    assert np.array_equal(_np(y), want)
    dy = _prep(rng.standard_normal(want.shape), dtype)
    dx = dev.max_pool2_backward(xd, dev.tensor(dy, dtype), size, strides)
    assert np.array_equal(_np(dx), oracle.max_pool2_backward(x, dy, size, strides))
    dx = dev.max_pool2_backward_from_input(xd, dev.tensor(dy, dtype), size, strides)
    assert np.array_equal(_np(dx), oracle.max_pool2_backward(x, dy, size, strides))
    # an input that does not start on a 16-byte boundary (the staged copy keeps the source phase)
    flat = dev.empty((x.size + 3,), dtype)
    flat[3:].copy_(xd.reshape(-1))
    dx = dev.max_pool2_backward_from_input(flat[3:].reshape(xd.shape), dev.tensor(dy, dtype), size, strides)
    assert np.array_equal(_np(dx), oracle.max_pool2_backward(x, dy, size, strides))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(100, 6, 24, 24), (100, 16, 8, 8), (3, 5, 2, 2), (2, 3, 6, 10),
                                   (0, 4, 8, 8)])
def test_relu_max_pool2_equals_the_two_layers(dev, dtype, shape):
    """One pass gives what Relu then MaxPool2 give, forward and backward (ties, zeros, -0.0)."""
    rng = np.random.default_rng(21)
    x = _prep(rng.integers(-3, 4, shape).astype(np.float32) * 0.5, dtype)
    if x.size:
        x.reshape(-1)[::7] = -0.0
    xd = dev.tensor(x, dtype)
    y = dev.relu_max_pool2(xd)
    want = oracle.max_pool2(oracle.relu(x)) if x.size else np.zeros(y.shape, np.float32)
    assert np.array_equal(_np(y), want)
    dy = _prep(rng.standard_normal(want.shape), dtype)
    dx = dev.relu_max_pool2_backward(xd, dev.tensor(dy, dtype))
    if x.size:
        want_dx = oracle.relu_backward(x, oracle.max_pool2_backward(oracle.relu(x), dy))
        assert np.array_equal(_np(dx), want_dx)
        # and bit for bit what the separate kernels give
        r = dev.relu(xd)
        sep = dev.relu_backward(xd, dev.max_pool2_backward_from_input(r, dev.tensor(dy, dtype)))
        assert np.array_equal(_np(dx).view(np.uint32), _np(sep).view(np.uint32))


def test_relu_max_pool2_rejects_odd_planes(dev):
    import autograph_b200 as ag
    with pytest.raises(ag.AgError, match="even"):
        dev.relu_max_pool2(dev.empty((1, 1, 5, 4), torch.float32))


def test_max_pool2_errors(dev):
    import autograph_b200 as ag
    with pytest.raises(ag.AgError):
        dev.max_pool2(dev.empty((1, 1, 1, 4), torch.float32))
    x = dev.empty((1, 1, 6, 6), torch.float32)
    with pytest.raises(ag.AgError, match="non-overlapping"):
        dev.max_pool2_backward(x, dev.empty((1, 1, 5, 5), torch.float32), (2, 2), (1, 1))


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_add(dev, golden, dtype):
    for c in golden.meta["axpy"]:  # scaled_add_<T> (tests/integration_tests.rs:425-452)
        n = c["n"]
        y = dev.tensor(cycle(11, 20, n), dtype)
        dev.scaled_add(y, 2.0, dev.tensor(cycle(1, 10, n), dtype))
        assert np.array_equal(_np(y), golden[c["name"]])
    rng = np.random.default_rng(3)
    for n in [5, 4096, 46920, 1000001]:
        x = _prep(rng.standard_normal(n), dtype)
        y = _prep(rng.standard_normal(n), dtype)
        yd = dev.tensor(y, dtype)
        dev.scaled_add(yd, -0.01, dev.tensor(x, dtype))
        want = oracle.scaled_add(oracle.round_bf16(np.float32([-0.01]))[0]
                                 if dtype == torch.bfloat16 else -0.01, x, y,
                                 bf16=dtype == torch.bfloat16)
        assert np.array_equal(_np(yd), want)
    # unaligned views take the scalar path
    base = dev.tensor(np.zeros(1003, np.float32))
    src = dev.tensor(np.arange(1003, dtype=np.float32))
    dev.scaled_add(base[1:1002], 3.0, src[2:1003])
    assert np.array_equal(_np(base)[1:1002], 3.0 * np.arange(2, 1003, dtype=np.float32))
    assert _np(base)[0] == 0 and _np(base)[1002] == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_bias_add_and_grad(dev, golden, dtype):
    for c in golden.meta["colsum"]:
        x = cycle(1, 16, c["rows"] * c["cols"] * c["inner"]).reshape(c["rows"], c["cols"], c["inner"])
        got = _np(dev.bias_grad(dev.tensor(x, dtype)))
        want = golden[c["name"]]
        assert np.array_equal(got, oracle.round_bf16(want) if dtype == torch.bfloat16 else want)
    rng = np.random.default_rng(4)
    for shape in [(100, 10), (7, 6, 24, 24), (1000, 84)]:
        y = _prep(rng.standard_normal(shape), dtype)
        b = _prep(rng.standard_normal(shape[1]), dtype)
        yd = dev.tensor(y, dtype)
        dev.bias_add(yd, dev.tensor(b, dtype))
        assert np.array_equal(_np(yd), oracle.bias_add(y, b, bf16=dtype == torch.bfloat16))
        g = _np(dev.bias_grad(dev.tensor(y, dtype)))
        ref = y.astype(np.float64).sum(axis=tuple(i for i in range(len(shape)) if i != 1))
        tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
        assert np.abs(g - ref).max() <= tol * max(np.abs(ref).max(), 1.0)
    acc = dev.tensor(np.ones(10, np.float32))
    dev.bias_grad(dev.tensor(np.ones((100, 10), np.float32)), beta=2.0, out=acc)
    assert np.array_equal(_np(acc), np.full(10, 102.0, np.float32))


@pytest.mark.parametrize("dtype", DTYPES)
def test_sgd(dev, dtype):
    rng = np.random.default_rng(5)
    n = 46920
    bf = dtype == torch.bfloat16
    w, g, v = (_prep(rng.standard_normal(n) * s, dtype) for s in (0.1, 0.01, 0.001))
    wd = dev.tensor(w, dtype)
    dev.sgd_update(wd, dev.tensor(g, dtype), 0.01)
    assert np.array_equal(_np(wd), oracle.sgd_update(w, g, 0.01, bf16=bf))
    wd, vd = dev.tensor(w, dtype), dev.tensor(v, dtype)
    dev.sgd_update_momentum(wd, dev.tensor(g, dtype), vd, 0.01, 0.01)
    w2, v2 = oracle.sgd_update_momentum(w, g, v, 0.01, 0.01, bf16=bf)
    assert np.array_equal(_np(wd), w2) and np.array_equal(_np(vd), v2)
