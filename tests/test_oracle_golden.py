"""CPU: the oracle reproduces the reference's generator-defined test vectors exactly."""
import itertools

import numpy as np
import pytest

import oracle
from conftest import cycle


def test_dot_all_layouts(golden):
    for n in [2, 4, 5, 8, 16, 32, 64, 128]:
        a = cycle(1, 10, n * n).reshape(n, n)
        b = cycle(1, 10, n * n).reshape(n, n)
        for ta, tb in itertools.product("nt", "nt"):
            av = a.T if ta == "t" else a
            bv = b.T if tb == "t" else b
            for acc in ("f32", "f64"):
                c = oracle.gemm(av, bv, acc=acc)
                assert np.array_equal(c, golden[f"dot_n{n}_{ta}{tb}"]), (n, ta, tb, acc)
            # threaded GEMM used for the CPU baseline
            assert np.array_equal(oracle.gemm_f32_fast(av, bv), golden[f"dot_n{n}_{ta}{tb}"])


def test_dot_alpha_beta():
    rng = np.random.default_rng(1)
    a = rng.integers(-4, 5, (7, 9)).astype(np.float32)
    b = rng.integers(-4, 5, (9, 5)).astype(np.float32)
    c0 = rng.integers(-4, 5, (7, 5)).astype(np.float32)
    c = oracle.gemm(a, b, c0.copy(), alpha=2.0, beta=-3.0)
    assert np.array_equal(c, 2 * (a @ b) - 3 * c0)


def _conv_kw(c):
    return dict(padding=tuple(c["padding"]), stride=tuple(c["stride"]), dilation=tuple(c["dilation"]))


def test_conv_forward_backward(golden):
    for c in golden.meta["conv"]:
        bs, ic, ih, iw = c["x_shape"]
        f = tuple(c["filter"])
        x = cycle(1, 11, bs * ic * ih * iw).reshape(bs, ic, ih, iw)
        w = cycle(1, 11, c["oc"] * ic * f[0] * f[1]).reshape(c["oc"], ic, *f)
        y_true = golden[c["name"] + "_y"]
        for acc64 in (False, True):
            y = oracle.conv2_naive(x, w, acc64=acc64, **_conv_kw(c))
            assert np.array_equal(y, y_true), c
        dy = cycle(1, 11, y_true.size).reshape(y_true.shape)
        dx = oracle.conv2_backward_input_naive(w, dy, (ih, iw), **_conv_kw(c))
        dw = oracle.conv2_backward_weight_naive(x, dy, f, **_conv_kw(c))
        assert np.array_equal(dx, golden[c["name"] + "_dx"]), c
        assert np.array_equal(dw, golden[c["name"] + "_dw"]), c
        if c["padding"] == [0, 0] and c["stride"] == [1, 1] and c["dilation"] == [1, 1]:
            # the reference's host production path (conv_direct.rs), all three directions
            assert np.array_equal(oracle.conv2_direct_f32(x, w), y_true), c
            assert np.array_equal(oracle.conv2_direct_backward_input_f32(w, dy, (ih, iw)),
                                  golden[c["name"] + "_dx"]), c
            for threads in (1, 3, 16):
                assert np.array_equal(oracle.conv2_direct_backward_weight_f32(x, dy, f, threads=threads),
                                      golden[c["name"] + "_dw"]), (c, threads)


def fingerprint(a):
    """Same two numbers as tests/golden/gen_golden.py stores for every case of the full grid."""
    v = np.rint(np.asarray(a, np.float64)).astype(np.int64).ravel()
    wts = (np.arange(v.size, dtype=np.int64) * 2654435761 % 1000003) + 1
    return [int(v.sum()), int((v * wts).sum())]


def grid_kw(row, at):
    return dict(padding=(int(row[at]), int(row[at + 1])), stride=(int(row[at + 2]), int(row[at + 3])),
                dilation=(int(row[at + 4]), int(row[at + 5])))


def test_conv_full_reference_grid(golden):
    """Every case of the reference's conv grid (7 filters x 7 option sets x 10 (bs, ic, oc) x 16
    output shapes, tests/integration_tests.rs:884-923): the oracle's three results match the
    fingerprints computed from torch float64."""
    grid, fp = golden["conv_grid"], golden["conv_grid_fp"]
    assert len(grid) > 7000
    for row, want in zip(grid, fp):
        bs, ic, ih, iw, oc, fh, fw = (int(v) for v in row[:7])
        kw = grid_kw(row, 7)
        x = cycle(1, 11, bs * ic * ih * iw).reshape(bs, ic, ih, iw)
        w = cycle(1, 11, oc * ic * fh * fw).reshape(oc, ic, fh, fw)
        y = oracle.conv2_naive(x, w, **kw)
        dy = cycle(1, 11, y.size).reshape(y.shape)
        dx = oracle.conv2_backward_input_naive(w, dy, (ih, iw), **kw)
        dw = oracle.conv2_backward_weight_naive(x, dy, (fh, fw), **kw)
        got = [fingerprint(y), fingerprint(dx), fingerprint(dw)]
        assert got == want.tolist(), row.tolist()


def test_im2col_full_reference_grid(golden):
    grid, fp = golden["im2col_grid"], golden["im2col_grid_fp"]
    assert len(grid) > 5000
    for row, want in zip(grid, fp):
        bs, ch, ih, iw, gh, gw, fh, fw = (int(v) for v in row[:8])
        kw = grid_kw(row, 8)
        x = np.arange(1, bs * ch * ih * iw + 1, dtype=np.float32).reshape(bs, ch, ih, iw)
        y = oracle.im2col_conv2(x, (fh, fw), **kw)
        dy = np.arange(1, y.size + 1, dtype=np.float32).reshape(y.shape)
        dx = oracle.col2im_conv2(dy, (gh, gw), (fh, fw), **kw)
        assert [fingerprint(y), fingerprint(dx)] == want.tolist(), row.tolist()


def test_im2col_col2im(golden):
    for c in golden.meta["im2col"]:
        bs, ch, ih, iw = c["x_shape"]
        f = tuple(c["filter"])
        x = np.arange(1, bs * ch * ih * iw + 1, dtype=np.float32).reshape(bs, ch, ih, iw)
        y = oracle.im2col_conv2(x, f, **_conv_kw(c))
        y_true = golden[c["name"] + "_y"]
        assert np.array_equal(y, y_true), c
        dy = np.arange(1, y.size + 1, dtype=np.float32).reshape(y.shape)
        for device_acc in (False, True):
            dx = oracle.col2im_conv2(dy, c["grid"], f, device_acc=device_acc, **_conv_kw(c))
            assert np.array_equal(dx, golden[c["name"] + "_dx"]), c


def test_conv_is_im2col_times_weight():
    # conv2_im2col of the reference: im2col -> dot(W^T) -> [b,oh,ow,oc] -> NCHW (layer.rs:950-1005)
    rng = np.random.default_rng(3)
    x = rng.integers(-3, 4, (2, 3, 7, 6)).astype(np.float32)
    w = rng.integers(-3, 4, (4, 3, 3, 2)).astype(np.float32)
    im = oracle.im2col_conv2(x, (3, 2), (1, 0), (2, 1), (1, 2))
    y = oracle.gemm(im, w.reshape(4, -1).T)
    oh, ow = oracle.conv2_output_shape(7, 6, (3, 2), (1, 0), (2, 1), (1, 2))
    y = y.reshape(2, oh, ow, 4).transpose(0, 3, 1, 2)
    assert np.array_equal(y, oracle.conv2_naive(x, w, (1, 0), (2, 1), (1, 2)))


def test_pool(golden):
    for c in golden.meta["pool"]:
        shape = tuple(c["shape"])
        x = cycle(0, 10, int(np.prod(shape))).reshape(shape)
        y = oracle.max_pool2(x)
        assert np.array_equal(y, golden[c["name"] + "_y"])
        dy = np.arange(y.size, dtype=np.float32).reshape(y.shape)
        assert np.array_equal(oracle.max_pool2_backward(x, dy), golden[c["name"] + "_dx"])


def test_pool_backward_keeps_uncovered_cells():
    # A 5x5 input with a 2x2 window leaves row / column 4 uncovered: they keep x's values.
    x = np.arange(25, dtype=np.float32).reshape(1, 1, 5, 5)
    dy = np.ones((1, 1, 2, 2), np.float32)
    dx = oracle.max_pool2_backward(x, dy)
    assert np.array_equal(dx[0, 0, 4, :], x[0, 0, 4, :])
    assert np.array_equal(dx[0, 0, :, 4], x[0, 0, :, 4])
    assert dx[0, 0, :4, :4].sum() == 4


def test_relu(golden):
    for c in golden.meta["relu"]:
        shape = tuple(c["shape"])
        n = shape[0] * shape[1]
        x = cycle(-10, 10, n).reshape(shape)
        assert np.array_equal(oracle.relu(x), golden[c["name"] + "_y"])
        xb = cycle(-1, 1, n).reshape(shape)
        dy = np.arange(n, dtype=np.float32).reshape(shape)
        assert np.array_equal(oracle.relu_backward(xb, dy), golden[c["name"] + "_dx"])
    # -0.0 passes through, NaN becomes 0 (x >= 0 ? x : 0)
    y = oracle.relu(np.array([-0.0, np.nan, -1.0, 2.0], np.float32))
    assert np.signbit(y[0]) and y[1] == 0 and y[2] == 0 and y[3] == 2


def test_criterion(golden):
    for c in golden.meta["criterion"]:
        bs, classes = c["bs"], c["classes"]
        x = cycle(0, 10, bs * classes).reshape(bs, classes)
        t = (np.arange(bs) % classes).astype(np.uint32)
        loss = oracle.cross_entropy_loss(x, t)
        # the reference's own tolerance for f32: bs * f32::EPSILON, relative
        assert abs(loss - c["loss"]) <= max(abs(c["loss"]), 1.0) * bs * 1.2e-7 + 1e-5
        dx = oracle.cross_entropy_loss_backward(x, t, 1.0)
        np.testing.assert_allclose(dx, golden[c["name"] + "_dx"], rtol=2e-6, atol=1e-9)
        xa = ((np.arange(bs * classes) + classes // 2 + 1) % classes).astype(np.float32)
        assert oracle.accuracy(xa.reshape(bs, classes), t) == c["correct"]


def test_axpy_and_colsum(golden):
    for c in golden.meta["axpy"]:
        n = c["n"]
        out = oracle.scaled_add(2.0, cycle(1, 10, n), cycle(11, 20, n))
        assert np.array_equal(out, golden[c["name"]])
    for c in golden.meta["colsum"]:
        x = cycle(1, 16, c["rows"] * c["cols"] * c["inner"]).reshape(c["rows"], c["cols"], c["inner"])
        for acc64 in (False, True):
            assert np.array_equal(oracle.bias_grad(x, acc64=acc64), golden[c["name"]])


def test_sgd():
    w = np.array([1.0, -2.0, 0.5], np.float32)
    g = np.array([0.5, 0.25, -1.0], np.float32)
    assert np.array_equal(oracle.sgd_update(w, g, 0.5), w - 0.5 * g)
    v = np.array([1.0, 0.0, -1.0], np.float32)
    w2, v2 = oracle.sgd_update_momentum(w, g, v, 0.5, 0.25)
    vv = np.float32(0.25) * v + g
    assert np.array_equal(v2, vv) and np.array_equal(w2, w - np.float32(0.5) * vv)


def test_bf16_rounding():
    x = np.array([1.0, 1.00390625, 1.01171875, 3.14159265, -2.71828], np.float32)
    import torch
    expect = torch.tensor(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(oracle.round_bf16(x), expect)
    rng = np.random.default_rng(0)
    y = rng.standard_normal(10000).astype(np.float32)
    assert np.array_equal(oracle.round_bf16(y), torch.tensor(y).to(torch.bfloat16).float().numpy())


def test_lenet5_against_torch_f64():
    """The composed network and its training step agree with an independent torch f64 model."""
    import torch
    import torch.nn.functional as F
    from oracle import models
    P = models.init_params(models.LENET5, 2000)
    assert sum(p.size for p in P) == 46920
    x = np.random.default_rng(4000).uniform(0, 1, (100, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(4001).integers(0, 10, 100).astype(np.uint32)
    loss, grads, new_p, _ = models.train_step(models.LENET5, P, x, t, 0.01)
    tp = [torch.tensor(p, dtype=torch.float64, requires_grad=True) for p in P]
    h = torch.tensor(x, dtype=torch.float64)
    h = F.max_pool2d(torch.relu(F.conv2d(h, tp[0])), 2)
    h = F.max_pool2d(torch.relu(F.conv2d(h, tp[1])), 2).flatten(1)
    h = torch.relu(h @ tp[2])
    h = torch.relu(h @ tp[3])
    h = h @ tp[4] + tp[5]
    L = F.cross_entropy(h, torch.tensor(t.astype(np.int64)), reduction="sum")
    (L / 100).backward()
    assert abs(loss - L.item()) < 1e-3
    for g, p in zip(grads, tp):
        ref = p.grad.numpy()
        assert np.abs(g - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-8
    for w, g, nw in zip(P, grads, new_p):
        assert np.array_equal(nw, np.float32(-0.01) * g + w)


def test_direct_conv_backward_matches_the_plain_loops():
    """conv_direct.rs backward kernels restated (order of accumulation: blocks of 8 output
    channels, tiles of 7 positions, per-thread partial sums) against the naive loops on random
    data: same values up to f32 rounding, for LeNet5's two layers and a ragged shape."""
    rng = np.random.default_rng(12)
    for bs, ic, ih, iw, oc, f in [(9, 1, 28, 28, 6, 5), (5, 6, 12, 12, 16, 5), (4, 11, 9, 10, 19, 3)]:
        x = rng.standard_normal((bs, ic, ih, iw)).astype(np.float32)
        w = rng.standard_normal((oc, ic, f, f)).astype(np.float32)
        dy = rng.standard_normal((bs, oc, ih - f + 1, iw - f + 1)).astype(np.float32)
        dx64 = oracle.conv2_backward_input_naive(w, dy, (ih, iw), acc64=True)
        dw64 = oracle.conv2_backward_weight_naive(x, dy, (f, f), acc64=True)
        dx = oracle.conv2_direct_backward_input_f32(w, dy, (ih, iw))
        assert np.abs(dx - dx64).max() <= 1e-5 * np.sqrt(oc * f * f) * np.abs(dx64).max()
        for threads in (1, 4, 16):
            dw = oracle.conv2_direct_backward_weight_f32(x, dy, (f, f), threads=threads)
            assert np.abs(dw - dw64).max() <= 1e-5 * np.sqrt(bs * ih * iw) * np.abs(dw64).max()
