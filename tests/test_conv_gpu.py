"""GPU: convolution entry points against the reference's conv vectors and the oracle."""
import numpy as np
import pytest
import torch

import oracle
from conftest import cycle

pytestmark = pytest.mark.gpu


def _kw(c):
    return dict(padding=tuple(c["padding"]), stride=tuple(c["stride"]), dilation=tuple(c["dilation"]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2_golden(dev, golden, dtype):
    """conv2_im2col_<T>_<options> and the direct-conv backward tests
    (tests/integration_tests.rs:884-1034, 1182-1497): inputs cycle 1..=10."""
    cases = golden.meta["conv"]
    step = 1 if dtype == torch.float32 else 4
    for c in cases[::step]:
        bs, ic, ih, iw = c["x_shape"]
        f = tuple(c["filter"])
        x = cycle(1, 11, bs * ic * ih * iw).reshape(bs, ic, ih, iw)
        w = cycle(1, 11, c["oc"] * ic * f[0] * f[1]).reshape(c["oc"], ic, *f)
        y_true = golden[c["name"] + "_y"]
        dy = cycle(1, 11, y_true.size).reshape(y_true.shape)
        xd, wd, dyd = dev.tensor(x, dtype), dev.tensor(w, dtype), dev.tensor(dy, dtype)
        y = dev.conv2_forward(xd, wd, **_kw(c)).float().cpu().numpy()
        dx = dev.conv2_backward_input(wd, dyd, (ih, iw), **_kw(c)).float().cpu().numpy()
        dw = dev.conv2_backward_weight(xd, dyd, f, **_kw(c)).float().cpu().numpy()
        if dtype == torch.float32:
            assert np.array_equal(y, y_true), c
            assert np.array_equal(dx, golden[c["name"] + "_dx"]), c
            assert np.array_equal(dw, golden[c["name"] + "_dw"]), c
        else:
            # integer sums are exact in the f32 accumulator; one bf16 rounding at the store
            assert np.array_equal(y, oracle.round_bf16(y_true)), c
            assert np.array_equal(dx, oracle.round_bf16(golden[c["name"] + "_dx"])), c
            assert np.array_equal(dw, oracle.round_bf16(golden[c["name"] + "_dw"])), c


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2_full_reference_grid(dev, golden, dtype):
    """Every case of the reference's grid (7 filters x 7 option sets x 10 (bs, ic, oc) x 16 output
    shapes, tests/integration_tests.rs:884-923).  The expected tensors come from the oracle, which
    the CPU suite pins on this grid's fingerprints; f32 must equal them, bf16 after one rounding."""
    grid = golden["conv_grid"]
    step = 1 if dtype == torch.float32 else 5
    for row in grid[::step]:
        bs, ic, ih, iw, oc, fh, fw = (int(v) for v in row[:7])
        kw = dict(padding=(int(row[7]), int(row[8])), stride=(int(row[9]), int(row[10])),
                  dilation=(int(row[11]), int(row[12])))
        x = cycle(1, 11, bs * ic * ih * iw).reshape(bs, ic, ih, iw)
        w = cycle(1, 11, oc * ic * fh * fw).reshape(oc, ic, fh, fw)
        y_true = oracle.conv2_naive(x, w, **kw)
        dy = cycle(1, 11, y_true.size).reshape(y_true.shape)
        want = [y_true, oracle.conv2_backward_input_naive(w, dy, (ih, iw), **kw),
                oracle.conv2_backward_weight_naive(x, dy, (fh, fw), **kw)]
        xd, wd, dyd = (torch.from_numpy(a).to(dtype).to(dev.torch_device, non_blocking=True)
                       for a in (x, w, dy))
        got = [dev.conv2_forward(xd, wd, **kw), dev.conv2_backward_input(wd, dyd, (ih, iw), **kw),
               dev.conv2_backward_weight(xd, dyd, (fh, fw), **kw)]
        for g, t in zip(got, want):
            if dtype == torch.bfloat16:
                t = oracle.round_bf16(t)
            assert np.array_equal(g.float().cpu().numpy(), t), row.tolist()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_im2col_col2im_golden(dev, golden, dtype):
    """im2col_conv2_<T>_* / col2im_conv2_<T>_* (tests/integration_tests.rs:1499-1552)."""
    cases = golden.meta["im2col"]
    step = 1 if dtype == torch.float32 else 4
    for c in cases[::step]:
        bs, ch, ih, iw = c["x_shape"]
        f = tuple(c["filter"])
        n = bs * ch * ih * iw
        if dtype == torch.bfloat16 and n > 256:
            continue  # 1..len is not representable in bf16 beyond 256
        x = np.arange(1, n + 1, dtype=np.float32).reshape(bs, ch, ih, iw)
        y = dev.im2col_conv2(dev.tensor(x, dtype), f, **_kw(c)).float().cpu().numpy()
        y_true = golden[c["name"] + "_y"]
        assert np.array_equal(y, y_true), c
        if dtype == torch.bfloat16 and y.size > 256:
            continue
        dy = np.arange(1, y.size + 1, dtype=np.float32).reshape(y.shape)
        dx = dev.col2im_conv2(dev.tensor(dy, dtype), c["grid"], f, **_kw(c)).float().cpu().numpy()
        want = golden[c["name"] + "_dx"]
        if dtype == torch.bfloat16:
            want = oracle.round_bf16(want)
        assert np.array_equal(dx, want), c


SHAPES = [
    # (bs, ic, ih, iw, oc, fh, fw)  -- LeNet5 and wide-stack layers at small batch
    (16, 1, 28, 28, 6, 5, 5), (16, 6, 12, 12, 16, 5, 5), (2, 3, 64, 64, 64, 3, 3),
    (2, 64, 31, 31, 128, 3, 3), (3, 5, 9, 11, 7, 3, 2),
    # several images per CTA in the direct forward / backward kernels, ragged last group
    (601, 6, 12, 12, 16, 5, 5), (303, 1, 28, 28, 6, 5, 5), (5, 2, 10, 8, 3, 3, 3),
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv2_random_vs_oracle(dev, shape, dtype):
    bs, ic, ih, iw, oc, fh, fw = shape
    rng = np.random.default_rng(5000 + ic + oc)
    x = rng.standard_normal((bs, ic, ih, iw)).astype(np.float32)
    a = np.sqrt(2.0 / (ic * fh * fw))
    w = rng.uniform(-a, a, (oc, ic, fh, fw)).astype(np.float32)
    bias = rng.uniform(-a, a, oc).astype(np.float32)
    bf = dtype == torch.bfloat16
    if bf:
        x, w, bias = oracle.round_bf16(x), oracle.round_bf16(w), oracle.round_bf16(bias)
    K = ic * fh * fw
    tol = 1e-2 if bf else 1e-5 * np.sqrt(K)

    def close(got, ref, k):
        t = 1e-2 if bf else 1e-5 * np.sqrt(k)
        err = np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30)
        assert err <= t, err

    xd, wd, bd = dev.tensor(x, dtype), dev.tensor(w, dtype), dev.tensor(bias, dtype)
    y_ref = oracle.conv2_naive(x, w, acc64=True)
    y = dev.conv2_forward(xd, wd).float().cpu().numpy()
    close(y, y_ref.astype(np.float64), K)
    # fused bias + relu equals the unfused sequence bit for bit
    y_fused = dev.conv2_forward(xd, wd, bias=bd, relu=True)
    y_seq = dev.relu(dev.bias_add(dev.conv2_forward(xd, wd), bd))
    assert torch.equal(y_fused, y_seq)
    dy = rng.standard_normal(y.shape).astype(np.float32)
    if bf:
        dy = oracle.round_bf16(dy)
    dyd = dev.tensor(dy, dtype)
    dx = dev.conv2_backward_input(wd, dyd, (ih, iw)).float().cpu().numpy()
    close(dx, oracle.conv2_backward_input_naive(w, dy, (ih, iw), acc64=True).astype(np.float64),
          oc * fh * fw)
    dw = dev.conv2_backward_weight(xd, dyd, (fh, fw)).float().cpu().numpy()
    close(dw, oracle.conv2_backward_weight_naive(x, dy, (fh, fw), acc64=True).astype(np.float64),
          bs * y.shape[2] * y.shape[3])
    # accumulate into an existing gradient (second edge into the same node)
    dw2 = dev.conv2_backward_weight(xd, dyd, (fh, fw), beta=1.0,
                                    dw=dev.tensor(np.ones_like(w), dtype)).float().cpu().numpy()
    close(dw2, dw.astype(np.float64) + 1.0, bs * y.shape[2] * y.shape[3])


def test_conv2_equals_im2col_gemm(dev):
    """The implicit GEMM equals the reference's im2col -> dot -> permute sequence."""
    rng = np.random.default_rng(9)
    x = dev.tensor(rng.integers(-3, 4, (4, 3, 10, 9)).astype(np.float32))
    w = dev.tensor(rng.integers(-3, 4, (5, 3, 3, 3)).astype(np.float32))
    kw = dict(padding=(1, 0), stride=(2, 1), dilation=(1, 2))
    y = dev.conv2_forward(x, w, **kw)
    im = dev.im2col_conv2(x, (3, 3), **kw)
    oh, ow = y.shape[2:]
    y2 = dev.dot(im, w.reshape(5, -1).T).reshape(4, oh, ow, 5).permute(0, 3, 1, 2)
    assert torch.equal(y, y2.contiguous())


def test_conv2_errors(dev):
    import autograph_b200 as ag
    x = dev.empty((1, 2, 4, 4), torch.float32)
    with pytest.raises(ag.AgError):
        dev.conv2_forward(x, dev.empty((3, 1, 3, 3), torch.float32))      # channel mismatch
    with pytest.raises(ag.AgError):
        dev.conv2_forward(x, dev.empty((3, 2, 5, 5), torch.float32))      # filter larger than input
    assert dev.conv2_forward(dev.empty((0, 2, 4, 4), torch.float32),
                             dev.empty((3, 2, 3, 3), torch.float32)).shape == (0, 3, 2, 2)
