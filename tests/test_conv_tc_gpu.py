"""GPU: the tensor-core (tcgen05 implicit-GEMM) bf16 convolution against the oracle's naive
convolution -- forward with the fused bias + ReLU epilogue, and the input gradient."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

SHAPES = [
    # bs, ic, ih, iw, oc, f, pad      every one large enough for the tensor-core kernel
    (8, 64, 31, 31, 128, 3, 0),      # the wide stack's second layer (4 x 32 pixel tiles)
    (5, 40, 30, 37, 72, 3, 0),       # channel counts that need zero padding to 64 / 128
    (6, 32, 28, 28, 32, 5, 2),       # 5x5 filter with "same" padding, 64-wide accumulator
    (4, 64, 40, 40, 300, 3, 1),      # two 256-wide output-channel blocks, the second ragged
    (5, 96, 14, 150, 64, 3, 0),      # wide rows: 1 x 128 pixel tiles, two channel blocks
    (70, 128, 9, 9, 64, 3, 1),       # small images: 8 x 16 tiles hanging over both edges
    (3, 3, 64, 64, 64, 3, 0),        # the wide stack's first layer: 3 channels padded to 64
]


WGRAD_SHAPES = SHAPES + [
    (16, 3, 64, 64, 64, 3, 0),       # the wide stack's first layer: 3 channels padded to 64
    (12, 130, 20, 20, 40, 3, 1),     # three blocks of input channels, 40 output channels
    (12, 64, 24, 24, 96, 5, 0),      # 5x5: five taps per CTA
]


def _ints(rng, shape, lo, hi):
    return rng.integers(lo, hi + 1, shape).astype(np.float32)


@pytest.mark.parametrize("shape", SHAPES)
def test_conv_tc_exact_on_small_integers(dev, shape):
    """With small integer inputs every product and sum is exact in f32, so the result must
    equal the oracle's, rounded once to bf16, bit for bit (forward and input gradient)."""
    bs, ic, ih, iw, oc, f, pad = shape
    rng = np.random.default_rng(900 + ic + oc)
    x = _ints(rng, (bs, ic, ih, iw), -2, 2)
    w = _ints(rng, (oc, ic, f, f), -1, 1)
    kw = dict(padding=(pad, pad))
    y_ref = oracle.conv2_naive(x, w, **kw)
    xd, wd = dev.tensor(x, torch.bfloat16), dev.tensor(w, torch.bfloat16)
    y = dev.conv2_forward(xd, wd, **kw).float().cpu().numpy()
    assert np.array_equal(y, oracle.round_bf16(y_ref))
    dy = _ints(rng, y_ref.shape, -2, 2)
    dx_ref = oracle.conv2_backward_input_naive(w, dy, (ih, iw), **kw)
    dx = dev.conv2_backward_input(wd, dev.tensor(dy, torch.bfloat16), (ih, iw), **kw)
    assert np.array_equal(dx.float().cpu().numpy(), oracle.round_bf16(dx_ref))
    dev.wait()   # raises if a bounded device-side wait gave up


@pytest.mark.parametrize("shape", SHAPES[:4])
def test_conv_tc_random_vs_oracle(dev, shape):
    """bf16 inputs, f32 accumulation: within 1e-2 of an f64 host convolution; the fused
    bias + ReLU epilogue equals the separate bias_add and relu calls bit for bit."""
    bs, ic, ih, iw, oc, f, pad = shape
    rng = np.random.default_rng(950 + ic + oc)
    a = np.sqrt(2.0 / (ic * f * f))
    x = oracle.round_bf16(rng.standard_normal((bs, ic, ih, iw)).astype(np.float32))
    w = oracle.round_bf16(rng.uniform(-a, a, (oc, ic, f, f)).astype(np.float32))
    bias = oracle.round_bf16(rng.uniform(-a, a, oc).astype(np.float32))
    kw = dict(padding=(pad, pad))

    def close(got, ref):
        err = np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30)
        assert err <= 1e-2, err

    xd, wd, bd = (dev.tensor(t, torch.bfloat16) for t in (x, w, bias))
    y = dev.conv2_forward(xd, wd, **kw)
    close(y.float().cpu().numpy(), oracle.conv2_naive(x, w, acc64=True, **kw).astype(np.float64))
    fused = dev.conv2_forward(xd, wd, bias=bd, relu=True, **kw)
    assert torch.equal(fused, dev.relu(dev.bias_add(y, bd)))
    dy = oracle.round_bf16(rng.standard_normal(y.shape).astype(np.float32))
    dx = dev.conv2_backward_input(wd, dev.tensor(dy, torch.bfloat16), (ih, iw), **kw)
    close(dx.float().cpu().numpy(),
          oracle.conv2_backward_input_naive(w, dy, (ih, iw), acc64=True, **kw).astype(np.float64))
    dev.wait()


@pytest.mark.parametrize("shape", WGRAD_SHAPES)
def test_conv_tc_weight_gradient(dev, shape):
    """dw on the tensor cores: exact on small integers (every partial sum is an integer below
    2^24), beta = 1 accumulates into an existing gradient, and random data stays within 1e-2
    of an f64 host reduction."""
    bs, ic, ih, iw, oc, f, pad = shape
    rng = np.random.default_rng(990 + ic + oc)
    kw = dict(padding=(pad, pad))
    oh, ow = oracle.conv2_output_shape(ih, iw, (f, f), **kw)
    x = _ints(rng, (bs, ic, ih, iw), -2, 2)
    dy = _ints(rng, (bs, oc, oh, ow), -2, 2)
    ref = oracle.conv2_backward_weight_naive(x, dy, (f, f), **kw)
    xd, dyd = dev.tensor(x, torch.bfloat16), dev.tensor(dy, torch.bfloat16)
    dw = dev.conv2_backward_weight(xd, dyd, (f, f), **kw)
    assert np.array_equal(dw.float().cpu().numpy(), oracle.round_bf16(ref))
    ones = dev.tensor(np.ones_like(ref), torch.bfloat16)
    dw2 = dev.conv2_backward_weight(xd, dyd, (f, f), beta=1.0, dw=ones, **kw)
    assert np.array_equal(dw2.float().cpu().numpy(), oracle.round_bf16(ref + 1.0))
    xr = oracle.round_bf16(rng.standard_normal(x.shape).astype(np.float32))
    dyr = oracle.round_bf16(rng.standard_normal(dy.shape).astype(np.float32))
    ref64 = oracle.conv2_backward_weight_naive(xr, dyr, (f, f), acc64=True, **kw).astype(np.float64)
    got = dev.conv2_backward_weight(dev.tensor(xr, torch.bfloat16), dev.tensor(dyr, torch.bfloat16),
                                    (f, f), **kw).float().cpu().numpy()
    assert np.abs(got - ref64).max() / np.abs(ref64).max() <= 1e-2
    dev.wait()
