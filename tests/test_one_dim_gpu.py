"""GPU: the 1-D wrappers (Conv1, MaxPool1) are the 2-D operators on [n, c, l, 1], as in the
reference (layer.rs:1007-1033, 1173-1191); checked against the oracle's naive loops."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", [(4, 3, 50, 8, 5, 0, 1, 1), (3, 6, 33, 7, 3, 1, 2, 1),
                                  (2, 2, 40, 4, 4, 2, 1, 2)])
def test_conv1_matches_oracle(dev, case):
    n, c, l, oc, f, pad, stride, dil = case
    rng = np.random.default_rng(60 + l)
    x = rng.integers(-3, 4, (n, c, l)).astype(np.float32)
    w = rng.integers(-2, 3, (oc, c, f)).astype(np.float32)
    kw2 = dict(padding=(pad, 0), stride=(stride, 1), dilation=(dil, 1))
    y_ref = oracle.conv2_naive(x.reshape(n, c, l, 1), w.reshape(oc, c, f, 1), **kw2)
    xd, wd = dev.tensor(x), dev.tensor(w)
    y = dev.conv1_forward(xd, wd, padding=pad, stride=stride, dilation=dil)
    assert np.array_equal(y.cpu().numpy(), y_ref[..., 0])
    dy = rng.integers(-2, 3, y_ref.shape[:3]).astype(np.float32)
    dx = dev.conv1_backward_input(wd, dev.tensor(dy), l, padding=pad, stride=stride, dilation=dil)
    dx_ref = oracle.conv2_backward_input_naive(w.reshape(oc, c, f, 1), dy[..., None], (l, 1), **kw2)
    assert np.array_equal(dx.cpu().numpy(), dx_ref[..., 0])
    dw = dev.conv1_backward_weight(xd, dev.tensor(dy), f, padding=pad, stride=stride, dilation=dil)
    dw_ref = oracle.conv2_backward_weight_naive(x.reshape(n, c, l, 1), dy[..., None], (f, 1), **kw2)
    assert np.array_equal(dw.cpu().numpy(), dw_ref[..., 0])


def test_max_pool1_matches_oracle(dev):
    rng = np.random.default_rng(61)
    x = rng.standard_normal((5, 4, 37)).astype(np.float32)
    y = dev.max_pool1(dev.tensor(x), 3, 2).cpu().numpy()
    ref = oracle.max_pool2(x.reshape(5, 4, 37, 1), (3, 1), (2, 1))[..., 0]
    assert np.array_equal(y, ref)
