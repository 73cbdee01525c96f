"""GPU: the inference fusions (conv+relu+pool, dense+bias+relu) equal the separate
operator calls bit for bit, and match the oracle."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _prep(a, dtype):
    return oracle.round_bf16(a.astype(np.float32)) if dtype == torch.bfloat16 else a.astype(np.float32)


CONV_SHAPES = [
    # bs, ic, ih, iw, oc, fh, fw, pool      (first four take the direct kernel)
    (37, 1, 28, 28, 6, 5, 5, (2, 2)), (37, 6, 12, 12, 16, 5, 5, (2, 2)),
    (3, 3, 64, 64, 64, 3, 3, (2, 2)), (1000, 1, 28, 28, 6, 5, 5, (2, 2)),
    (2, 64, 31, 31, 128, 3, 3, (2, 2)), (3, 5, 9, 11, 7, 3, 2, (2, 3)), (4, 2, 10, 10, 8, 3, 3, (3, 3)),
    # many output channels: the banded direct kernel, with and without aligned runs
    (5, 3, 20, 22, 34, 3, 3, (2, 2)), (3, 2, 16, 16, 48, 5, 5, (2, 2)),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", CONV_SHAPES)
def test_conv_relu_pool_equals_separate_calls(dev, dtype, shape):
    bs, ic, ih, iw, oc, fh, fw, pool = shape
    rng = np.random.default_rng(31 + ic + oc)
    x = _prep(rng.standard_normal((bs, ic, ih, iw)), dtype)
    a = np.sqrt(2.0 / (ic * fh * fw))
    w = _prep(rng.uniform(-a, a, (oc, ic, fh, fw)), dtype)
    b = _prep(rng.uniform(-a, a, oc), dtype)
    xd, wd, bd = dev.tensor(x, dtype), dev.tensor(w, dtype), dev.tensor(b, dtype)
    for bias in (None, bd):
        for relu in (True, False):
            fused = dev.conv2_relu_max_pool2(xd, wd, bias=bias, relu=relu, pool=pool)
            y = dev.conv2_forward(xd, wd)
            if bias is not None:
                y = dev.bias_add(y, bias)
            if relu:
                y = dev.relu(y)
            sep = dev.max_pool2(y, pool)
            assert torch.equal(fused, sep), (shape, bias is not None, relu)
        if pool == (2, 2):  # the gradient-recording form keeps the convolution's output
            pre, kept = dev.conv2_relu_max_pool2_keep(xd, wd, bias=bias)
            assert torch.equal(pre, dev.conv2_forward(xd, wd, bias=bias)), (shape, bias is not None)
            assert torch.equal(kept, dev.max_pool2(dev.relu(pre), pool)), (shape, bias is not None)
    # against the oracle (f64 accumulation): tolerance of the convolution
    ref = oracle.max_pool2(oracle.relu(oracle.conv2_naive(x, w, acc64=True)), pool)
    got = dev.conv2_relu_max_pool2(xd, wd, pool=pool).float().cpu().numpy()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5 * np.sqrt(ic * fh * fw)
    assert np.abs(got - ref).max() <= tol * max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1000, 256, 128), (1000, 128, 84), (1000, 84, 10), (100, 256, 128),
                                   (7, 5, 3), (256, 25088, 512), (300, 512, 10), (512, 512, 512)])
def test_dense_forward_equals_separate_calls(dev, dtype, shape):
    bs, ins, outs = shape
    rng = np.random.default_rng(41 + outs)
    x = _prep(rng.standard_normal((bs, ins)), dtype)
    a = np.sqrt(2.0 / ins)
    w = _prep(rng.uniform(-a, a, (ins, outs)), dtype)
    b = _prep(rng.uniform(-a, a, outs), dtype)
    xd, wd, bd = dev.tensor(x, dtype), dev.tensor(w, dtype), dev.tensor(b, dtype)
    for bias in (None, bd):
        for relu in (False, True):
            fused = dev.dense_forward(xd, wd, bias=bias, relu=relu)
            y = dev.dot(xd, wd)
            if bias is not None:
                y = dev.bias_add(y, bias)
            if relu:
                y = dev.relu(y)
            assert torch.equal(fused, y), (shape, bias is not None, relu)
    ref = x.astype(np.float64) @ w.astype(np.float64) + b
    got = dev.dense_forward(xd, wd, bias=bd).float().cpu().numpy()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5 * np.sqrt(ins)
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [(1000, [256, 128, 84, 10]), (37, [256, 128, 84, 10]),
                                  (5, [7, 3, 9]), (256, [25088, 512, 10]), (9000, [64, 32, 16])])
def test_dense_chain_equals_separate_calls(dev, dtype, case):
    bs, widths = case
    rng = np.random.default_rng(51 + bs)
    x = _prep(rng.standard_normal((bs, widths[0])), dtype)
    ws, bs_, relus = [], [], []
    for i in range(len(widths) - 1):
        a = np.sqrt(2.0 / widths[i])
        ws.append(dev.tensor(_prep(rng.uniform(-a, a, (widths[i], widths[i + 1])), dtype), dtype))
        last = i == len(widths) - 2
        bs_.append(dev.tensor(_prep(rng.uniform(-a, a, widths[i + 1]), dtype), dtype) if last else None)
        relus.append(not last)
    xd = dev.tensor(x, dtype)
    fused = dev.dense_chain_forward(xd, ws, bs_, relus)
    pre, act = dev.dense_chain_forward_keep(xd, ws, bs_, relus)
    h = xd
    for i, (w, b, r) in enumerate(zip(ws, bs_, relus)):
        p = dev.dense_forward(h, w, bias=b, relu=False)
        assert torch.equal(pre[i], p), i  # the values a gradient-recording pass keeps
        h = dev.dense_forward(h, w, bias=b, relu=r)
        if r:
            assert torch.equal(act[i], h), i
        else:
            assert act[i] is None
    assert torch.equal(fused, h)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [(100, [256, 128, 84, 10], True), (37, [256, 128, 84, 10], False),
                                  (5, [7, 3, 9], True), (300, [64, 32, 16], True),
                                  (600, [64, 32, 16], True), (100, [40, 12], True)])
def test_dense_chain_backward_equals_separate_calls(dev, dtype, case):
    """One call gives the gradients of the layer-by-layer edges (products within the GEMM
    tolerance, gates and zeros exactly)."""
    bs, widths, want_dx = case
    rng = np.random.default_rng(77 + bs)
    n = len(widths) - 1
    x = dev.tensor(_prep(rng.standard_normal((bs, widths[0])), dtype), dtype)
    ws = [dev.tensor(_prep(rng.uniform(-0.3, 0.3, (widths[i], widths[i + 1])), dtype), dtype)
          for i in range(n)]
    relus = [i < n - 1 for i in range(n)] if len(widths) != 3 else [True, True]
    has_bias = [i == n - 1 for i in range(n)]
    pre, act = dev.dense_chain_forward_keep(x, ws, None, relus)
    dy = dev.tensor(_prep(rng.standard_normal((bs, widths[-1])), dtype), dtype)
    dx, dw, db, g = dev.dense_chain_backward(x, ws, relus, pre, act, dy, has_bias, want_dx)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4

    def close(a, b):
        a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
        return np.abs(a - b).max() <= tol * max(np.abs(b).max(), 1e-6)

    incoming = dy
    for l in range(n - 1, -1, -1):
        gl = dev.relu_backward(pre[l], incoming) if relus[l] else incoming
        if relus[l] or l < n - 1:
            assert close(g[l], gl), l
            assert torch.equal(g[l] == 0, gl == 0) or dtype == torch.bfloat16
        lin = x if l == 0 else (act[l - 1] if relus[l - 1] else pre[l - 1])
        assert close(dw[l], dev.dot(lin.T, gl)), l
        if has_bias[l]:
            assert close(db[l], dev.bias_grad(gl)), l
        incoming = dev.dot(gl, ws[l].T)
    if want_dx:
        assert close(dx, incoming)
    else:
        assert dx is None


NETS = [
    # bs, (ic, ih, iw), conv stages [(oc, f, relu, pool)], dense widths after the flatten
    (1000, (1, 28, 28), [(6, 5, True, (2, 2)), (16, 5, True, (2, 2))], [120, 84, 10]),   # LeNet5
    (9, (1, 28, 28), [(6, 5, True, (2, 2)), (16, 5, True, (2, 2))], [120, 84, 10]),
    (7, (1, 28, 28), [(6, 5, True, (2, 2)), (16, 5, True, (2, 2))], [120, 84, 10]),
    (1, (1, 28, 28), [(6, 5, True, (2, 2)), (16, 5, True, (2, 2))], [120, 84, 10]),
    (21, (3, 12, 14), [(5, 3, True, (2, 2))], [33, 7]),               # one 3x3 stage, odd widths
    (18, (2, 10, 10), [(4, 3, False, None), (7, 3, True, (2, 2))], [10]),  # no pool, no relu
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("net", NETS)
def test_conv_dense_chain_equals_separate_calls(dev, dtype, net):
    """The one-kernel form of a small network gives the bits of the layer-by-layer calls."""
    bs, (ic, ih, iw), convs, widths = net
    rng = np.random.default_rng(77 + bs)
    x = dev.tensor(_prep(rng.uniform(0, 1, (bs, ic, ih, iw)), dtype), dtype)
    stages, c, h, w = [], ic, ih, iw
    for oc, f, relu, pool in convs:
        a = np.sqrt(2.0 / (c * f * f))
        wt = dev.tensor(_prep(rng.uniform(-a, a, (oc, c, f, f)), dtype), dtype)
        b = dev.tensor(_prep(rng.uniform(-a, a, oc), dtype), dtype)
        stages.append((wt, b, relu, pool))
        c, h, w = oc, h - f + 1, w - f + 1
        if pool:
            h, w = h // 2, w // 2
    dims = [c * h * w] + widths
    ws, bs_, relus = [], [], []
    for i in range(len(dims) - 1):
        a = np.sqrt(2.0 / dims[i])
        ws.append(dev.tensor(_prep(rng.uniform(-a, a, (dims[i], dims[i + 1])), dtype), dtype))
        bs_.append(dev.tensor(_prep(rng.uniform(-a, a, dims[i + 1]), dtype), dtype))
        relus.append(i < len(dims) - 2)
    fused = dev.conv_dense_chain_forward(x, stages, ws, bs_, relus)
    v = x
    for wt, b, relu, pool in stages:
        v = dev.conv2_forward(v, wt, bias=b, relu=relu)
        if pool:
            v = dev.max_pool2(v, pool)
    v = v.reshape(bs, -1)
    for wd, b, r in zip(ws, bs_, relus):
        v = dev.dense_forward(v, wd, bias=b, relu=r)
    assert torch.equal(fused, v)


@pytest.mark.parametrize("dtype,tensor_cores", [(torch.float32, False), (torch.bfloat16, False),
                                                 (torch.bfloat16, True)])
@pytest.mark.parametrize("bs", [1, 6, 7, 8, 50, 1000, 1037, 9000])
def test_lenet5_geometry_kernel(dev, dtype, tensor_cores, bs, monkeypatch):
    """LeNet5 itself (no convolution bias) takes the kernels specialised for its geometry.  f32:
    the bits of the layer-by-layer calls.  bf16: the second convolution runs on the tensor
    cores, whose f32 sums are added in another order, so values agree within bf16 rounding (one
    rounding step at a layer boundary moves a logit by about 2^-8 of its size) and with an f64
    reference within the bf16 tolerance."""
    rng = np.random.default_rng(500 + bs)
    bf = dtype == torch.bfloat16
    # AG_LENET_TC=1 (read per call) selects the bf16 kernel whose conv2 is on tcgen05; batch 9000
    # takes the split form (the kernel stops after the flatten, dense layers over the batch)
    monkeypatch.setenv("AG_LENET_TC", "1" if tensor_cores else "0")
    xn = _prep(rng.uniform(0, 1, (bs, 1, 28, 28)), dtype)
    shapes = [(6, 1, 5, 5), (16, 6, 5, 5), (256, 120), (120, 84), (84, 10)]
    fan = [25, 150, 256, 120, 84]
    P = [_prep(rng.uniform(-1, 1, s) * np.sqrt(2.0 / f), dtype) for s, f in zip(shapes, fan)]
    bias = _prep(rng.uniform(-0.1, 0.1, 10), dtype)
    x = dev.tensor(xn, dtype)
    Pd = [dev.tensor(p, dtype) for p in P]
    bd = dev.tensor(bias, dtype)
    stages = [(Pd[0], None, True, (2, 2)), (Pd[1], None, True, (2, 2))]
    fused = dev.conv_dense_chain_forward(x, stages, Pd[2:], [None, None, bd], [True, True, False])
    v = x
    for wt, b, relu, pool in stages:
        v = dev.max_pool2(dev.conv2_forward(v, wt, bias=b, relu=relu), pool)
    v = v.reshape(bs, -1)
    for wd, b, r in zip(Pd[2:], [None, None, bd], [True, True, False]):
        v = dev.dense_forward(v, wd, bias=b, relu=r)
    if not tensor_cores:
        assert torch.equal(fused, v)
    else:
        scale = v.float().abs().max().item()
        assert (fused.float() - v.float()).abs().max().item() <= 2e-2 * scale
    # f64 reference of the same network
    h = torch.tensor(xn, dtype=torch.float64)
    rd = (lambda t: t.to(torch.bfloat16).to(torch.float64)) if bf else (lambda t: t.to(torch.float32).to(torch.float64))
    import torch.nn.functional as F
    for w in P[:2]:
        h = F.max_pool2d(torch.relu(rd(F.conv2d(h, torch.tensor(w, dtype=torch.float64)))), 2)
    h = h.reshape(bs, -1)
    h = torch.relu(rd(h @ torch.tensor(P[2], dtype=torch.float64)))
    h = torch.relu(rd(h @ torch.tensor(P[3], dtype=torch.float64)))
    h = rd(rd(h @ torch.tensor(P[4], dtype=torch.float64)) + torch.tensor(bias, dtype=torch.float64))
    tol = 1e-2 if bf else 1e-5 * np.sqrt(256)
    assert (fused.double().cpu() - h).abs().max().item() <= tol * h.abs().max().item()


def test_conv_dense_chain_unsupported(dev):
    """Networks the one-kernel form does not take are refused, not approximated."""
    import autograph_b200 as ag
    x = dev.empty((4, 1, 28, 28), torch.float32)
    w = dev.empty((6, 1, 4, 4), torch.float32)                       # 4x4 filter
    d = dev.empty((6 * 25 * 25, 10), torch.float32)
    with pytest.raises(ag.AgError) as e:
        dev.conv_dense_chain_forward(x, [(w, None, True, None)], [d])
    assert e.value.status == ag._capi.AG_ERR_UNSUPPORTED
    w5 = dev.empty((6, 1, 5, 5), torch.float32)
    wide = dev.empty((6 * 12 * 12, 4096), torch.float32)              # dense layer too wide
    with pytest.raises(ag.AgError):
        dev.conv_dense_chain_forward(x, [(w5, None, True, (2, 2))], [wide])


def test_fused_errors(dev):
    import autograph_b200 as ag
    x = dev.empty((2, 1, 6, 6), torch.float32)
    w = dev.empty((4, 1, 5, 5), torch.float32)
    with pytest.raises(ag.AgError):
        dev.conv2_relu_max_pool2(x, w, pool=(3, 3))       # conv output 2x2 < window
    with pytest.raises(ag.AgError, match="a_cols != b_rows"):
        dev.dense_forward(dev.empty((2, 3), torch.float32), dev.empty((4, 5), torch.float32))
