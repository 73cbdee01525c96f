"""GPU: the tcgen05 bf16 GEMM (shapes large and aligned enough for the tensor-core path)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _views(a, b, layout):
    return (a.T if layout[0] == "t" else a), (b.T if layout[1] == "t" else b)


def _operands(rng, m, k, n, layout):
    a = rng.uniform(-1, 1, (m, k) if layout[0] == "n" else (k, m)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n) if layout[1] == "n" else (n, k)).astype(np.float32)
    return oracle.round_bf16(a), oracle.round_bf16(b)


def _check(c, ref, tol=1e-2):
    # bf16 result within 1e-2 relative (to max|C|) of the f64 product; the rounding
    # of one bf16 store alone is 2^-9 = 2e-3 relative to the element.
    err = np.abs(c.astype(np.float64) - ref).max() / np.abs(ref).max()
    assert err <= tol, err
    # and element-wise: within bf16 half-ulp of the f64 value plus accumulation noise
    bound = np.abs(ref) * 2.0 ** -8 + 1e-3 * np.abs(ref).max()
    assert (np.abs(c.astype(np.float64) - ref) <= bound).all()


@pytest.mark.parametrize("layout", ["nt", "nn", "tn", "tt"])
@pytest.mark.parametrize("shape", [(128, 64, 256), (256, 256, 256), (384, 200, 520),
                                   (1024, 1024, 1024),
                                   # 84 tiles of 256x256 on 74 SM pairs: the 10 tiles of the
                                   # partial wave are cut into 2 pieces along n
                                   (3072, 256, 1792), (2560, 192, 2000)])
def test_bf16_vs_f64(dev, layout, shape):
    m, k, n = shape
    rng = np.random.default_rng(3000 + m + k)
    a, b = _operands(rng, m, k, n, layout)
    av, bv = _views(a, b, layout)
    ref = av.astype(np.float64) @ bv.astype(np.float64)
    ad, bd = dev.tensor(a, torch.bfloat16), dev.tensor(b, torch.bfloat16)
    c = dev.dot(*_views(ad, bd, layout)).float().cpu().numpy()
    dev.wait()
    _check(c, ref)


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_bf16_identity_exact(dev, layout):
    """A . I = A exactly: catches any mis-addressed tile or swizzle error."""
    m, k = 256, 512
    rng = np.random.default_rng(11)
    a = oracle.round_bf16(rng.uniform(-1, 1, (m, k) if layout[0] == "n" else (k, m)).astype(np.float32))
    eye = np.eye(k, dtype=np.float32)
    ad, bd = dev.tensor(a, torch.bfloat16), dev.tensor(eye, torch.bfloat16)
    av, bv = _views(ad, bd, layout)
    c = dev.dot(av, bv).float().cpu().numpy()
    assert np.array_equal(c, a if layout[0] == "n" else a.T)


def test_bf16_alpha_beta(dev):
    m, k, n = 256, 128, 512
    rng = np.random.default_rng(12)
    a = rng.integers(-2, 3, (m, k)).astype(np.float32)
    b = rng.integers(-2, 3, (k, n)).astype(np.float32)
    c0 = rng.integers(-4, 5, (m, n)).astype(np.float32)
    ad, bd, cd = (dev.tensor(v, torch.bfloat16) for v in (a, b, c0))
    dev.gemm(0.5, ad, bd, 2.0, cd)
    want = oracle.round_bf16((0.5 * (a @ b) + 2.0 * c0).astype(np.float32))
    assert np.array_equal(cd.float().cpu().numpy(), want)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_bf16_4096_sampled(dev, layout):
    n = 4096
    rng = np.random.default_rng(3012)
    a, b = _operands(rng, n, n, n, layout)
    av, bv = _views(a, b, layout)
    ad, bd = dev.tensor(a, torch.bfloat16), dev.tensor(b, torch.bfloat16)
    c = dev.dot(*_views(ad, bd, layout)).float().cpu().numpy()
    rows = rng.choice(n, 32, replace=False)
    ref = av[rows].astype(np.float64) @ bv.astype(np.float64)
    _check(c[rows], ref)
    cols = rng.choice(n, 32, replace=False)
    ref = av.astype(np.float64) @ bv[:, cols].astype(np.float64)
    _check(c[:, cols], ref)


@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
@pytest.mark.parametrize("shape", [(256, 25088, 512), (130, 4100, 264)])
def test_bf16_split_k(dev, layout, shape):
    """Few output tiles and a long k: slices of k become work items (f32 partial tiles, added
    in a fixed order).  Within 1e-2 of an f64 product, identical from run to run, and exact
    with alpha / beta on small integers."""
    m, k, n = shape
    rng = np.random.default_rng(4000 + m)
    a, b = _operands(rng, m, k, n, layout)
    av, bv = _views(a, b, layout)
    ref = av.astype(np.float64) @ bv.astype(np.float64)
    ad, bd = dev.tensor(a, torch.bfloat16), dev.tensor(b, torch.bfloat16)
    c1 = dev.dot(*_views(ad, bd, layout))
    c2 = dev.dot(*_views(ad, bd, layout))
    dev.wait()
    assert torch.equal(c1, c2)
    _check(c1.float().cpu().numpy(), ref)
    ai = rng.integers(-1, 2, a.shape).astype(np.float32)
    bi = rng.integers(-1, 2, b.shape).astype(np.float32)
    c0 = rng.integers(-4, 5, (m, n)).astype(np.float32)
    aiv, biv = _views(ai, bi, layout)
    cd = dev.tensor(c0, torch.bfloat16)
    dev.gemm(0.5, *_views(dev.tensor(ai, torch.bfloat16), dev.tensor(bi, torch.bfloat16), layout), 2.0, cd)
    want = oracle.round_bf16((0.5 * (aiv @ biv) + 2.0 * c0).astype(np.float32))
    assert np.array_equal(cd.float().cpu().numpy(), want)


@pytest.mark.parametrize("shape", [(512, 1024, 512), (192, 640, 384), (256, 25088, 512), (300, 520, 264)])
@pytest.mark.parametrize("with_bias,relu", [(True, True), (True, False), (False, True)])
def test_dense_epilogue_fused_on_the_tensor_cores(dev, shape, with_bias, relu):
    """Dense::forward (+ Relu) on the tcgen05 kernels: bias add and ReLU happen in the kernel's
    epilogue (paired-CTA kernel, one-CTA kernel, and the reduction of the k-split kernel).  The
    result equals the product, the bias add and the ReLU as three separate calls bit for bit, and
    an f64 reference within the bf16 tolerance."""
    import autograph_b200 as ag
    bs, ins, outs = shape
    rng = np.random.default_rng(bs + ins)
    x = oracle.round_bf16(rng.uniform(-1, 1, (bs, ins)).astype(np.float32))
    w = oracle.round_bf16(rng.uniform(-1, 1, (ins, outs)).astype(np.float32) / np.sqrt(ins))
    b = oracle.round_bf16(rng.uniform(-1, 1, outs).astype(np.float32))
    xd, wd, bd = (dev.tensor(a, torch.bfloat16) for a in (x, w, b))
    launches = ag.kernel_launch_count()
    y = dev.dense_forward(xd, wd, bias=bd if with_bias else None, relu=relu)
    fused_launches = ag.kernel_launch_count() - launches
    sep = dev.dot(xd, wd)
    if with_bias:
        sep = dev.bias_add(sep, bd)
    if relu:
        sep = dev.relu(sep, inplace=True)
    assert torch.equal(y, sep)
    assert fused_launches <= 2          # the product (and, when k is split, its reduction)
    ref = x.astype(np.float64) @ w.astype(np.float64)
    if with_bias:
        ref = ref + b
    if relu:
        ref = np.maximum(ref, 0)
    assert np.abs(y.float().cpu().numpy() - ref).max() <= 1e-2 * max(np.abs(ref).max(), 1e-6)
