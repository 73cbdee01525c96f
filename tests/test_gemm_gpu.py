"""GPU: ag_gemm / dot against the reference's tensor_dot vectors and the oracle."""
import itertools

import numpy as np
import pytest
import torch

import oracle
from conftest import cycle

pytestmark = pytest.mark.gpu


def _views(a, b, ta, tb):
    return (a.T if ta == "t" else a), (b.T if tb == "t" else b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tensor_dot_golden(dev, golden, dtype):
    """tensor_dot_<T>_m{n}_k{n}_n{n}_{nn,tn,nt,tt} (tests/integration_tests.rs:272-376)."""
    for n in [2, 4, 5, 8, 16, 32, 64, 128]:
        a = dev.tensor(cycle(1, 10, n * n).reshape(n, n), dtype)
        b = dev.tensor(cycle(1, 10, n * n).reshape(n, n), dtype)
        for ta, tb in itertools.product("nt", "nt"):
            av, bv = _views(a, b, ta, tb)
            c = dev.dot(av, bv).float().cpu().numpy()
            want = golden[f"dot_n{n}_{ta}{tb}"]
            if dtype == torch.bfloat16:
                want = oracle.round_bf16(want)  # f32 accumulation is exact here; one rounding
            assert np.array_equal(c, want), (n, ta, tb, dtype)


def _rel_err(c, ref):
    return float(np.abs(c.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.mark.parametrize("n", [256, 1024])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_f32_random_vs_oracle(dev, n, layout):
    """Uniform [-1,1) operands; max error relative to max|C| within 1e-5*sqrt(K)."""
    rng = np.random.default_rng(3000 + n)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    av, bv = _views(a, b, *layout)
    ref = av.astype(np.float64) @ bv.astype(np.float64)
    if n <= 256:
        ref_o = oracle.gemm(av, bv, acc="f64")
        assert _rel_err(ref_o, ref) < 1e-6
    ad, bd = dev.tensor(a), dev.tensor(b)
    c = dev.dot(*_views(ad, bd, *layout)).cpu().numpy()
    assert _rel_err(c, ref) <= 1e-5 * np.sqrt(n)


def test_f32_4096_sampled_rows(dev):
    n = 4096
    rng = np.random.default_rng(3012)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    ad, bd = dev.tensor(a), dev.tensor(b)
    rows = rng.choice(n, 48, replace=False)
    for layout in ["nn", "tn", "nt"]:
        av, bv = _views(a, b, *layout)
        c = dev.dot(*_views(ad, bd, *layout)).cpu().numpy()
        ref = av[rows].astype(np.float64) @ bv.astype(np.float64)
        assert _rel_err(c[rows], ref) <= 1e-5 * np.sqrt(n), layout
        # linearity: column checksum of C equals (1^T A) B
        chk = (av.astype(np.float64).sum(0) @ bv.astype(np.float64))
        assert np.abs(c.astype(np.float64).sum(0) - chk).max() <= 1e-5 * np.sqrt(n) * n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_alpha_beta_strides_offsets(dev, dtype):
    rng = np.random.default_rng(5)
    big_a = rng.integers(-3, 4, (40, 70)).astype(np.float32)
    big_b = rng.integers(-3, 4, (70, 50)).astype(np.float32)
    big_c = rng.integers(-3, 4, (45, 60)).astype(np.float32)
    ad, bd, cd = dev.tensor(big_a, dtype), dev.tensor(big_b, dtype), dev.tensor(big_c, dtype)
    # sub-views with offsets and non-unit column strides
    av, bv = ad[3:33, 5:65:2], bd[4:64:2, 1:49:3]       # 30x30, 30x16
    cv = cd[2:32, 7:39:2]                                # 30x16
    want = 2.0 * (big_a[3:33, 5:65:2] @ big_b[4:64:2, 1:49:3]) - 1.0 * big_c[2:32, 7:39:2]
    dev.gemm(2.0, av, bv, -1.0, cv)
    got = cd.float().cpu().numpy()
    expect = big_c.copy()
    expect[2:32, 7:39:2] = want
    assert np.array_equal(got, expect)  # small integers: exact in both types


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_split_k_and_skinny_shapes(dev, dtype):
    """The LeNet5 products the reference's author benchmarks (src/tensor/linalg.rs:507-519)."""
    rng = np.random.default_rng(6)
    shapes = [(57600, 25, 6, "nt"), (6400, 150, 16, "nt"), (100, 256, 128, "nn"),
              (100, 128, 84, "nn"), (100, 84, 10, "nn"), (100, 10, 84, "nt"), (84, 100, 10, "tn"),
              (128, 100, 84, "tn"), (256, 100, 128, "tn"), (16, 6400, 150, "tn"),
              (6, 57600, 25, "tn"), (3, 5000, 2, "nn")]
    for m, k, n, layout in shapes:
        a = rng.uniform(-1, 1, (m, k) if layout[0] == "n" else (k, m)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n) if layout[1] == "n" else (n, k)).astype(np.float32)
        if dtype == torch.bfloat16:
            a, b = oracle.round_bf16(a), oracle.round_bf16(b)
        av, bv = _views(a, b, *layout)
        ref = av.astype(np.float64) @ bv.astype(np.float64)
        c = dev.dot(*_views(dev.tensor(a, dtype), dev.tensor(b, dtype), *layout))
        c = c.float().cpu().numpy()
        tol = 1e-5 * np.sqrt(k) if dtype == torch.float32 else 1e-2
        assert _rel_err(c, ref) <= tol, (m, k, n, layout)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_short_reductions_all_layouts(dev, dtype, layout):
    """k <= 128 with few output tiles takes the kernel that stages the whole k range."""
    rng = np.random.default_rng(61)
    for m, k, n in [(1, 1, 1), (33, 7, 5), (100, 8, 84), (97, 33, 130), (84, 100, 10),
                    (256, 128, 128), (130, 127, 31)]:
        a = rng.uniform(-1, 1, (m, k) if layout[0] == "n" else (k, m)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n) if layout[1] == "n" else (n, k)).astype(np.float32)
        if dtype == torch.bfloat16:
            a, b = oracle.round_bf16(a), oracle.round_bf16(b)
        av, bv = _views(a, b, *layout)
        ref = av.astype(np.float64) @ bv.astype(np.float64)
        ad, bd = dev.tensor(a, dtype), dev.tensor(b, dtype)
        c1 = dev.dot(*_views(ad, bd, *layout)).float().cpu().numpy()
        c2 = dev.dot(*_views(ad, bd, *layout)).float().cpu().numpy()
        tol = 1e-5 * np.sqrt(k) if dtype == torch.float32 else 1e-2
        assert _rel_err(c1, ref) <= tol, (m, k, n)
        assert np.array_equal(c1, c2)


def test_split_k_is_deterministic(dev):
    rng = np.random.default_rng(7)
    a = dev.tensor(rng.uniform(-1, 1, (16, 6400)).astype(np.float32))
    b = dev.tensor(rng.uniform(-1, 1, (6400, 150)).astype(np.float32))
    c1 = dev.dot(a, b).cpu().numpy()
    c2 = dev.dot(a, b).cpu().numpy()
    assert np.array_equal(c1, c2)


def test_empty_and_k_zero(dev):
    a = dev.empty((0, 5), torch.float32)
    b = dev.empty((5, 3), torch.float32)
    assert dev.dot(a, b).shape == (0, 3)
    a = dev.empty((4, 0), torch.float32)
    b = dev.empty((0, 3), torch.float32)
    c = dev.tensor(np.ones((4, 3), np.float32))
    dev.gemm(1.0, a, b, 2.0, c)
    assert np.array_equal(c.cpu().numpy(), 2 * np.ones((4, 3), np.float32))
    assert np.array_equal(dev.dot(a, b).cpu().numpy(), np.zeros((4, 3), np.float32))


def test_errors_like_reference(dev):
    import autograph_b200 as ag
    a = dev.empty((4, 5), torch.float32)
    with pytest.raises(ag.AgError, match="a_cols != b_rows"):
        dev.dot(a, dev.empty((4, 3), torch.float32))
    with pytest.raises(ag.AgError, match="different types"):
        dev.dot(a, dev.empty((5, 3), torch.bfloat16))
    with pytest.raises(ag.AgError):
        dev.gemm(1.0, a, dev.empty((5, 3), torch.float32), 0.0, dev.empty((4, 4), torch.float32))
    with pytest.raises(ag.AgError, match="unimplemented"):
        dev.dot(dev.empty((2, 2), torch.float64), dev.empty((2, 2), torch.float64))
