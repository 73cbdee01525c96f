"""GPU: the benchmark configurations at their full sizes.

  configs[1]  8192^3 dot, f32 and bf16, nn / tn / nt: 4096 sampled elements against an f64
              product of the sampled rows and columns, plus row and column checksums
              (the reference's own dot tests compare whole matrices at small sizes,
              tests/integration_tests.rs:353-371; at this size the checks are the
              size-independent ones)
  configs[3]  wide conv stack at batch 256: logits of 16 sampled rows against the oracle and
              every gradient against torch-CPU float64 autograd (an implementation that shares
              nothing with the oracle or the kernels)
  configs[4a] 65536 images through LeNet5: every row's argmax and the logits against the oracle
  autograd    a parameter used by two layers (two gradients arriving at one node)
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from oracle import models
from torch_reference import wide_stack_torch

pytestmark = pytest.mark.gpu


def _rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() /
                 max(np.abs(ref).max(), 1e-30))


# ------------------------------------------------------------------ configs[1] at 8192^3
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt"])
def test_dot_8192(dev, dtype, layout):
    n = 8192
    bf = dtype == torch.bfloat16
    rng = np.random.default_rng(3000 + 13)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    if bf:
        a, b = oracle.round_bf16(a), oracle.round_bf16(b)
    # the logical operands are a and b; a transposed layout stores the transpose and passes a view
    ad = dev.tensor(np.ascontiguousarray(a.T) if layout[0] == "t" else a, dtype)
    bd = dev.tensor(np.ascontiguousarray(b.T) if layout[1] == "t" else b, dtype)
    c = dev.dot(ad.t() if layout[0] == "t" else ad, bd.t() if layout[1] == "t" else bd)
    dev.wait()
    tol = 1e-2 if bf else 1e-5 * np.sqrt(n)
    # 64 x 64 = 4096 sampled elements against the f64 product of those rows and columns
    rows = np.sort(rng.choice(n, 64, replace=False))
    cols = np.sort(rng.choice(n, 64, replace=False))
    ref = a[rows].astype(np.float64) @ b[:, cols].astype(np.float64)
    got = c[torch.from_numpy(rows).to(c.device)][:, torch.from_numpy(cols).to(c.device)]
    got = got.float().cpu().numpy()
    scale = np.abs(a[rows]).astype(np.float64) @ np.abs(b[:, cols]).astype(np.float64)
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()
    assert (np.abs(got - ref) <= tol * scale).all()
    # checksums over the whole result: C.1 = A.(B.1) and 1^T.C = (1^T.A).B in f64; every element
    # of C may be off by tol * (|A|.|B|) at most, so each checksum by the sum of those bounds
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    row_ref, col_ref = a64 @ b64.sum(1), a64.sum(0) @ b64
    row_bound = np.abs(a64) @ np.abs(b64).sum(1)
    col_bound = np.abs(a64).sum(0) @ np.abs(b64)
    c64 = c.double()
    row_got, col_got = c64.sum(1).cpu().numpy(), c64.sum(0).cpu().numpy()
    assert (np.abs(row_got - row_ref) <= tol * row_bound).all()
    assert (np.abs(col_got - col_ref) <= tol * col_bound).all()
    # a kernel that skipped tiles or wrote them twice would also show here
    assert np.isfinite(row_got).all() and abs(row_got.sum() - row_ref.sum()) <= tol * row_bound.sum()


# ------------------------------------------------------------------ configs[3] at batch 256
def test_wide_stack_bf16_batch_256(dev):
    import autograph_b200 as ag
    dtype = torch.bfloat16
    P = models.init_params(models.WIDE_STACK, 5100, bf16=True)
    bs = 256
    x = oracle.round_bf16(np.random.default_rng(5000).standard_normal((bs, 3, 64, 64)).astype(np.float32))
    t = np.random.default_rng(5001).integers(0, 10, bs).astype(np.uint8)
    model = ag.Model(dev, ag.WIDE_STACK_SPEC, dtype, seed=1)
    model.set_parameters(P)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    logits = model.infer(xh).float().numpy()
    # 16 sampled rows against the oracle (rows are independent of the rest of the batch)
    rows = np.sort(np.random.default_rng(5).choice(bs, 16, replace=False))
    ref_rows = models.forward(models.WIDE_STACK, P, x[rows], acc="f64", bf16=True)
    assert _rel(logits[rows], ref_rows) <= 2e-2
    # all rows and every gradient against torch float64
    ref_loss, ref_logits, ref_grads = wide_stack_torch(P, x, t)
    assert _rel(logits, ref_logits) <= 2e-2
    loss = model.train_step(xh, torch.from_numpy(t).pin_memory(), 0.01)
    assert abs(loss - ref_loss) <= 3e-2 * abs(ref_loss)
    for i, g in enumerate(ref_grads):
        assert _rel(model.get_gradient(i), g.ravel()) <= 5e-2, i
    model.close()


# ------------------------------------------------------------------ configs[4a]: 65536 images
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lenet5_inference_65536(dev, dtype):
    import autograph_b200 as ag
    bf = dtype == torch.bfloat16
    n = 65536
    P = models.init_params(models.LENET5, 2000, bf16=bf)
    x = np.random.default_rng(6000).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    if bf:
        x = oracle.round_bf16(x)
    model = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=1)
    model.set_parameters(P)
    xd = torch.from_numpy(x).to(dtype).to(dev.torch_device)
    logits = model.forward_device(xd).float().cpu().numpy()
    assert logits.shape == (n, 10) and np.isfinite(logits).all()
    oracle.use_all_cores()
    if not bf:
        ref32 = models.forward(models.LENET5, P, x, fast=True)   # the reference's host arithmetic
        assert _rel(logits, ref32) <= 1e-5 * np.sqrt(256)
        assert np.array_equal(logits.argmax(1), ref32.argmax(1))   # all 65536 rows
        rows = np.sort(np.random.default_rng(6).choice(n, 2048, replace=False))
        ref64 = models.forward(models.LENET5, P, x[rows], acc="f64")
        assert _rel(logits[rows], ref64) <= 1e-5 * np.sqrt(256)
        assert np.array_equal(logits[rows].argmax(1), ref64.argmax(1))
    else:
        rows = np.sort(np.random.default_rng(6).choice(n, 4096, replace=False))
        ref = models.forward(models.LENET5, P, x[rows], acc="f64", bf16=True)
        assert _rel(logits[rows], ref) <= 1e-2
        disagree = np.flatnonzero(logits[rows].argmax(1) != ref.argmax(1))
        top2 = np.sort(ref, axis=1)[:, -2:]
        margin = (top2[:, 1] - top2[:, 0]) / np.abs(ref).max()
        print(f"bf16 argmax: {len(disagree)} of {len(rows)} sampled rows differ; "
              f"largest top-2 margin among them {margin[disagree].max() if len(disagree) else 0:.2e}")
        # a row may differ only where its two best logits are closer than bf16 can resolve
        assert (margin[disagree] <= 2 ** -7).all()
        assert len(disagree) <= len(rows) // 100
    # the same images as a 1000-image batch: that size keeps the dense layers inside the
    # one-kernel network, this one runs them as products over the whole batch, so the sums are
    # added in another order
    part = model.forward_device(xd[:1000].contiguous()).float().cpu().numpy()
    assert _rel(part, logits[:1000]) <= (1e-2 if bf else 1e-6)
    model.close()


# ------------------------------------------------------------------ two gradients at one node
TIED_RUN = [("flatten",), ("dense", 64, 64, True), ("relu",), ("dense", 64, 64, True, 1), ("relu",),
            ("dense", 64, 10, False)]
# the same network with a (no-op) Flatten between the Dense layers, which keeps the model from
# treating them as one run: every Dense then has its own node and its own three edges
TIED_SPLIT = [("flatten",), ("dense", 64, 64, True), ("relu",), ("flatten",),
              ("dense", 64, 64, True, 1), ("relu",), ("flatten",), ("dense", 64, 10, False)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bs", [24, 5000])
@pytest.mark.parametrize("TIED", [TIED_RUN, TIED_SPLIT], ids=["run", "split"])
def test_parameter_used_by_two_layers(dev, dtype, bs, TIED):
    """The second Dense shares the first one's weight and bias, so each of the two parameter nodes
    has two incoming edges: the second gradient to arrive is added to the first
    (Node::backward_grad, src/learn/neural_network/autograd.rs:126-131).  "run": the Dense layers
    are one fused run (one kernel pair at batch 24, layer by layer inside the call at 5000);
    "split": separate Dense nodes, whose weight edges meet in the backward walk."""
    import autograph_b200 as ag
    bf = dtype == torch.bfloat16
    P = models.init_params(TIED, 77, bf16=bf)
    assert [p.shape for p in P] == [(64, 64), (64,), (64, 10)]
    rng = np.random.default_rng(78)
    x = rng.uniform(0, 1, (bs, 1, 8, 8)).astype(np.float32)
    if bf:
        x = oracle.round_bf16(x)
    t = rng.integers(0, 10, bs).astype(np.uint8)
    model = ag.Model(dev, TIED, dtype, seed=1)
    assert model.parameter_lens == [4096, 64, 640]
    model.set_parameters(P)
    model.set_sgd(None)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    th = torch.from_numpy(t).pin_memory()
    ref_loss, grads, new_p, _ = models.train_step(TIED, P, x, t.astype(np.uint32), 0.01,
                                                  acc="f64", bf16=bf)
    # and the same gradients from torch float64 autograd, where sharing is plain reuse of a tensor
    ps = [torch.tensor(p, dtype=torch.float64, requires_grad=True) for p in P]
    h = torch.tensor(x, dtype=torch.float64).reshape(bs, 64)
    h = torch.relu(h @ ps[0] + ps[1])
    h = torch.relu(h @ ps[0] + ps[1])
    (F.cross_entropy(h @ ps[2], torch.tensor(t.astype(np.int64)), reduction="sum") / bs).backward()
    for step in range(3):   # eager passes, then the captured graph
        model.set_parameters(P)
        loss = model.train_step(xh, th, 0.01)
        assert abs(loss - ref_loss) <= (3e-2 if bf else 1e-4) * abs(ref_loss), step
        for i, g in enumerate(grads):
            got = model.get_gradient(i)
            assert _rel(got, g.ravel()) <= (4e-2 if bf else 1e-4), (step, i)
            assert _rel(got, ps[i].grad.numpy().ravel()) <= (4e-2 if bf else 1e-4), (step, i)
            assert _rel(model.get_parameter(i), new_p[i].ravel()) <= (1e-2 if bf else 1e-6), (step, i)
    model.close()


# ------------------------------------------------------------------ scratch growth under graphs
def test_captured_passes_survive_scratch_growth(dev, monkeypatch):
    """A captured pass keeps the addresses of the device's scratch blocks.  Running a larger
    batch afterwards makes those blocks grow; replaying the small batch's graph must still give
    the eager result (the outgrown blocks stay allocated)."""
    import autograph_b200 as ag
    dtype = torch.bfloat16
    own = ag.Device(0)          # its scratch blocks start empty
    torch.cuda.set_stream(own.stream)
    rng = np.random.default_rng(11)
    xs = torch.from_numpy(rng.standard_normal((16, 3, 64, 64)).astype(np.float32)).to(dtype).pin_memory()
    xl = torch.from_numpy(rng.standard_normal((96, 3, 64, 64)).astype(np.float32)).to(dtype).pin_memory()
    ts = torch.from_numpy(rng.integers(0, 10, 16).astype(np.uint8)).pin_memory()
    tl = torch.from_numpy(rng.integers(0, 10, 96).astype(np.uint8)).pin_memory()
    monkeypatch.setenv("AG_GRAPH", "0")
    eager = ag.Model(own, ag.WIDE_STACK_SPEC, dtype, seed=9)
    monkeypatch.delenv("AG_GRAPH")
    graphed = ag.Model(own, ag.WIDE_STACK_SPEC, dtype, seed=9)
    # pinned outputs: only passes between pinned buffers are captured
    os_, ol = (torch.empty((n, 10), dtype=dtype).pin_memory() for n in (16, 96))
    want_small = eager.infer(xs, os_).clone()
    want_large = eager.infer(xl, ol).clone()
    for _ in range(3):                                  # eager call, capture, replay
        assert torch.equal(graphed.infer(xs, os_.zero_()), want_small)
    for _ in range(3):                                  # scratch grows here
        assert torch.equal(graphed.infer(xl, ol.zero_()), want_large)
    for _ in range(2):
        assert torch.equal(graphed.infer(xs, os_.zero_()), want_small)   # replay of the old graph
    for m in (eager, graphed):
        m.set_sgd(None)
    for step in range(3):
        assert graphed.train_step(xs, ts, 0.01) == eager.train_step(xs, ts, 0.01), step
    assert graphed.train_step(xl, tl, 0.01) == eager.train_step(xl, tl, 0.01)
    for step in range(2):
        assert graphed.train_step(xs, ts, 0.01) == eager.train_step(xs, ts, 0.01), step
    for i in range(len(eager.parameter_lens)):
        assert np.array_equal(eager.get_parameter(i), graphed.get_parameter(i)), i
    eager.close()
    graphed.close()
    own.wait()
    own.close()
    torch.cuda.set_stream(dev.stream)
