"""CPU: the oracle's composition of the wide conv stack (forward, loss, every gradient)
against torch float64 autograd, an implementation that shares nothing with it.  The same torch
reference checks the CUDA path at batch 256 (tests/test_parity_configs_gpu.py)."""
import numpy as np

import oracle
from oracle import models
from torch_reference import wide_stack_torch


def _rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() /
                 max(np.abs(ref).max(), 1e-30))


def test_wide_stack_oracle_equals_torch_autograd():
    P = models.init_params(models.WIDE_STACK, 5100, bf16=True)
    bs = 2
    x = oracle.round_bf16(np.random.default_rng(5000).standard_normal((bs, 3, 64, 64)).astype(np.float32))
    t = np.random.default_rng(5001).integers(0, 10, bs).astype(np.uint8)
    loss, grads, _, _ = models.train_step(models.WIDE_STACK, P, x, t.astype(np.uint32), 0.01,
                                          acc="f64", bf16=True)
    logits = models.forward(models.WIDE_STACK, P, x, acc="f64", bf16=True)
    ref_loss, ref_logits, ref_grads = wide_stack_torch(P, x, t)
    # both round to bf16 at every layer boundary; they may differ by a rounding where a sum lands
    # on a tie, hence a tolerance of a few bf16 steps rather than equality
    assert _rel(logits, ref_logits) <= 1e-2
    assert abs(loss - ref_loss) <= 1e-2 * abs(ref_loss)
    for i, (g, r) in enumerate(zip(grads, ref_grads)):
        assert _rel(g, r) <= 2e-2, i
