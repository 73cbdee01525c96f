"""GPU: cross-entropy loss / backward and accuracy (tests/integration_tests.rs:722-827, 1091-1125)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import cycle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("label", [torch.uint8, torch.uint16, torch.uint32])
def test_criterion_golden(dev, golden, dtype, label):
    for c in golden.meta["criterion"]:
        bs, classes = c["bs"], c["classes"]
        x = cycle(0, 10, bs * classes).reshape(bs, classes)
        tn = (np.arange(bs) % classes)
        t = torch.from_numpy(tn.astype(np.int64)).to(label).to(dev.torch_device)
        xd = dev.tensor(x, dtype)
        loss = dev.cross_entropy_loss(xd, t)
        # the reference's tolerance: bs*1e-3 for bf16, bs*f32::EPSILON for f32 (relative)
        eps = bs * 1e-3 if dtype == torch.bfloat16 else bs * 1.2e-7
        assert abs(loss - c["loss"]) <= eps * max(abs(c["loss"]), 1.0) + 1e-5
        dx = dev.cross_entropy_loss_backward(xd, t, 1.0).float().cpu().numpy()
        want = golden[c["name"] + "_dx"]
        if dtype == torch.bfloat16:
            np.testing.assert_allclose(dx, want, rtol=1e-2, atol=1e-6)
        else:
            np.testing.assert_allclose(dx, want, rtol=1e-5, atol=1e-9)
        xa = ((np.arange(bs * classes) + classes // 2 + 1) % classes).astype(np.float32)
        assert dev.accuracy(dev.tensor(xa.reshape(bs, classes), dtype), t) == c["correct"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_criterion_random_vs_oracle(dev, dtype):
    rng = np.random.default_rng(8)
    for bs, classes in [(100, 10), (1000, 10), (65, 1000), (3, 33)]:
        x = (rng.standard_normal((bs, classes)) * 3).astype(np.float32)
        if dtype == torch.bfloat16:
            x = oracle.round_bf16(x)
        t = rng.integers(0, classes, bs).astype(np.uint32)
        td = torch.from_numpy(t.astype(np.int64)).to(torch.uint8 if classes <= 256 else torch.uint32)
        td = td.to(dev.torch_device)
        xd = dev.tensor(x, dtype)
        loss = dev.cross_entropy_loss(xd, td)
        ref = oracle.cross_entropy_loss(x, t)
        assert abs(loss - ref) <= 2e-6 * bs * max(abs(ref) / bs, 1.0) + 1e-4
        dx = dev.cross_entropy_loss_backward(xd, td, 0.5).float().cpu().numpy()
        want = oracle.cross_entropy_loss_backward(x, t, 0.5, bf16=dtype == torch.bfloat16)
        # loss and gradient from one call
        loss1, dx1 = dev.cross_entropy_loss_with_grad(xd, td, 0.5)
        assert abs(float(loss1.cpu()[0]) - loss) <= 1e-6 * max(abs(loss), 1.0)
        dx1 = dx1.float().cpu().numpy()
        assert np.abs(dx1 - want).max() <= (1e-2 if dtype == torch.bfloat16 else 2e-5) * max(np.abs(want).max(), 1e-30)
        np.testing.assert_allclose(dx, want, rtol=1e-2 if dtype == torch.bfloat16 else 2e-5,
                                   atol=1e-8)
        assert dev.accuracy(xd, td) == oracle.accuracy(x, t)


def test_criterion_errors_and_empty(dev):
    import autograph_b200 as ag
    x = dev.empty((4, 3), torch.float32)
    with pytest.raises(ag.AgError, match="Expected target with shape"):
        dev.cross_entropy_loss(x, torch.zeros(5, dtype=torch.uint8, device=dev.torch_device))
    with pytest.raises(ag.AgError):
        dev.cross_entropy_loss(x, torch.zeros(4, dtype=torch.float32, device=dev.torch_device))
    e = dev.empty((0, 3), torch.float32)
    assert dev.cross_entropy_loss(e, torch.zeros(0, dtype=torch.uint8, device=dev.torch_device)) == 0.0
