"""GPU: the u8 image pipeline (scaled_cast, and the same cast folded into the one-kernel
network) against the oracle and against the float path."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 15, 16, 1000 * 784, 784 * 3 + 5])
def test_scaled_cast_u8_bit_exact(dev, dtype, n):
    """alpha * x in the output type: bit-exact against the oracle, aligned and ragged sizes."""
    rng = np.random.default_rng(n)
    x = rng.integers(0, 256, n).astype(np.uint8)
    xd = torch.from_numpy(x).to(dev.torch_device)
    y = dev.scaled_cast_u8(xd, 1.0 / 255.0, dtype).float().cpu().numpy()
    assert np.array_equal(y, oracle.scaled_cast_u8(x, 1.0 / 255.0, bf16=dtype == torch.bfloat16))
    # an unaligned view takes the scalar path
    if n > 3:
        y1 = dev.scaled_cast_u8(xd[1:], 0.5, dtype).float().cpu().numpy()
        assert np.array_equal(y1, oracle.scaled_cast_u8(x[1:], 0.5, bf16=dtype == torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bs", [1000, 37])
def test_model_infer_u8_equals_scaled_cast_then_infer(dev, dtype, bs):
    """LeNet5 on u8 images (cast folded into the network kernel) gives the bits of
    scaled_cast followed by the float inference, pinned and pageable buffers alike."""
    import autograph_b200 as ag
    model = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=11)
    rng = np.random.default_rng(bs)
    x8 = torch.from_numpy(rng.integers(0, 256, (bs, 1, 28, 28)).astype(np.uint8))
    xf = dev.scaled_cast_u8(x8.to(dev.torch_device), 1.0 / 255.0, dtype)
    want = model.forward_device(xf).cpu()
    got_pinned = model.infer_u8(x8.pin_memory(), out_host=torch.empty((bs, 10), dtype=dtype).pin_memory())
    assert torch.equal(got_pinned, want)
    got_pageable = model.infer_u8(x8)
    assert torch.equal(got_pageable, want)
    # and it matches the oracle's forward on the oracle's cast
    if dtype == torch.float32:
        from oracle import models
        P = [model.get_parameter(i) for i in range(len(model.parameter_lens))]
        shapes = [(6, 1, 5, 5), (16, 6, 5, 5), (256, 128), (128, 84), (84, 10), (10,)]
        P = [p.reshape(s) for p, s in zip(P, shapes)]
        ref = models.forward(models.LENET5, P, oracle.scaled_cast_u8(x8.numpy(), 1.0 / 255.0), acc="f64")
        err = np.abs(got_pinned.numpy() - ref).max() / np.abs(ref).max()
        assert err <= 1e-5 * np.sqrt(256)
    model.close()
