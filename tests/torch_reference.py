"""torch float64 autograd restatement of the wide conv stack (TEST INFRASTRUCTURE): a second
checker that shares no code with the oracle or the CUDA kernels.  It follows the reference's
semantics where torch's defaults differ: bf16 stores at every layer boundary, the max-pool
gradient of MaxPool2's backward edge, and a summed loss whose gradient is scaled by 1 / batch."""
import numpy as np
import torch
import torch.nn.functional as F


class _RoundBf16(torch.autograd.Function):
    """Value rounded to bf16 (the store at every layer boundary), gradient passed through."""

    @staticmethod
    def forward(ctx, x):
        return x.to(torch.bfloat16).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g.to(torch.bfloat16).to(g.dtype)


class _PoolAsTheReference(torch.autograd.Function):
    """2x2 max pool whose gradient follows MaxPool2's backward edge (layer.rs:1203-1212 ->
    src/tensor/ops.rs:1144-1207): the gradient buffer starts as a copy of the input, every window
    is zeroed and receives dy at its first maximum, and cells that no window covers (the last row
    and column of an odd plane) keep the input's value."""

    @staticmethod
    def forward(ctx, x):
        y, idx = F.max_pool2d(x, 2, return_indices=True)
        ctx.save_for_backward(x, idx)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, idx = ctx.saved_tensors
        h, w = x.shape[-2:]
        dx = F.max_unpool2d(dy, idx, 2, output_size=(h, w))
        ch, cw = (h // 2) * 2, (w // 2) * 2
        dx[..., ch:, :] = x[..., ch:, :]
        dx[..., :, cw:] = x[..., :, cw:]
        return dx


def wide_stack_torch(P, x, t):
    """Loss and parameter gradients of the wide stack in float64 with bf16 stores."""
    rd = _RoundBf16.apply
    ps = [torch.tensor(p, dtype=torch.float64, requires_grad=True) for p in P]
    h = torch.tensor(x, dtype=torch.float64)
    h = _PoolAsTheReference.apply(torch.relu(rd(F.conv2d(h, ps[0]))))
    h = _PoolAsTheReference.apply(torch.relu(rd(F.conv2d(h, ps[1]))))
    h = h.reshape(h.shape[0], -1)
    h = torch.relu(rd(h @ ps[2]))
    logits = rd(rd(h @ ps[3]) + ps[4])
    loss = F.cross_entropy(logits, torch.tensor(t.astype(np.int64)), reduction="sum")
    # the loss is a sum over the batch whose gradient is scaled by 1 / batch
    # (src/learn/neural_network/criterion.rs:73-84)
    (loss / x.shape[0]).backward()
    return float(loss.detach()), logits.detach().numpy(), [p.grad.numpy() for p in ps]
