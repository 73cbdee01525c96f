"""Batch-sharded data parallelism: one process per GPU, torch.distributed for the plumbing.

The reference has no multi-device code; its networks shard naturally by batch
(every image is independent, parameters are replicated).  Inference needs no
collective.  Training needs one sum all-reduce of the flat gradient bucket per
step; because the loss gradient is scaled by the *local* batch size
(src/learn/neural_network/criterion.rs:84) the reduced sum is multiplied by
1/world so that the update equals a single-device step on the global batch.
"""
from __future__ import annotations

import os


def env_world():
    """(rank, local_rank, world_size) from the torchrun environment (1 process -> 0, 0, 1)."""
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


def shard_range(n: int, rank: int, world: int):
    """Contiguous slice [begin, end) of n items owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def init_process_group(backend: str):
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=backend)
    return dist


def allreduce_gradients(bucket, world: int):
    """Sum-all-reduce the flat gradient bucket in place (NCCL over NVLink on GPUs, gloo on
    CPU).  Returns the scale (1/world) the optimizer must apply to the sum."""
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM)
    return 1.0 / world


def bucket_view(ptr: int, length: int, dtype, device):
    """torch tensor aliasing the model's gradient bucket (no copy)."""
    import torch

    class _Iface:
        pass

    elem = torch.empty((), dtype=dtype).element_size()
    typestr = {torch.float32: "<f4", torch.bfloat16: "<u2"}[dtype]
    holder = _Iface()
    holder.__cuda_array_interface__ = {
        "shape": (length,), "typestr": typestr, "data": (ptr, False), "version": 3,
        "strides": (elem,),
    }
    t = torch.as_tensor(holder, device=device)
    return t.view(dtype) if dtype == torch.bfloat16 else t
