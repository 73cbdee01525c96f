"""Batch-sharded data parallelism: one process per GPU, torch.distributed for the plumbing.

The reference has no multi-device code; its networks shard naturally by batch
(every image is independent, parameters are replicated).  Inference needs no
collective.  Training needs one sum all-reduce of the flat gradient bucket per
step; because the loss gradient is scaled by the *local* batch size
(src/learn/neural_network/criterion.rs:84) the reduced sum is multiplied by
1/world so that the update equals a single-device step on the global batch.
"""
from __future__ import annotations

import ctypes
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


def init_process_group(backend: str, timeout_s: float | None = None):
    """Joins the torchrun world.  timeout_s bounds every collective of the group: a rank whose
    peer never enters a collective gets an error after that long instead of waiting forever."""
    import datetime

    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {} if timeout_s is None else {"timeout": datetime.timedelta(seconds=timeout_s)}
        dist.init_process_group(backend=backend, **kw)
    return dist


def allreduce_gradients(bucket, world: int):
    """Sum-all-reduce the flat gradient bucket in place (NCCL over NVLink on GPUs, gloo on
    CPU).  Returns the scale (1/world) the optimizer must apply to the sum.  A collective that
    a peer never joins ends with AgError(AG_ERR_DEVICE_TIMEOUT) once the group's timeout has
    passed; the bucket's contents are then undefined and the step must not be applied."""
    if world > 1:
        import torch.distributed as dist

        from ._capi import AG_ERR_DEVICE_TIMEOUT, AgError
        try:
            dist.all_reduce(bucket, op=dist.ReduceOp.SUM)
        except RuntimeError as exc:   # torch reports timeouts and lost peers this way
            raise AgError(AG_ERR_DEVICE_TIMEOUT,
                          f"gradient all-reduce failed (a rank did not join?): {exc}") from exc
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


class Comm:
    """≙ ag_comm: a communicator over the GPUs of one box, behind the C ABI (NCCL for the plain
    all-reduce, peer loads over NVLink for the fused all-reduce + update).

    ``Comm.single_process(devices)``: this process drives every rank; rank r is devices[r].
    ``Comm.per_process(device, world, rank, unique_id)``: one process per GPU; rank 0 makes
    the id with ``Comm.unique_id()`` and hands it to the others (any transport).
    ``Comm.from_torch_distributed(device)``: the same, the id travelling over an initialised
    torch.distributed group.
    After a call has failed with AG_ERR_DEVICE_TIMEOUT (a peer never arrived) the ranks'
    sequence numbers differ: close the communicator and make a new one."""

    def __init__(self, handle, world, ranks):
        self._h = handle
        self.world = world
        self.ranks = ranks          # {rank: Device} driven by this process

    @staticmethod
    def _lib():
        from . import _capi
        return _capi.lib(), _capi

    @classmethod
    def single_process(cls, devices):
        lib, _capi = cls._lib()
        arr = (ctypes.c_void_p * len(devices))(*[d._h for d in devices])
        h = ctypes.c_void_p()
        _capi.check(lib.ag_comm_create(arr, len(devices), ctypes.byref(h)))
        return cls(h, len(devices), dict(enumerate(devices)))

    @staticmethod
    def unique_id() -> bytes:
        lib, _capi = Comm._lib()
        buf = ctypes.create_string_buffer(128)
        _capi.check(lib.ag_comm_unique_id(buf, 128))
        return buf.raw

    @classmethod
    def per_process(cls, device, world, rank, unique_id: bytes):
        lib, _capi = cls._lib()
        h = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(unique_id, 128)
        _capi.check(lib.ag_comm_create_rank(device._h, world, rank, buf, 128, ctypes.byref(h)))
        return cls(h, world, {rank: device})

    @classmethod
    def from_torch_distributed(cls, device):
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        on_gpu = dist.get_backend() == "nccl"
        raw = cls.unique_id() if rank == 0 else bytes(128)
        t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
        if on_gpu:
            t = t.to(device.torch_device)
        dist.broadcast(t, src=0)
        return cls.per_process(device, world, rank, bytes(t.cpu().numpy().tobytes()))

    def _rank(self, rank):
        if rank is None:
            if len(self.ranks) != 1:
                raise ValueError("this process drives several ranks: name one")
            return next(iter(self.ranks))
        return rank

    @property
    def fused_available(self) -> bool:
        lib, _capi = self._lib()
        w, f = ctypes.c_int(), ctypes.c_int()
        _capi.check(lib.ag_comm_world(self._h, ctypes.byref(w), ctypes.byref(f)))
        return bool(f.value)

    def set_timeout(self, seconds: float):
        lib, _capi = self._lib()
        _capi.check(lib.ag_comm_set_timeout(self._h, ctypes.c_double(seconds)))

    def allreduce_sum(self, tensor, rank=None):
        """In-place sum over all ranks of a contiguous f32 / bf16 / u8 device tensor."""
        from . import _dtype_code
        lib, _capi = self._lib()
        if not tensor.is_contiguous() or not tensor.is_cuda:
            raise _capi.AgError(_capi.AG_ERR_INVALID, "allreduce needs a contiguous device tensor")
        _capi.check(lib.ag_allreduce_sum(self._h, self._rank(rank), _dtype_code(tensor.dtype),
                                         ctypes.c_void_p(tensor.data_ptr()), tensor.numel()))
        return tensor

    def allreduce_sum_all(self, tensors):
        """Single process: every rank's tensor (in rank order) in one grouped call."""
        from . import _dtype_code
        lib, _capi = self._lib()
        arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        _capi.check(lib.ag_allreduce_sum_all(self._h, _dtype_code(tensors[0].dtype), arr,
                                             tensors[0].numel()))
        return tensors

    def allreduce_bucket(self, ptr: int, length: int, dtype, rank=None):
        """The same on a raw device pointer (a model's gradient bucket)."""
        from . import _dtype_code
        lib, _capi = self._lib()
        _capi.check(lib.ag_allreduce_sum(self._h, self._rank(rank), _dtype_code(dtype),
                                         ctypes.c_void_p(ptr), length))

    def allreduce_update(self, model, lr: float, rank=None):
        """Fused gradient all-reduce + 1/world scaling + SGD update: one kernel on the rank."""
        lib, _capi = self._lib()
        _capi.check(lib.ag_model_allreduce_update(model._h, self._h, self._rank(rank),
                                                  ctypes.c_float(lr)))

    def wait(self, rank=None):
        lib, _capi = self._lib()
        _capi.check(lib.ag_comm_wait(self._h, self._rank(rank)))

    def close(self):
        if getattr(self, "_h", None):
            self._lib()[0].ag_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
