"""GPU (needs 2 GPUs): data-parallel training over NCCL equals the single-GPU step on the
global batch.  Two ranks, 100 images each; the gradient bucket is sum-all-reduced and the
optimizer applies 1/world."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _data(n):
    x = np.random.default_rng(7000).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(7001).integers(0, 10, n).astype(np.uint8)
    return x, t


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    import autograph_b200 as ag
    from autograph_b200 import data_parallel as dp
    torch.cuda.set_device(rank)
    dist = dp.init_process_group("nccl")
    dev = ag.Device(rank)
    model = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    model.set_sgd(None)
    model.set_grad_scale(1.0 / world)
    x, t = _data(200)
    b, e = dp.shard_range(200, rank, world)
    xd = torch.from_numpy(x[b:e]).to(dev.torch_device)
    td = torch.from_numpy(t[b:e]).to(dev.torch_device)
    loss, ptr, length = model.train_forward_backward(xd, td)
    bucket = dp.bucket_view(ptr, length, torch.float32, dev.torch_device)
    dp.allreduce_gradients(bucket, world)
    model.apply_update(0.01)
    params = np.concatenate([model.get_parameter(i) for i in range(len(model.parameter_lens))])
    np.save(Path(out_dir) / f"p{rank}.npy", params)
    np.save(Path(out_dir) / f"l{rank}.npy", np.float32(loss))
    dist.barrier()
    model.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_step_matches_global_batch(tmp_path, dev):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    p0, p1 = np.load(tmp_path / "p0.npy"), np.load(tmp_path / "p1.npy")
    assert np.array_equal(p0, p1)                      # replicas stay identical
    import autograph_b200 as ag
    model = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    model.set_sgd(None)
    x, t = _data(200)
    loss = model.train_step(torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory(), 0.01)
    ref = np.concatenate([model.get_parameter(i) for i in range(len(model.parameter_lens))])
    assert np.abs(p0 - ref).max() <= 1e-6 * max(np.abs(ref).max(), 1.0) + 1e-7
    total = float(np.load(tmp_path / "l0.npy")) + float(np.load(tmp_path / "l1.npy"))
    assert abs(total - loss) <= 1e-4 * abs(loss)       # the loss is a sum over the batch
    model.close()
