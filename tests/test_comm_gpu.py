"""GPU: the communicator of the C ABI (ag_comm_*) and the fused gradient all-reduce + SGD update.

World size 1 runs on any box.  The two-GPU cases need two GPUs: one process driving both
ranks (ag_comm_create, peer access), and one process per GPU with no torch.distributed at all
(ag_comm_create_rank; the 128-byte id travels through a file, the peers' blocks through CUDA
IPC).  Each checks: replicas end bit-identical, the fused kernel equals the NCCL all-reduce
followed by ag_model_apply_update bit for bit, and both equal a single-GPU step on the global
batch (the loss gradient is scaled by the local batch, src/learn/neural_network/criterion.rs:84,
hence the factor 1 / world).  NVLS is switched off for NCCL in these tests.
"""
import os
import sys
import time
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


def _data(n, seed=7000):
    x = np.random.default_rng(seed).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(seed + 1).integers(0, 10, n).astype(np.uint8)
    return x, t


def _all_params(model):
    return np.concatenate([model.get_parameter(i) for i in range(len(model.parameter_lens))])


def _all_grads(model):
    return np.concatenate([model.get_gradient(i) for i in range(len(model.parameter_lens))])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("momentum", [None, 0.01])
def test_world_of_one_equals_apply_update(dev, dtype, momentum):
    """With one rank the fused kernel is the update alone: same bits as ag_model_apply_update."""
    import autograph_b200 as ag
    from autograph_b200.data_parallel import Comm
    comm = Comm.single_process([dev])
    assert comm.world == 1 and comm.fused_available
    x, t = _data(100)
    xd = torch.from_numpy(x).to(dtype).to(dev.torch_device)
    td = torch.from_numpy(t).to(dev.torch_device)
    a = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=2000)
    b = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=2000)
    for m in (a, b):
        m.set_sgd(momentum)
        m.set_grad_scale(0.25)        # exercises the scaling arithmetic as well
    for step in range(4):
        la, _, _ = a.train_forward_backward(xd, td)
        a.apply_update(0.05)
        lb, _, _ = b.train_forward_backward(xd, td)
        comm.allreduce_update(b, 0.05)
        comm.wait()
        assert la == lb, step
        assert np.array_equal(_all_grads(a), _all_grads(b)), step
        assert np.array_equal(_all_params(a), _all_params(b)), step
    # the plain all-reduce over one rank leaves the buffer as it is
    v = torch.arange(1000, dtype=torch.float32, device=dev.torch_device)
    comm.allreduce_sum(v)
    comm.wait()
    assert torch.equal(v.cpu(), torch.arange(1000, dtype=torch.float32))
    a.close()
    b.close()
    comm.close()


def test_fused_update_refuses_large_buckets(dev):
    """Beyond the 512 KiB limit of the symmetric block the fused call says so and changes nothing."""
    import autograph_b200 as ag
    from autograph_b200.data_parallel import Comm
    comm = Comm.single_process([dev])
    wide = ag.Model(dev, ag.WIDE_STACK_SPEC, torch.bfloat16, seed=3)   # 12.9 M parameters
    before = wide.get_parameter(3)
    with pytest.raises(ag.AgError) as err:
        comm.allreduce_update(wide, 0.01)
    assert err.value.status == ag._capi.AG_ERR_LIMIT
    assert np.array_equal(before, wide.get_parameter(3))
    wide.close()
    comm.close()


# ------------------------------------------------------------------ one process, two GPUs
@two_gpus
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_single_process_two_gpus(dev, dtype):
    import autograph_b200 as ag
    from autograph_b200.data_parallel import Comm, shard_range
    d1 = ag.Device(1)
    devs = [dev, d1]
    comm = Comm.single_process(devs)
    assert comm.world == 2 and comm.fused_available
    # plain all-reduce, all ranks from one thread
    bufs = [torch.full((5000,), float(r + 1), dtype=dtype, device=d.torch_device)
            for r, d in enumerate(devs)]
    comm.allreduce_sum_all(bufs)
    for r in range(2):
        comm.wait(r)
        assert (bufs[r].float().cpu() == 3.0).all()
    # data-parallel step, two ways, against the single-GPU step on the global batch
    x, t = _data(200)
    bf = dtype == torch.bfloat16
    fused, plain = [], []
    for r, d in enumerate(devs):
        for group in (fused, plain):
            m = ag.Model(d, ag.LENET5_SPEC, dtype, seed=2000)
            m.set_sgd(None)
            m.set_grad_scale(0.5)
            group.append(m)
    shards = []
    for r, d in enumerate(devs):
        b, e = shard_range(200, r, 2)
        shards.append((torch.from_numpy(x[b:e]).to(dtype).to(d.torch_device),
                       torch.from_numpy(t[b:e]).to(d.torch_device)))
    for step in range(3):
        losses = []
        for r in range(2):
            fused[r].train_forward_backward(*shards[r], sync=False)
            comm.allreduce_update(fused[r], 0.01, rank=r)
        for r in range(2):
            comm.wait(r)
            losses.append(fused[r].last_loss())
        buckets = []
        for r in range(2):
            _, ptr, n = plain[r].train_forward_backward(*shards[r], sync=False)
            buckets.append((ptr, n))
        import ctypes
        arr = (ctypes.c_void_p * 2)(buckets[0][0], buckets[1][0])
        ag._capi.check(ag.lib().ag_allreduce_sum_all(comm._h, 1 if bf else 0, arr, buckets[0][1]))
        for r in range(2):
            plain[r].apply_update(0.01)
            comm.wait(r)
        p = [_all_params(m) for m in fused]
        assert np.array_equal(p[0], p[1]), step                      # replicas identical
        assert np.array_equal(p[0], _all_params(plain[0])), step     # fused == NCCL + update
        assert np.array_equal(p[0], _all_params(plain[1])), step
        assert np.array_equal(_all_grads(fused[0]), _all_grads(plain[0])), step
    torch.cuda.set_stream(dev.stream)
    single = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=2000)
    single.set_sgd(None)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    th = torch.from_numpy(t).pin_memory()
    for step in range(3):
        loss = single.train_step(xh, th, 0.01)
    ref = _all_params(single)
    tol = 2e-2 if bf else 1e-5
    assert np.abs(p[0] - ref).max() <= tol * max(np.abs(ref).max(), 1.0)
    assert abs(sum(losses) - loss) <= (2e-2 if bf else 1e-4) * abs(loss)   # summed loss
    for m in fused + plain + [single]:
        m.close()
    comm.close()
    d1.close()


@two_gpus
def test_fused_wait_runs_out_when_a_rank_never_joins(dev):
    """Failure detection without a fault: rank 1 never enqueues its half of the step, so rank 0's
    kernel gives up after the (shortened) limit, leaves the parameters untouched and reports
    through the status word; the GPU and the library stay usable."""
    import autograph_b200 as ag
    from autograph_b200.data_parallel import Comm
    d1 = ag.Device(1)
    comm = Comm.single_process([dev, d1])
    comm.set_timeout(0.05)
    torch.cuda.set_stream(dev.stream)
    x, t = _data(100)
    xd = torch.from_numpy(x).to(dev.torch_device)
    td = torch.from_numpy(t).to(dev.torch_device)
    m = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    m.set_sgd(None)
    before = _all_params(m)
    m.train_forward_backward(xd, td, sync=False)
    t0 = time.time()
    comm.allreduce_update(m, 0.01, rank=0)
    with pytest.raises(ag.AgError) as err:
        comm.wait(0)
    assert err.value.status == ag._capi.AG_ERR_DEVICE_TIMEOUT
    assert "151" in err.value.message            # 150 + the rank that never arrived
    assert time.time() - t0 < 5.0
    assert np.array_equal(before, _all_params(m))
    comm.close()                                  # sequence numbers now differ: start over
    # everything still works on this GPU
    loss, _, _ = m.train_forward_backward(xd, td)
    m.apply_update(0.01)
    dev.wait()
    assert np.isfinite(loss) and not np.array_equal(before, _all_params(m))
    m.close()
    d1.close()


# ------------------------------------------------------------------ one process per GPU
def _rank_worker(rank, world, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, str(ROOT))
    import autograph_b200 as ag
    from autograph_b200.data_parallel import Comm, shard_range
    torch.cuda.set_device(rank)
    dev = ag.Device(rank)
    id_file = Path(out_dir) / "nccl_id"
    if rank == 0:
        tmp = Path(out_dir) / "nccl_id.tmp"
        tmp.write_bytes(Comm.unique_id())
        tmp.rename(id_file)
    else:
        for _ in range(600):
            if id_file.exists():
                break
            time.sleep(0.05)
    comm = Comm.per_process(dev, world, rank, id_file.read_bytes())
    assert comm.fused_available
    x, t = _data(25 * world)
    b, e = shard_range(25 * world, rank, world)
    xd = torch.from_numpy(x[b:e]).to(dev.torch_device)
    td = torch.from_numpy(t[b:e]).to(dev.torch_device)
    fused = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    plain = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    for m in (fused, plain):
        m.set_sgd(0.01)
        m.set_grad_scale(1.0 / world)
    for step in range(3):
        fused.train_forward_backward(xd, td, sync=False)
        comm.allreduce_update(fused, 0.01)
        _, ptr, n = plain.train_forward_backward(xd, td, sync=False)
        comm.allreduce_bucket(ptr, n, torch.float32)
        plain.apply_update(0.01)
        comm.wait()
    np.save(Path(out_dir) / f"fused{rank}.npy", _all_params(fused))
    np.save(Path(out_dir) / f"plain{rank}.npy", _all_params(plain))
    np.save(Path(out_dir) / f"loss{rank}.npy", np.float32(fused.last_loss()))
    fused.close()
    plain.close()
    comm.close()


@two_gpus
@pytest.mark.parametrize("world", [2, 4, 8])
def test_one_process_per_gpu_without_torch_distributed(tmp_path, dev, world):
    import torch.multiprocessing as mp
    import autograph_b200 as ag
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_rank_worker, args=(world, str(tmp_path)), nprocs=world, join=True)
    f0 = np.load(tmp_path / "fused0.npy")
    for r in range(1, world):
        assert np.array_equal(f0, np.load(tmp_path / f"fused{r}.npy")), r   # replicas identical
    if world == 2:
        # a sum of two terms has one order: the fused kernel and NCCL agree bit for bit
        assert np.array_equal(f0, np.load(tmp_path / "plain0.npy"))
        assert np.array_equal(f0, np.load(tmp_path / "plain1.npy"))
    else:
        p0 = np.load(tmp_path / "plain0.npy")
        assert np.abs(f0 - p0).max() <= 1e-6 * max(np.abs(p0).max(), 1.0)
    single = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    single.set_sgd(0.01)
    x, t = _data(25 * world)
    xh, th = torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory()
    for step in range(3):
        loss = single.train_step(xh, th, 0.01)
    ref = _all_params(single)
    assert np.abs(f0 - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1.0)
    total = sum(float(np.load(tmp_path / f"loss{r}.npy")) for r in range(world))
    assert abs(total - loss) <= 1e-4 * abs(loss)
    single.close()
