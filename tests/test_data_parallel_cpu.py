"""CPU, gloo, world_size 2: the data-parallel host logic (sharding + gradient all-reduce +
1/world scaling) reproduces the single-process step on the global batch."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, str(ROOT))
    from autograph_b200 import data_parallel as dp
    from oracle import models
    import oracle
    dist = dp.init_process_group("gloo")
    P = models.init_params(models.LENET5, 2000)
    n = 40
    x = np.random.default_rng(7000).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(7001).integers(0, 10, n).astype(np.uint32)
    b, e = dp.shard_range(n, rank, world)
    logits, saved = models.forward(models.LENET5, P, x[b:e], keep=True)
    dl = oracle.cross_entropy_loss_backward(logits, t[b:e], 1.0)   # scaled by the LOCAL batch
    grads = models.backward(models.LENET5, P, saved, dl)
    bucket = torch.from_numpy(np.concatenate([g.ravel() for g in grads]))
    scale = dp.allreduce_gradients(bucket, world)
    np.save(Path(out_dir) / f"g{rank}.npy", bucket.numpy() * np.float32(scale))
    dist.barrier()
    dist.destroy_process_group()


def test_shard_range():
    from autograph_b200.data_parallel import shard_range
    for n, world in [(65536, 8), (10, 3), (7, 8), (0, 2)]:
        spans = [shard_range(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        sizes = [e - b for b, e in spans]
        assert max(sizes) - min(sizes) <= 1


def test_gloo_two_ranks_match_global_batch(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    g0 = np.load(tmp_path / "g0.npy")
    g1 = np.load(tmp_path / "g1.npy")
    assert np.array_equal(g0, g1)
    from oracle import models
    import oracle
    P = models.init_params(models.LENET5, 2000)
    n = 40
    x = np.random.default_rng(7000).uniform(0, 1, (n, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(7001).integers(0, 10, n).astype(np.uint32)
    logits, saved = models.forward(models.LENET5, P, x, keep=True)
    dl = oracle.cross_entropy_loss_backward(logits, t, 1.0)
    grads = models.backward(models.LENET5, P, saved, dl)
    full = np.concatenate([g.ravel() for g in grads])
    assert np.abs(g0 - full).max() <= 1e-5 * np.abs(full).max()


def _absent_peer_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.path.insert(0, str(ROOT))
    import time
    from autograph_b200 import AgError, _capi
    from autograph_b200 import data_parallel as dp
    dist = dp.init_process_group("gloo", timeout_s=1.0)
    bucket = torch.ones(1000)
    dp.allreduce_gradients(bucket, world)          # a step both ranks take
    assert bucket[0].item() == world
    if rank == 1:
        time.sleep(4.0)                            # rank 1 never enters the next collective
        return
    t0 = time.time()
    try:
        dp.allreduce_gradients(bucket, world)
        outcome = "completed"
    except AgError as exc:
        outcome = f"{exc.status} {time.time() - t0:.2f}"
        assert exc.status == _capi.AG_ERR_DEVICE_TIMEOUT
    (Path(out_dir) / "outcome.txt").write_text(outcome)


def test_gloo_rank_that_never_joins_is_detected(tmp_path):
    """Failure detection on the host: one rank skips a collective; the other gets an error
    after the group's short timeout instead of waiting forever."""
    port = _free_port()
    mp.spawn(_absent_peer_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    status, waited = (tmp_path / "outcome.txt").read_text().split()
    assert int(status) == -6 and float(waited) < 3.5
