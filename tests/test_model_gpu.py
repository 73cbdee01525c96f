"""GPU: the layer chain (LeNet5 and the wider conv stack) against the oracle composition:
inference logits + argmax, and a full training step (loss, every gradient, every update)."""
import numpy as np
import pytest
import torch

import oracle
from oracle import models

pytestmark = pytest.mark.gpu


def _params(spec, seed, bf16):
    return models.init_params(spec, seed, bf16=bf16)


def _rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() /
                 max(np.abs(ref).max(), 1e-30))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lenet5_inference_bs1000(dev, dtype):
    """Benchmark configuration 0: x [1000,1,28,28] U[0,1) seed 1000, default-init weights seed 2000."""
    import autograph_b200 as ag
    bf = dtype == torch.bfloat16
    P = _params(models.LENET5, 2000, bf)
    x = np.random.default_rng(1000).uniform(0, 1, (1000, 1, 28, 28)).astype(np.float32)
    if bf:
        x = oracle.round_bf16(x)
    model = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=1)
    model.set_parameters(P)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    logits = model.infer(xh).float().numpy()
    ref64 = models.forward(models.LENET5, P, x, acc="f64")           # f64 accumulation, f32 stores
    if bf:
        assert _rel(logits, ref64) <= 1e-2 * 4                        # 5 layers of bf16 stores
        ref_bf = models.forward(models.LENET5, P, x, acc="f64", bf16=True)
        assert _rel(logits, ref_bf) <= 1e-2
        # argmax must match wherever the top-2 margin exceeds the bf16 resolution
        top2 = np.sort(ref_bf, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2e-2 * np.abs(ref_bf).max()
        assert (logits.argmax(1) == ref_bf.argmax(1))[clear].all()
        assert (logits.argmax(1) == ref_bf.argmax(1)).mean() > 0.97
    else:
        ref32 = models.forward(models.LENET5, P, x)                    # the reference's host arithmetic
        assert _rel(logits, ref64) <= 1e-5 * np.sqrt(256)
        assert _rel(logits, ref32) <= 1e-5 * np.sqrt(256)
        assert np.array_equal(logits.argmax(1), ref64.argmax(1))       # all 1000 rows
        assert np.array_equal(logits.argmax(1), ref32.argmax(1))
    # device-resident path gives the same bits as the host-buffer path
    out = model.forward_device(xh.to(dev.torch_device)).float().cpu().numpy()
    assert np.array_equal(out, logits)
    # batch independence: the first 10 rows alone give the same logits
    small = model.infer(xh[:10].contiguous()).float().numpy()
    assert _rel(small, logits[:10]) <= (1e-2 if bf else 1e-6)
    model.close()


@pytest.mark.parametrize("bs", [1, 3, 7, 8, 100, 1000, 1003, 9000])
def test_lenet5_host_images_equal_device_images(dev, bs):
    """f32 images in pinned host memory (read over PCIe by the kernel itself) give the logits of
    the device-resident pass bit for bit, at every group size (1 to 7 images per CTA, ragged last
    group, and the split form for large batches), and so does a host view that does not start
    on a 16-byte boundary."""
    import autograph_b200 as ag
    model = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=7)
    x = torch.from_numpy(np.random.default_rng(bs).uniform(0, 1, (bs, 1, 28, 28)).astype(np.float32))
    xh = x.pin_memory()
    out_h = torch.empty((bs, 10), dtype=torch.float32).pin_memory()
    for _ in range(3):     # eager, captured and replayed forms of the call
        out_h.fill_(float("nan"))
        got = model.infer(xh, out_h)
        ref = model.forward_device(x.to(dev.torch_device)).cpu()
        assert torch.equal(got, ref)
    # a host view that does not start on a 16-byte boundary takes the scalar staging loop
    buf = torch.empty((bs * 784 + 1,), dtype=torch.float32).pin_memory()
    buf[1:] = x.reshape(-1)
    got = model.infer(buf[1:].reshape(bs, 1, 28, 28), out_h)
    assert torch.equal(got, ref)
    model.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("momentum", [None, 0.01])
def test_lenet5_train_step_bs100(dev, dtype, momentum):
    """Benchmark configuration 2: x [100,1,28,28] seed 4000, labels seed 4001, lr 0.01."""
    import autograph_b200 as ag
    bf = dtype == torch.bfloat16
    P = _params(models.LENET5, 2000, bf)
    x = np.random.default_rng(4000).uniform(0, 1, (100, 1, 28, 28)).astype(np.float32)
    if bf:
        x = oracle.round_bf16(x)
    t = np.random.default_rng(4001).integers(0, 10, 100).astype(np.uint8)
    model = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=1)
    model.set_parameters(P)
    model.set_sgd(momentum)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    th = torch.from_numpy(t).pin_memory()
    loss = model.train_step(xh, th, 0.01)
    ref_loss, grads, new_p, vel = models.train_step(models.LENET5, P, x, t.astype(np.uint32), 0.01,
                                                    momentum=momentum, acc="f64", bf16=bf)
    assert abs(loss - ref_loss) <= (2e-2 if bf else 1e-4) * abs(ref_loss)
    for i, (g, w) in enumerate(zip(grads, new_p)):
        got_g = model.get_gradient(i)
        got_w = model.get_parameter(i)
        gtol = 3e-2 if bf else 1e-4
        assert _rel(got_g, g.ravel()) <= gtol, (i, _rel(got_g, g.ravel()))
        assert _rel(got_w, w.ravel()) <= (1e-2 if bf else 1e-6), i
        if not bf:
            # the update itself is exact given the device's own gradient
            if momentum is None:
                assert np.array_equal(got_w, oracle.sgd_update(P[i].ravel(), got_g, 0.01))
    # a second step runs on the updated parameters and lowers the loss on the same batch
    loss2 = model.train_step(xh, th, 0.01)
    assert loss2 < loss
    model.close()


def test_enqueued_forward_backward_equals_the_blocking_call(dev):
    """The data-parallel half step without its host synchronisation: same loss, same update."""
    import autograph_b200 as ag
    rng = np.random.default_rng(5)
    x = dev.tensor(rng.uniform(0, 1, (100, 1, 28, 28)).astype(np.float32))
    t = torch.from_numpy(rng.integers(0, 10, 100).astype(np.uint8)).to(dev.torch_device)
    a = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=3)
    b = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=3)
    for m in (a, b):
        m.set_sgd(None)
    for step in range(4):  # eager passes first, then the captured graph
        la, _, _ = a.train_forward_backward(x, t)
        a.apply_update(0.05)
        lb, ptr, n = b.train_forward_backward(x, t, sync=False)
        assert lb is None and ptr and n > 0
        b.apply_update(0.05)
        assert b.last_loss() == la, step
    for i in range(len(a.parameter_lens)):
        assert np.array_equal(a.get_parameter(i), b.get_parameter(i))
    a.close()
    b.close()


def test_wide_stack_bf16_forward_backward(dev):
    """Benchmark configuration 3 at batch 8 (the oracle's naive loops finish in seconds), bf16."""
    import autograph_b200 as ag
    dtype = torch.bfloat16
    P = _params(models.WIDE_STACK, 5100, True)
    bs = 8
    x = oracle.round_bf16(np.random.default_rng(5000).standard_normal((bs, 3, 64, 64)).astype(np.float32))
    t = np.random.default_rng(5001).integers(0, 10, bs).astype(np.uint8)
    model = ag.Model(dev, ag.WIDE_STACK_SPEC, dtype, seed=1)
    model.set_parameters(P)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    logits = model.infer(xh).float().numpy()
    ref = models.forward(models.WIDE_STACK, P, x, acc="f64", bf16=True)
    assert _rel(logits, ref) <= 2e-2
    loss = model.train_step(xh, torch.from_numpy(t).pin_memory(), 0.01)
    ref_loss, grads, new_p, _ = models.train_step(models.WIDE_STACK, P, x, t.astype(np.uint32), 0.01,
                                                  acc="f64", bf16=True)
    assert abs(loss - ref_loss) <= 3e-2 * abs(ref_loss)
    for i, g in enumerate(grads):
        assert _rel(model.get_gradient(i), g.ravel()) <= 5e-2, i
    model.close()


def test_pipelined_inference_equals_the_blocking_call(dev):
    """Two batches in flight (the copy of one overlaps the network pass of the other): every
    batch's logits are those of the blocking call; a third enqueue without a wait, a ticket that
    is not in flight and pageable buffers are refused."""
    import autograph_b200 as ag
    model = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=11)
    rng = np.random.default_rng(8200)
    xs = [torch.from_numpy(rng.uniform(0, 1, (1000, 1, 28, 28)).astype(np.float32)).pin_memory() for _ in range(5)]
    want = [model.infer(x).clone() for x in xs]
    outs = [torch.empty((1000, 10), dtype=torch.float32).pin_memory() for _ in range(2)]
    for _ in range(2):
        tickets = []
        for i, x in enumerate(xs):
            if len(tickets) == 2:
                j, t = tickets.pop(0)
                model.infer_wait(t)
                assert torch.equal(outs[j % 2], want[j])
            outs[i % 2].fill_(float("nan"))
            tickets.append((i, model.infer_enqueue(x, outs[i % 2])))
        with pytest.raises(ag.AgError):
            model.infer_enqueue(xs[0], torch.empty((1000, 10)).pin_memory())   # both slots in flight
        for j, t in tickets:
            model.infer_wait(t)
            assert torch.equal(outs[j % 2], want[j])
    with pytest.raises(ag.AgError):
        model.infer_wait(0)                                                    # nothing in flight
    with pytest.raises(ag.AgError):
        model.infer_enqueue(xs[0].clone(), outs[0])                            # pageable input
    # another batch size re-sizes the slot
    small = xs[0][:64].contiguous().pin_memory()
    o = torch.empty((64, 10), dtype=torch.float32).pin_memory()
    model.infer_wait(model.infer_enqueue(small, o))
    assert torch.equal(o, want[0][:64])
    model.close()


def test_learning_rate_schedule_reuses_one_graph(dev):
    """A different learning rate every step: the captured step without the update serves all of
    them (the update follows as a plain launch) and the parameters equal those of the
    enqueue-then-update form bit for bit."""
    import autograph_b200 as ag
    rng = np.random.default_rng(8100)
    xs = [torch.from_numpy(rng.uniform(0, 1, (100, 1, 28, 28)).astype(np.float32)).pin_memory() for _ in range(3)]
    ts = [torch.from_numpy(rng.integers(0, 10, 100).astype(np.uint8)).pin_memory() for _ in range(3)]
    a = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=5)
    b = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=5)
    rates = [0.01, 0.01, 0.01, 0.02, 0.03, 0.01, 0.04, 0.05, 0.06, 0.07, 0.08, 0.09, 0.1, 0.11]
    before = ag.kernel_launch_count()
    for i, lr in enumerate(rates):
        la = a.train_step(xs[i % 3], ts[i % 3], lr)
        lb = b.train_forward_backward(xs[i % 3].to(dev.torch_device), ts[i % 3].to(dev.torch_device))[0]
        b.apply_update(lr)
        assert la == lb
    assert ag.kernel_launch_count() > before
    for i in range(len(a.parameter_lens)):
        assert np.array_equal(a.get_parameter(i), b.get_parameter(i)), i
    a.close()
    b.close()


STAGE_SPECS = {
    # second stage inside a run that must hand a gradient to the layer before it (first convolution
    # has too few output channels for the tensor cores), biases, odd planes (27 x 27 -> 13 x 13:
    # cells no pool window covers)
    "input_gradient_bias_odd": (8, 63, [
        ("conv", 3, 16, (5, 5), True), ("relu",), ("pool", (2, 2)),
        ("conv", 16, 64, (3, 3), True), ("relu",), ("pool", (2, 2)),
        ("flatten",), ("dense", 64 * 13 * 13, 32, False), ("relu",), ("dense", 32, 10, True)]),
    # a run of two stages: patches first layer with bias, odd second plane (17 x 17 -> 8 x 8)
    "two_stages_bias_odd": (16, 40, [
        ("conv", 3, 64, (3, 3), True), ("relu",), ("pool", (2, 2)),
        ("conv", 64, 64, (3, 3), True), ("relu",), ("pool", (2, 2)),
        ("flatten",), ("dense", 64 * 8 * 8, 32, False), ("relu",), ("dense", 32, 10, True)]),
}


@pytest.mark.parametrize("case", sorted(STAGE_SPECS))
def test_channels_last_stage_runs(dev, case):
    """Conv2 -> Relu -> MaxPool2 stages of a bf16 training pass that run channels-last as one
    node: loss and every gradient against the oracle's layer-by-layer composition, for the forms
    the wide stack does not reach (gradient handed to an earlier layer, biases, odd planes)."""
    import autograph_b200 as ag
    bs, size, spec = STAGE_SPECS[case]
    P = _params(spec, 7300, True)
    x = oracle.round_bf16(np.random.default_rng(7301).standard_normal((bs, 3, size, size)).astype(np.float32))
    t = np.random.default_rng(7302).integers(0, 10, bs).astype(np.uint8)
    model = ag.Model(dev, spec, torch.bfloat16, seed=1)
    model.set_parameters(P)
    xh = torch.from_numpy(x).to(torch.bfloat16).pin_memory()
    loss = model.train_step(xh, torch.from_numpy(t).pin_memory(), 0.01)
    ref_loss, grads, _, _ = models.train_step(spec, P, x, t.astype(np.uint32), 0.01, acc="f64", bf16=True)
    assert abs(loss - ref_loss) <= 3e-2 * abs(ref_loss)
    for i, g in enumerate(grads):
        assert _rel(model.get_gradient(i), g.ravel()) <= 5e-2, i
    model.close()


def test_wide_stack_full_batch_properties(dev):
    """Config 3 at its full batch 256: rows are independent, so the first 8 rows of the
    batch-256 forward equal the batch-8 forward."""
    import autograph_b200 as ag
    dtype = torch.bfloat16
    P = _params(models.WIDE_STACK, 5100, True)
    x = np.random.default_rng(5000).standard_normal((256, 3, 64, 64)).astype(np.float32)
    model = ag.Model(dev, ag.WIDE_STACK_SPEC, dtype, seed=1)
    model.set_parameters(P)
    xh = torch.from_numpy(x).to(dtype).pin_memory()
    full = model.infer(xh).float().numpy()
    part = model.infer(xh[:8].contiguous()).float().numpy()
    assert np.isfinite(full).all()
    assert _rel(full[:8], part) <= 1e-2
    loss = model.train_step(xh, torch.zeros(256, dtype=torch.uint8).pin_memory(), 0.01)
    assert np.isfinite(loss) and loss > 0
    model.close()


def test_default_initialiser_distribution(dev):
    """Parameters are U(-a, a), a = sqrt(2/fan_in) (layer.rs:345-389, 463-503); seeded."""
    import autograph_b200 as ag
    m1 = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=42)
    m2 = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=42)
    m3 = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=43)
    assert m1.parameter_lens == [150, 2400, 32768, 10752, 840, 10]
    fan_in = [25, 150, 256, 128, 84, 84]
    for i, f in enumerate(fan_in):
        w = m1.get_parameter(i)
        a = np.sqrt(2.0 / f)
        assert np.abs(w).max() <= a and np.array_equal(w, m2.get_parameter(i))
        assert not np.array_equal(w, m3.get_parameter(i))
        if w.size > 1000:
            assert abs(w.mean()) < 0.05 * a and abs(w.std() - a / np.sqrt(3)) < 0.05 * a
    for m in (m1, m2, m3):
        m.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_checkpoint_round_trip_in_the_reference_layout(dev, dtype):
    """to_serde_json / load_serde_json: a second model loaded from the text gives the same logits."""
    import autograph_b200 as ag
    names = ["conv1", "relu1", "pool1", "conv2", "relu2", "pool2", "flatten", "dense1", "relu3",
             "dense2", "relu4", "dense3"]
    a = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=21)
    b = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=22)
    x = torch.rand((64, 1, 28, 28)).to(dtype).to(dev.torch_device)
    assert not torch.equal(a.forward_device(x), b.forward_device(x))
    b.load_serde_json(a.to_serde_json(names))
    assert torch.equal(a.forward_device(x), b.forward_device(x))
    a.close()
    b.close()


def test_model_wrappers_refuse_tensors_the_library_would_misread(dev):
    """The C entry points take raw pointers; the Python front end checks dtype, contiguity and
    which side (host / device) a tensor lives on before handing its address over."""
    import autograph_b200 as ag
    m = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=1)
    x = torch.rand((8, 1, 28, 28))
    t = torch.zeros(8, dtype=torch.uint8)
    with pytest.raises(ag.AgError):
        m.infer(x.to(torch.bfloat16))                       # wrong dtype
    with pytest.raises(ag.AgError):
        m.infer(torch.rand((8, 1, 28, 56))[..., ::2])       # not contiguous
    with pytest.raises(ag.AgError):
        m.infer(x.to(dev.torch_device))                     # device tensor where host is expected
    with pytest.raises(ag.AgError):
        m.forward_device(x)                                 # host tensor where device is expected
    with pytest.raises(ag.AgError):
        m.train_step(x, t.to(torch.int64), 0.01)            # labels must be u8
    with pytest.raises(ag.AgError):
        m.train_step(x, t[:4], 0.01)                        # one label per image
    with pytest.raises(ag.AgError):
        m.infer(x, torch.empty((8, 12)))                    # wrong output shape
    assert m.infer(x).shape == (8, 10)
    m.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_momentum_run_survives_a_checkpoint(dev, dtype):
    """The optimizer state (SGD's velocity) is part of the checkpoint: a model restored from the
    text continues a momentum run bit for bit (ParameterBase::optim_state, autograd.rs:647-656)."""
    import autograph_b200 as ag
    names = ["conv1", "relu1", "pool1", "conv2", "relu2", "pool2", "flatten", "dense1", "relu3",
             "dense2", "relu4", "dense3"]
    rng = np.random.default_rng(31)
    x = torch.from_numpy(rng.uniform(0, 1, (64, 1, 28, 28)).astype(np.float32)).to(dtype).pin_memory()
    t = torch.from_numpy(rng.integers(0, 10, 64).astype(np.uint8)).pin_memory()
    a = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=41)
    a.set_sgd(0.9)
    for _ in range(3):
        a.train_step(x, t, 0.05)
    text = a.to_serde_json(names)
    assert '"velocity"' in text
    b = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=42)
    b.set_sgd(0.9)
    b.load_serde_json(text)
    c = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=43)      # restored without its optimizer state
    c.set_sgd(0.9)
    c.set_parameters([a.get_parameter(i) for i in range(len(a.parameter_lens))])
    la, lb, lc = (m.train_step(x, t, 0.05) for m in (a, b, c))
    assert la == lb == lc                                   # same parameters, same loss
    for i in range(len(a.parameter_lens)):
        assert np.array_equal(a.get_parameter(i), b.get_parameter(i)), i
        assert np.array_equal(a.get_velocity(i), b.get_velocity(i)), i
    assert any(not np.array_equal(a.get_parameter(i), c.get_parameter(i))
               for i in range(len(a.parameter_lens)))      # the velocity mattered
    for m in (a, b, c):
        m.close()
