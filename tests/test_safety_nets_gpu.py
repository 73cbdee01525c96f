"""GPU: the safety nets that stand in for tools these machines cannot run.

* A bounded device-side wait that runs out: the kernel gives up after its limit, records a status
  code and returns; the host gets AG_ERR_DEVICE_TIMEOUT from the next ag_device_wait and the GPU
  stays usable.  Nothing faults, traps or hangs: the wait is on a barrier that nothing completes,
  with the limit lowered to a millisecond.
* The output guards every GPU test runs under (tests/conftest.py): red zones around operator
  outputs and a poison pre-fill catch an operator that writes outside its output or leaves part
  of it unwritten.  Both are provoked here inside the guarded allocation itself, so no access
  leaves memory the test owns.
"""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_device_stays_usable(dev):
    import autograph_b200 as ag
    lib = ag.lib()
    a = dev.tensor(np.random.default_rng(1).uniform(-1, 1, (256, 256)).astype(np.float32), torch.bfloat16)
    want = dev.dot(a, a).clone()
    dev.wait()
    t0 = time.time()
    ag._capi.check(lib.ag_debug_expiring_wait(dev._h, 1_000_000))      # one millisecond
    with pytest.raises(ag.AgError) as err:
        dev.wait()
    assert err.value.status == ag._capi.AG_ERR_DEVICE_TIMEOUT and "199" in err.value.message
    assert time.time() - t0 < 2.0
    dev.wait()                                            # the status word was consumed
    assert torch.equal(dev.dot(a, a), want)               # the tensor-core path still works
    # a limit outside (0, 1 s] is refused on the host
    assert lib.ag_debug_expiring_wait(dev._h, 0) == ag._capi.AG_ERR_INVALID
    assert lib.ag_debug_expiring_wait(dev._h, 5_000_000_000) == ag._capi.AG_ERR_INVALID


def test_guards_catch_a_write_past_the_output(dev):
    import autograph_b200 as ag
    x = torch.rand(1024 + 16, device=dev.torch_device) - 0.5
    y = dev._out((1024,), torch.float32)                  # guarded: 512 bytes of red zone each side
    # relu over 1040 elements into an output of 1024: the last 16 land in the red zone
    ag._capi.check(ag.lib().ag_relu(dev._h, 0, ctypes.c_void_p(x.data_ptr()),
                                    ctypes.c_void_p(y.data_ptr()), 1040))
    with pytest.raises(AssertionError, match="outside its output"):
        dev.check_guards()
    dev.check_guards()                                    # forgotten after the report


def test_guards_catch_an_unwritten_output(dev):
    import autograph_b200 as ag
    x = torch.rand(1024, device=dev.torch_device) - 0.5
    y = dev._out((1024,), torch.float32)
    ag._capi.check(ag.lib().ag_relu(dev._h, 0, ctypes.c_void_p(x.data_ptr()),
                                    ctypes.c_void_p(y.data_ptr()), 1000))   # 24 elements short
    with pytest.raises(AssertionError, match="24 of 1024 elements"):
        dev.check_guards()
    z = dev.relu(x)                                       # a correct call passes
    dev.check_guards()
    assert torch.equal(z, torch.clamp(x, min=0))
