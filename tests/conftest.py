import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


class Golden:
    """Committed vectors built from the reference's test generators
    (tests/golden/gen_golden.py)."""

    def __init__(self):
        self.z = np.load(ROOT / "tests" / "golden" / "golden_vectors.npz")
        self.meta = json.loads(bytes(self.z["meta"]).decode())

    def __getitem__(self, name):
        return self.z[name]


@pytest.fixture(scope="session")
def golden():
    return Golden()


@pytest.fixture(scope="session")
def dev():
    """One library device on cuda:0 (no CPU fallback: fails without a GPU)."""
    import autograph_b200 as ag
    d = ag.Device(0)
    yield d
    d.wait()


@pytest.fixture(autouse=True)
def _library_stream_is_current(request):
    """torch ops of a GPU test (comparisons, copies) must run on the stream the library's kernels
    run on; a Device created elsewhere in the session would have made its own stream current.

    Every GPU test also runs with the device's memory-safety net on (compute-sanitizer cannot be
    used on these machines): each operator output is allocated between two red zones and
    pre-filled with a poison pattern, and after the test every red zone must be intact and no
    output that is still alive may hold surviving poison (Device.set_guards / check_guards)."""
    if "dev" not in request.fixturenames:
        yield
        return
    import torch
    d = request.getfixturevalue("dev")
    torch.cuda.set_stream(d.stream)
    d.set_guards(True)
    yield
    try:
        d.check_guards()
    finally:
        d.set_guards(False)


def cycle(lo, hi, n):
    return (np.arange(n) % (hi - lo) + lo).astype(np.float32)
