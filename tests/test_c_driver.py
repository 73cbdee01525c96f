"""A caller of the C ABI that is neither Python nor PyTorch: tests/c_driver/lenet5_forward.c is
compiled with gcc against include/autograph_b200.h, linked with libautograph_b200.so, and runs
the derived Forward of the reference's LeNet5 layer by layer and as a model object.
Without a GPU only the build is checked (the header is valid C, every symbol links)."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "c_driver" / "lenet5_forward.c"


def _build(tmp_path):
    exe = tmp_path / "lenet5_forward"
    libdir = ROOT / "autograph_b200"
    cmd = ["gcc", "-std=c11", "-O2", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(SRC),
           "-L", str(libdir), "-lautograph_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_c_driver_builds_against_the_header(tmp_path):
    from autograph_b200 import _capi
    _capi.lib()                               # the library exists (built by __graft_entry__.build)
    exe = _build(tmp_path)
    # without arguments it only prints its usage: the dynamic loader resolved every symbol
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 2 and "usage" in res.stderr


@pytest.mark.gpu
def test_c_driver_matches_the_oracle(tmp_path):
    sys.path.insert(0, str(ROOT))
    from oracle import models
    exe = _build(tmp_path)
    bs = 250
    P = models.init_params(models.LENET5, 2000)
    x = np.random.default_rng(9).uniform(0, 1, (bs, 1, 28, 28)).astype(np.float32)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(np.int32(bs).tobytes())
        f.write(x.tobytes())
        for p in P:
            f.write(np.ascontiguousarray(p, np.float32).tobytes())
    res = subprocess.run([str(exe), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    out = np.fromfile(tmp_path / "out.bin", np.float32).reshape(2, bs, 10)
    ref = models.forward(models.LENET5, P, x)
    ref64 = models.forward(models.LENET5, P, x, acc="f64")
    for y in out:
        assert np.abs(y - ref64).max() <= 1e-5 * np.sqrt(256) * np.abs(ref64).max()
        assert np.array_equal(y.argmax(1), ref.argmax(1))
    # layer by layer (generic dot) and as one kernel: the same values up to summation order
    assert np.abs(out[0] - out[1]).max() <= 1e-5 * np.abs(ref64).max()
