"""CPU: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "autograph_b200.h").read_text()
    return sorted(set(re.findall(r"AG_API\s+[\w\s\*]+?\b(ag_\w+)\s*\(", text)))


def test_header_symbols_exported():
    from autograph_b200 import _capi
    lib = _capi.lib()
    names = _declared()
    assert len(names) >= 45
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    # and the Python declarations cover the same set
    assert sorted(_capi.signatures()) == names


def test_version_and_error_string():
    from autograph_b200 import _capi
    lib = _capi.lib()
    assert b"sm_100a" in lib.ag_version()
    # argument checks that need no GPU
    assert lib.ag_device_count(None) == _capi.AG_ERR_INVALID
    assert b"null" in lib.ag_last_error()
    assert lib.ag_device_wait(None) == _capi.AG_ERR_INVALID
    oh, ow = ctypes.c_int64(), ctypes.c_int64()
    o = _capi.ConvOptions()
    o.filter[0], o.filter[1] = 5, 5
    o.stride[0], o.stride[1] = 1, 1
    o.dilation[0], o.dilation[1] = 1, 1
    assert lib.ag_conv2_output_shape(28, 28, ctypes.byref(o), ctypes.byref(oh), ctypes.byref(ow)) == 0
    assert (oh.value, ow.value) == (24, 24)
    assert lib.ag_conv2_output_shape(3, 3, ctypes.byref(o), ctypes.byref(oh), ctypes.byref(ow)) == \
        _capi.AG_ERR_SHAPE


def test_no_cpu_fallback():
    """Without a GPU, creating a device fails loudly instead of computing on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import autograph_b200 as ag
    with pytest.raises(ag.AgError):
        ag.Device(0)
    h = ctypes.c_void_p()
    assert ag.lib().ag_device_create(0, ctypes.byref(h)) == ag._capi.AG_ERR_CUDA


def test_product_does_not_import_oracle():
    """The shipped package never routes through the oracle."""
    for path in (ROOT / "autograph_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".hpp", ".h"}:
            text = path.read_text()
            assert "import oracle" not in text and "from oracle" not in text, path
            assert "liboracle" not in text, path
