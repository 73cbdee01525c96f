"""GPU: ag_gemm_static_scratch, the split-k product for callers that may not allocate.

Some users of the library run where device memory cannot be requested after start-up
(the host application owns the whole GPU through its own arena, or forbids driver
allocations on its worker threads).  They call this entry point with a device ordinal
and a stream; its partial sums live in a fixed array inside the library.  The test
checks it against ag_gemm on shapes that are split along k, twice in a row (the
array keeps the previous call's contents), and checks the size limit, that device memory
does not change across calls and that the split path is the one taken.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, stream, a, b, c, alpha=1.0, beta=0.0):
    code = {torch.float32: 0, torch.bfloat16: 1}[a.dtype]
    m, k = a.shape
    n = b.shape[1]
    return lib.ag_gemm_static_scratch(
        0, ctypes.c_void_p(stream), code, m, k, n, ctypes.c_float(alpha),
        ctypes.c_void_p(a.data_ptr()), 0, a.stride(0), a.stride(1),
        ctypes.c_void_p(b.data_ptr()), 0, b.stride(0), b.stride(1),
        ctypes.c_float(beta), ctypes.c_void_p(c.data_ptr()), 0, c.stride(0), c.stride(1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_ag_gemm(dev, dtype):
    import autograph_b200 as ag
    lib = ag.lib()
    stream = dev.stream.cuda_stream
    rng = np.random.default_rng(21)
    # (m, k, n, layout): products the SIMT engine splits along k, in the layouts backward uses
    shapes = [(16, 6400, 150, "tn"), (6, 57600, 25, "tn"), (64, 4096, 64, "nn"),
              (100, 3000, 10, "nt"), (33, 1000, 7, "nn")]
    for rep in range(2):  # two calls in a row share the array
        for m, k, n, layout in shapes:
            a = rng.uniform(-1, 1, (m, k) if layout[0] == "n" else (k, m)).astype(np.float32)
            b = rng.uniform(-1, 1, (k, n) if layout[1] == "n" else (n, k)).astype(np.float32)
            ad, bd = dev.tensor(a, dtype), dev.tensor(b, dtype)
            av = ad.t() if layout[0] == "t" else ad
            bv = bd.t() if layout[1] == "t" else bd
            c0 = dev.tensor(rng.uniform(-1, 1, (m, n)).astype(np.float32), dtype)
            want = dev.gemm(0.5, av, bv, 2.0, c0.clone())
            got = c0.clone()
            assert _call(lib, stream, av, bv, got, 0.5, 2.0) == 0, lib.ag_last_error()
            torch.cuda.synchronize()
            ref = 0.5 * (av.double() @ bv.double()) + 2.0 * c0.double()
            tol = 1e-5 * np.sqrt(k) if dtype == torch.float32 else 1e-2
            scale = ref.abs().max().item()
            assert (got.double() - ref).abs().max().item() <= tol * scale
            assert (got.double() - want.double()).abs().max().item() <= tol * scale


def test_static_scratch_allocates_nothing_and_takes_the_split_path(dev):
    """The two properties the entry point exists for: device memory in use does not change
    across calls (after the first call on the GPU has looked up the array), and a product with
    a long k really goes through the array: two kernels, partial sums then their reduction."""
    import autograph_b200 as ag
    lib = ag.lib()
    stream = dev.stream.cuda_stream
    m, k, n = 16, 6400, 150
    a = torch.rand((m, k), device=dev.torch_device) - 0.5
    b = torch.rand((k, n), device=dev.torch_device) - 0.5
    c = torch.zeros((m, n), device=dev.torch_device)
    assert _call(lib, stream, a, b, c) == 0          # first call on this GPU: set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev.index)
    launches0 = ag.kernel_launch_count()
    for _ in range(10):
        assert _call(lib, stream, a, b, c) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(dev.index)
    assert free1 == free0, "device memory in use changed across ag_gemm_static_scratch calls"
    assert ag.kernel_launch_count() - launches0 == 20   # partial sums + reduction per call
    ref = a.double() @ b.double()
    assert (c.double() - ref).abs().max().item() <= 1e-5 * np.sqrt(k) * ref.abs().max().item()


def test_static_scratch_offsets_and_empty_k(dev):
    """Element offsets into larger buffers, and k = 0 with beta != 0 (C = beta * C)."""
    import autograph_b200 as ag
    lib = ag.lib()
    stream = dev.stream.cuda_stream
    rng = np.random.default_rng(22)
    m, k, n = 24, 2048, 40
    oa, ob, oc = 13, 6, 9
    abuf = dev.tensor(rng.uniform(-1, 1, oa + m * k).astype(np.float32))
    bbuf = dev.tensor(rng.uniform(-1, 1, ob + k * n).astype(np.float32))
    cbuf = dev.tensor(rng.uniform(-1, 1, oc + m * n + 5).astype(np.float32))
    c_before = cbuf.clone()
    call = lambda kk, alpha, beta: lib.ag_gemm_static_scratch(
        0, ctypes.c_void_p(stream), 0, m, kk, n, ctypes.c_float(alpha),
        ctypes.c_void_p(abuf.data_ptr()), oa, k, 1, ctypes.c_void_p(bbuf.data_ptr()), ob, n, 1,
        ctypes.c_float(beta), ctypes.c_void_p(cbuf.data_ptr()), oc, n, 1)
    assert call(k, 1.5, -0.5) == 0, lib.ag_last_error()
    torch.cuda.synchronize()
    a = abuf[oa:].reshape(m, k).double()
    b = bbuf[ob:].reshape(k, n).double()
    c0 = c_before[oc:oc + m * n].reshape(m, n).double()
    ref = 1.5 * (a @ b) - 0.5 * c0
    got = cbuf[oc:oc + m * n].reshape(m, n).double()
    assert (got - ref).abs().max().item() <= 1e-5 * np.sqrt(k) * ref.abs().max().item()
    assert torch.equal(cbuf[:oc], c_before[:oc]) and torch.equal(cbuf[oc + m * n:], c_before[oc + m * n:])
    mid = cbuf.clone()
    assert call(0, 1.0, 3.0) == 0, lib.ag_last_error()          # empty sum: C = 3 * C
    torch.cuda.synchronize()
    assert torch.equal(cbuf[oc:oc + m * n], 3.0 * mid[oc:oc + m * n])
    assert torch.equal(cbuf[:oc], c_before[:oc])
    # an ordinal the machine does not have: refused before anything is launched
    n_gpus = torch.cuda.device_count()
    bad = lib.ag_gemm_static_scratch(
        n_gpus, ctypes.c_void_p(stream), 0, m, k, n, ctypes.c_float(1.0),
        ctypes.c_void_p(abuf.data_ptr()), oa, k, 1, ctypes.c_void_p(bbuf.data_ptr()), ob, n, 1,
        ctypes.c_float(0.0), ctypes.c_void_p(cbuf.data_ptr()), oc, n, 1)
    assert bad == ag._capi.AG_ERR_CUDA
    assert torch.cuda.current_device() == dev.index


def test_static_scratch_limits_and_errors(dev):
    import autograph_b200 as ag
    lib = ag.lib()
    stream = dev.stream.cuda_stream
    a = dev.empty((1024, 8), torch.float32)
    b = dev.empty((8, 1024), torch.float32)
    c = dev.empty((1024, 1024), torch.float32)
    assert _call(lib, stream, a, b, c) == ag._capi.AG_ERR_LIMIT
    assert b"static scratch limit" in lib.ag_last_error()
    small = dev.empty((4, 8), torch.float32)
    bad_dtype = lib.ag_gemm_static_scratch(
        0, ctypes.c_void_p(stream), 3, 4, 8, 4, ctypes.c_float(1.0),
        ctypes.c_void_p(small.data_ptr()), 0, 8, 1, ctypes.c_void_p(small.data_ptr()), 0, 1, 8,
        ctypes.c_float(0.0), ctypes.c_void_p(small.data_ptr()), 0, 4, 1)
    assert bad_dtype == ag._capi.AG_ERR_DTYPE
    e = dev.empty((0, 8), torch.float32)
    assert _call(lib, stream, e, b[:, :4], dev.empty((0, 4), torch.float32)) == 0
