"""GPU checks of the helpers on the edges of the path, through the C ABI: the fill and iota
kernels (InitializeExtensions.cs:116-180, SequenceExtensions.cs:392-419 with the integer
sequencers of Sequencers.tt:26-38) against numpy, and a device-side wait that really runs out."""
import ctypes

import numpy as np
import pytest
import torch

from ilgpu_b200 import _native as N
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("elem_bytes", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("n,stride", [(1, 1), (33, 1), (1027, 1), (100_003, 1), (1027, 3), (4096, 2)])
def test_initialize_fills_exactly_the_view(elem_bytes, n, stride):
    L = N.lib()
    rng = np.random.default_rng(elem_bytes * 1000 + n)
    storage = rng.integers(0, 256, size=((n - 1) * stride + 1 + 5) * elem_bytes, dtype=np.uint8)
    value = rng.integers(1, 256, size=elem_bytes, dtype=np.uint8)
    expected = storage.copy().reshape(-1, elem_bytes)
    expected[0:(n - 1) * stride + 1:stride] = value
    dev = torch.from_numpy(storage).cuda()
    rc = L.b200alg_initialize(None, _ptr(dev), stride, n, elem_bytes, ctypes.c_void_p(value.ctypes.data))
    assert rc == N.OK
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dev.cpu().numpy().reshape(-1, elem_bytes), expected)


def test_initialize_rejects_bad_element_sizes_without_crashing():
    L = N.lib()
    dev = torch.zeros(64, dtype=torch.uint8, device="cuda")
    one = ctypes.c_uint64(1)
    for bad in (0, 3, -4, 32):
        assert L.b200alg_initialize(None, _ptr(dev), 1, 4, bad, ctypes.byref(one)) == N.UNSUPPORTED


@pytest.mark.parametrize("tname,code", [("int32", N.I32), ("uint32", N.U32), ("int64", N.I64), ("uint64", N.U64)])
@pytest.mark.parametrize("n", [1, 31, 1027, 1_000_003])
@pytest.mark.parametrize("start,step", [(0, 1), (-7, 3), (2 ** 31 - 5, 1), (5, -2)])
def test_sequence_matches_the_integer_sequencers(tname, code, n, start, step):
    L = N.lib()
    np_dtype = np.dtype(tname)
    dev = torch.zeros(n, dtype=getattr(torch, tname), device="cuda")
    assert L.b200alg_sequence(None, _ptr(dev), n, code, start, step) == N.OK
    torch.cuda.synchronize()
    with np.errstate(over="ignore"):
        wide = np.arange(n, dtype=np.int64) * np.int64(step) + np.int64(start)     # wraps like unchecked C# casts
    expected = wide.astype(np_dtype) if np_dtype.itemsize == 8 else wide.astype(np.int64).astype(np_dtype)
    got = dev.cpu().numpy() if tname in ("int32", "int64") else dev.view(getattr(torch, tname.replace("u", ""))).cpu().numpy().view(np_dtype)
    np.testing.assert_array_equal(got, expected)


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    """One warp polls a word nobody sets, with the bounded wait of the look-back loops and a
    limit of 1000 polls: the kernel records the give-up and returns, the status query reports
    it, and a scan on the same temp afterwards is correct and reports success."""
    L = N.lib()
    L.b200alg_testing_wait_limit.restype = ctypes.c_int
    L.b200alg_testing_wait_limit.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint]
    n = 300_001
    need = ctypes.c_int64(0)
    assert L.b200alg_scan_temp_bytes(N.I32, n, ctypes.byref(need)) == N.OK
    temp = torch.empty(need.value // 4 + 64, dtype=torch.int32, device="cuda")
    assert L.b200alg_testing_wait_limit(None, _ptr(temp), temp.numel() * 4, 1000) == N.OK
    assert L.b200alg_device_status(None, _ptr(temp)) == N.WAIT_LIMIT
    host = np.random.default_rng(9).integers(-50, 50, size=n).astype(np.int32)
    src = torch.from_numpy(host).cuda()
    out = torch.empty_like(src)
    assert L.b200alg_scan(None, _ptr(src), 1, _ptr(out), 1, n, N.I32, N.ADD, 1, _ptr(temp), temp.numel() * 4) == N.OK
    assert L.b200alg_device_status(None, _ptr(temp)) == N.OK
    np.testing.assert_array_equal(out.cpu().numpy(), oracle.scan(host, "add", True))
