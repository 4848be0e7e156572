"""GPU parity of Unique (the step after a sort) against the CPU oracle, through the C ABI.
Mirrors ILGPU.Algorithms.Tests/UniqueExtensionTests.tt:36-93: values 1..length, each repeated
`repeat` times, cut to `length`; then random data with runs, floats with NaN / signed zeros,
and sizes around the tile edges."""
import numpy as np
import pytest
import torch

from oracle import cpu_oracle as oracle
from tests.helpers import NP, to_device, to_host

pytestmark = pytest.mark.gpu


def _reference_input(np_dtype, repeat, length):
    return np.repeat(np.arange(1, length + 1), repeat)[:length].astype(np_dtype)


def _run(accelerator, host):
    dev = to_device(host)
    count = accelerator.Unique(None, dev)
    return to_host(dev)[:count]


@pytest.mark.parametrize("tname", list(NP.keys()))
@pytest.mark.parametrize("repeat", [1, 317, 1025])
def test_reference_cases(accelerator, tname, repeat):
    for length in (1025, 296 * 1024 + 1024):   # the second exceeds one pass of the reference's grid
        if length > 2000 and NP[tname] in (np.int8, np.uint8, np.float16):
            continue                            # values would wrap / lose precision; covered below
        host = _reference_input(NP[tname], repeat, length)
        expected = oracle.unique(host)
        # the reference test's own expectation: drop an element equal to the last kept one
        keep = np.concatenate([[True], host[1:] != host[:-1]])
        np.testing.assert_array_equal(expected, host[keep])
        np.testing.assert_array_equal(_run(accelerator, host), expected)


@pytest.mark.parametrize("n", [1, 2, 4095, 4096, 4097, 8191, 1_000_003])
def test_random_runs(accelerator, n):
    rng = np.random.default_rng(n)
    host = np.repeat(rng.integers(0, 5, size=n), rng.integers(1, 9, size=n))[:n].astype(np.uint32)
    np.testing.assert_array_equal(_run(accelerator, host), oracle.unique(host))


def test_sorted_zipf_keys_then_unique(accelerator):
    # sort -> unique -> count, the pipeline this primitive exists for
    from ilgpu_b200 import synthetic, RadixSortOperations as Sorts
    n = 1 << 20
    keys = synthetic.zipf_uint64(n, seed=4)
    dev = to_device(keys)
    op = Sorts.AscendingUInt64
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortTempStorageSize(op, n), torch.int32)
    accelerator.CreateRadixSort(op)(None, dev, temp)
    count = accelerator.Unique(None, dev)
    expected = np.unique(keys)
    assert count == expected.size
    np.testing.assert_array_equal(to_host(dev)[:count], expected)


@pytest.mark.parametrize("tname", ["Float", "Double", "Half"])
def test_float_equality_is_compare_to(accelerator, tname):
    t = NP[tname]
    host = np.asarray([0.0, -0.0, 1.0, 1.0, np.nan, np.nan, -np.nan, 2.0, np.inf, np.inf, -np.inf, 0.0] * 700, dtype=t)
    got, expected = _run(accelerator, host), oracle.unique(host)
    assert got.size == expected.size
    np.testing.assert_array_equal(got.view(f"u{host.itemsize}"), expected.view(f"u{host.itemsize}"))


def test_empty_and_count_only_output(accelerator):
    out = torch.full((1,), 7, dtype=torch.int64, device="cuda")
    data = torch.zeros(0, dtype=torch.int32, device="cuda")
    temp = accelerator.Allocate1D(256, torch.int32)
    accelerator.CreateUnique(torch.int32)(None, data, out, temp)
    assert int(out.cpu()[0]) == 0


@pytest.mark.parametrize("tname", ["UInt8", "Int32", "UInt64", "Float", "Half"])
@pytest.mark.parametrize("n", [1, 2, 4095, 4096, 4097, 1_000_003])
def test_run_length_encode(tname, n):
    """values / lengths / number of runs against numpy's run boundaries (equality as in Unique:
    NaNs are equal to each other)."""
    import ctypes
    from ilgpu_b200 import _native as N
    from ilgpu_b200.algorithms import dtype_code
    L = N.lib()
    rng = np.random.default_rng(n)
    host = np.repeat(rng.integers(0, 5, size=n), rng.integers(1, 9, size=n))[:n].astype(NP[tname])
    if tname in ("Float", "Half") and n > 10:
        host[3:6] = np.nan
    dev = to_device(host)
    values = torch.zeros_like(dev)
    lengths = torch.zeros(n, dtype=torch.int64, device="cuda")
    runs = torch.zeros(1, dtype=torch.int64, device="cuda")
    need = ctypes.c_int64(0)
    assert L.b200alg_run_length_encode_temp_bytes(dtype_code(dev.dtype), n, ctypes.byref(need)) == N.OK
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    assert L.b200alg_run_length_encode(None, p(dev), n, dtype_code(dev.dtype), p(values), p(lengths), p(runs), p(temp), need.value) == N.OK
    assert L.b200alg_device_status(None, p(temp)) == N.OK
    same = (host[1:] == host[:-1]) | ((host[1:] != host[1:]) & (host[:-1] != host[:-1]))
    starts = np.concatenate([[0], np.nonzero(~same)[0] + 1])
    m = int(runs.cpu()[0])
    assert m == len(starts)
    np.testing.assert_array_equal(to_host(lengths)[:m], np.diff(np.concatenate([starts, [n]])))
    np.testing.assert_array_equal(to_host(values)[:m].view(np.uint8), host[starts].view(np.uint8))
    np.testing.assert_array_equal(to_host(dev).view(np.uint8), host.view(np.uint8))     # the input is only read
