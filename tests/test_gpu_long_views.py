"""Views longer than int.MaxValue elements, through the C ABI.  The reference refuses them
(ErrorMessages.NotSupportedArrayView64: ScanExtensions.cs:681-685, RadixSortExtensions.cs:
1170-1174) and the host mirrors keep that check; the kernels themselves index with 64 bits.
Checked through properties that do not need a CPU run over 2^31 elements."""
import ctypes

import pytest
import torch

from ilgpu_b200 import _native as N

pytestmark = pytest.mark.gpu

LONG = (1 << 31) + 12_345


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_sort_of_more_than_int32_max_uint8_keys():
    L = N.lib()
    g = torch.Generator(device="cuda").manual_seed(7)
    keys = torch.randint(0, 256, (LONG,), dtype=torch.uint8, device="cuda", generator=g)
    before = torch.bincount(keys[: 1 << 30].to(torch.int32), minlength=256)
    for lo in range(1 << 30, LONG, 1 << 30):
        before += torch.bincount(keys[lo: lo + (1 << 30)].to(torch.int32), minlength=256)
    need = ctypes.c_int64(0)
    assert L.b200alg_radix_sort_temp_bytes(N.U8, LONG, 0, ctypes.byref(need)) == N.OK
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    assert L.b200alg_radix_sort_keys(None, _ptr(keys), LONG, 1, N.U8, 0, _ptr(temp), need.value) == N.OK
    assert L.b200alg_device_status(None, _ptr(temp)) == N.OK
    # ascending, and every value as often as before: that pins the result of a keys-only sort
    ends = torch.cumsum(before, 0)
    starts = ends - before
    for v in range(256):
        if int(before[v]):
            run = keys[int(starts[v]): int(ends[v])]
            assert int(run.min()) == v and int(run.max()) == v


def test_scan_and_reduce_of_more_than_int32_max_elements():
    L = N.lib()
    ones = torch.ones(LONG, dtype=torch.int32, device="cuda")
    out = torch.empty_like(ones)
    need = ctypes.c_int64(0)
    assert L.b200alg_scan_temp_bytes(N.I32, LONG, ctypes.byref(need)) == N.OK
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    assert L.b200alg_scan(None, _ptr(ones), 1, _ptr(out), 1, LONG, N.I32, N.ADD, 0, _ptr(temp), need.value) == N.OK
    assert L.b200alg_device_status(None, _ptr(temp)) == N.OK
    # exclusive scan of ones = the index, wrapping like unchecked int arithmetic
    for lo in range(0, LONG, 1 << 29):
        hi = min(LONG, lo + (1 << 29))
        expect = torch.arange(lo, hi, dtype=torch.int64, device="cuda").to(torch.int32)
        assert torch.equal(out[lo:hi], expect)
        del expect
    cell = torch.zeros(1, dtype=torch.int64, device="cuda")
    wide = ones.to(torch.int64)
    assert L.b200alg_reduce(None, _ptr(wide), 1, LONG, N.I64, N.ADD, _ptr(cell)) == N.OK
    assert int(cell.item()) == LONG
