"""The five benchmark configurations at their full sizes on one GPU, checked through
properties that do not need a CPU pass over the whole input: sortedness plus a checksum,
stability of equal keys, linearity of the histogram over chunks, scan values against
float64 / int64 sums at sampled positions, idempotence of sorting a sorted array.  (The
element-by-element comparison with the oracle is done at smaller sizes in the other files.)"""
import math

import numpy as np
import pytest
import torch

import ilgpu_b200 as ib
from ilgpu_b200 import synthetic
from oracle import cpu_oracle as oracle

pytestmark = pytest.mark.gpu
Ops, Sorts = ib.ScanReduceOperations, ib.RadixSortOperations


def _u32_as_i64(t):
    return t.view(torch.int32).to(torch.int64) & 0xFFFFFFFF


def test_config1_reduce_and_exclusive_scan_int32_2_24(accelerator):
    n = 1 << 24
    x = synthetic.uniform_int32_device(n, 1, "cuda")
    host = x.cpu().numpy()
    assert np.array_equal(host[:4096], synthetic.uniform_int32(4096, 1))          # device generator = host generator
    assert accelerator.Reduce(None, x, Ops.AddInt32) == int(oracle.reduce(host, "add"))   # bit-exact vs the oracle
    out = torch.empty_like(x)
    temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(torch.int32, n), torch.int32)
    accelerator.CreateScan(Ops.AddInt32, ib.ScanKind.Exclusive)(None, x, out, temp)
    accelerator.CheckDeviceStatus(None, temp)
    assert np.array_equal(out.cpu().numpy(), oracle.scan(host, "add", False))      # bit-exact vs the oracle


def test_config2_radix_sort_uint32_2_26(accelerator):
    n = 1 << 26
    keys = synthetic.uniform_uint32_device(n, 2, "cuda")
    checksum = int(_u32_as_i64(keys).sum())
    xor = int(torch.bitwise_xor(keys.view(torch.int32)[: n // 2], keys.view(torch.int32)[n // 2:]).sum())
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortTempStorageSize(Sorts.AscendingUInt32, n), torch.int32)
    sort = accelerator.CreateRadixSort(Sorts.AscendingUInt32)
    sort(None, keys, temp)
    accelerator.CheckDeviceStatus(None, temp)
    k = _u32_as_i64(keys)
    assert bool((k[1:] >= k[:-1]).all())
    assert int(k.sum()) == checksum
    # the first 2^20 sorted keys equal the smallest 2^20 of the oracle's sort of the same input
    host_sorted = oracle.radix_sort(synthetic.uniform_uint32(n, 2))[0]
    assert np.array_equal(keys[: 1 << 20].cpu().numpy(), host_sorted[: 1 << 20])
    assert np.array_equal(keys[-(1 << 20):].cpu().numpy(), host_sorted[-(1 << 20):])
    before = keys.clone()
    sort(None, keys, temp)                                  # idempotence
    assert torch.equal(keys.view(torch.int32), before.view(torch.int32))
    del xor


def test_config3_histogram_float32_2_28(accelerator):
    n = 1 << 28
    x = synthetic.normal_float32_device(n, 3, "cuda")
    loc = ib.EqualWidthClampLocator(-4.0, 4.0)
    bins = torch.zeros(256, dtype=torch.int32, device="cuda")
    ovf = torch.zeros(1, dtype=torch.int32, device="cuda")
    accelerator.Histogram(None, x, bins, ovf, loc)
    assert int(bins.sum()) == n and int(ovf[0]) == 0
    # linearity: the histogram of the whole equals the sum of the histograms of 7 uneven chunks
    parts = torch.zeros(256, dtype=torch.int32, device="cuda")
    cuts = [0, 1, 1 << 10, (1 << 20) + 3, 100_000_007, 200_000_001, n - 5, n]
    for a, b in zip(cuts[:-1], cuts[1:]):
        accelerator.HistogramUnchecked(None, x[a:b], parts, loc)
    assert torch.equal(bins, parts)
    # the first 2^22 elements against the oracle, bit-exact
    head = torch.zeros(256, dtype=torch.int32, device="cuda")
    accelerator.HistogramUnchecked(None, x[: 1 << 22], head, loc)
    expected, _ = oracle.histogram(x[: 1 << 22].cpu().numpy(), np.zeros(256, np.int32), "equal_width_clamp", -4.0, 4.0)
    assert np.array_equal(head.cpu().numpy(), expected)


def test_config4_radix_sort_pairs_uint64_zipf_2_28(accelerator):
    n = 1 << 28
    keys = synthetic.zipf_uint64_device(n, 4, "cuda")
    key_sum = int(keys.view(torch.int64).sum())
    values = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
    op = Sorts.AscendingUInt64
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, torch.uint32, n), torch.int32)
    original = keys.clone()
    accelerator.CreateRadixSortPairs(op)(None, keys, values, temp)
    accelerator.CheckDeviceStatus(None, temp)
    k = keys.view(torch.int64)
    assert bool((k[1:] >= k[:-1]).all())
    assert int(k.sum()) == key_sum
    v = values.view(torch.int32).to(torch.int64)
    assert int(v.sum()) == n * (n - 1) // 2                       # a permutation of the payload
    equal = k[1:] == k[:-1]
    assert int(equal.sum()) > n // 2                              # heavy duplicates, as configured
    assert bool((v[1:][equal] > v[:-1][equal]).all())             # stable: equal keys keep input order
    assert torch.equal(original.view(torch.int64)[v], k)          # every payload still sits beside its key


def test_config5_reduce_and_inclusive_scan_float32_2_30(accelerator):
    n = 1 << 30
    x = synthetic.uniform_float32_device(n, 5, "cuda")
    chunk = 1 << 24
    chunk_sums = torch.stack([x[i:i + chunk].double().sum() for i in range(0, n, chunk)])
    total = float(chunk_sums.sum())
    tol = 1e-5 * math.log2(n) * total                            # x >= 0, so sum|x| = sum x
    got = accelerator.Reduce(None, x, Ops.AddFloat)
    assert abs(got - total) <= tol
    out = torch.empty_like(x)
    temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(torch.float32, n), torch.int32)
    accelerator.CreateScan(Ops.AddFloat, ib.ScanKind.Inclusive)(None, x, out, temp)
    accelerator.CheckDeviceStatus(None, temp)
    # non-negative input: monotone up to float32 rounding of the partial prefixes (some ulp of the total)
    ulp = 2.0 ** (math.floor(math.log2(total)) - 23)
    assert float((out[:-1] - out[1:]).max()) <= 32 * ulp
    ends = torch.cumsum(chunk_sums, 0)                            # float64 truth at the chunk ends
    at_ends = out[chunk - 1::chunk].double()
    assert float((at_ends - ends).abs().max()) <= tol
    # inside one chunk in the middle of the array, element by element
    mid = (n // 2 // chunk) * chunk
    truth = ends[mid // chunk - 1] + torch.cumsum(x[mid:mid + chunk].double(), 0)
    assert float((out[mid:mid + chunk].double() - truth).abs().max()) <= tol


def test_more_than_2_30_keys_use_the_wide_look_back_words(accelerator):
    # from 2^30 keys on, the per-digit tile counts no longer fit 30 bits: the 64-bit status path
    n = (1 << 30) + 12345
    keys = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=torch.Generator("cuda").manual_seed(9))
    hist = torch.zeros(256, dtype=torch.int64, device="cuda")
    chunk = 1 << 28
    for i in range(0, n, chunk):
        hist += torch.bincount(keys[i:i + chunk].to(torch.int64), minlength=256)
    op = Sorts.AscendingUInt8
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortTempStorageSize(op, n), torch.int32)
    accelerator.CreateRadixSort(op)(None, keys, temp)
    accelerator.CheckDeviceStatus(None, temp)
    # a sorted array of bytes is the run-length expansion of its histogram
    ends = torch.cumsum(hist, 0)
    starts = ends - hist
    for d in (0, 1, 17, 128, 254, 255):
        a, b = int(starts[d]), int(ends[d])
        if b > a:
            assert int(keys[a]) == d and int(keys[b - 1]) == d
            if a > 0:
                assert int(keys[a - 1]) < d
    probe = keys[::4099].to(torch.int16)
    assert bool((probe[1:] >= probe[:-1]).all())
