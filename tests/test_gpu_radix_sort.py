"""GPU parity of the radix sort (keys and pairs) against the CPU oracle, through the C ABI.

Mirrors ILGPU.Algorithms.Tests/RadixSortExtensionTests.tt:144-432 (worst case = inverted
ramp, best case = sorted ramp, constants, ascending and descending, provider API, pairs)
and adds what those tests leave unpinned: random keys of every key type, duplicate keys
with payload = index (stability), negative and special float keys, strided views.
Everything is bit-exact.
"""
import numpy as np
import pytest
import torch

from ilgpu_b200 import RadixSortOperations as Ops
from oracle import cpu_oracle as oracle
from tests.helpers import ATOMIC, EDGE_SIZES, NP, REFERENCE_SIZES, compute_inverted_sequence, compute_sequence, to_device, to_host

pytestmark = pytest.mark.gpu

ALL_KEYS = list(NP.keys())


def _sort_keys(accelerator, op, host, stride=1):
    dev = to_device(host)
    view = dev[::stride] if stride != 1 else dev
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortTempStorageSize(op, view.numel()), torch.int32)
    accelerator.CreateRadixSort(op)(None, view, temp)
    accelerator.CheckDeviceStatus(None, temp)
    return to_host(dev)


def _bits(a):
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


@pytest.mark.parametrize("tname", ATOMIC)
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
def test_reference_cases(accelerator, tname, direction):
    op = getattr(Ops, direction + tname)
    t = NP[tname]
    for size in REFERENCE_SIZES:
        ramp = compute_sequence(t, 0, 1, size)
        inverted = compute_inverted_sequence(t, 0, 1, size)
        expected = ramp if direction == "Ascending" else inverted
        for seq in (inverted, ramp):  # worst case, best case
            got = _sort_keys(accelerator, op, seq)
            np.testing.assert_array_equal(got, expected)
            np.testing.assert_array_equal(got, oracle.radix_sort(seq, descending=op.descending)[0])
        consts = [0, 1] + ([] if tname.startswith("U") else [-1])
        for c in consts:
            seq = compute_sequence(t, c, 0, size)
            np.testing.assert_array_equal(_sort_keys(accelerator, op, seq), seq)


@pytest.mark.parametrize("tname", ATOMIC)
def test_pairs_reference_case(accelerator, tname):
    # RadixSortExtensionTests.tt:319-365: keys = values = inverted ramp
    op = getattr(Ops, "Ascending" + tname)
    for size in [127, 1027]:
        seq = compute_inverted_sequence(NP[tname], 0, 1, size)
        keys, values = to_device(seq), to_device(seq)
        provider = accelerator.CreateRadixSortProvider(op, size, values.dtype)
        provider.CreateRadixSortPairs(op)(None, keys, values)
        accelerator.Synchronize()
        ramp = compute_sequence(NP[tname], 0, 1, size)
        np.testing.assert_array_equal(to_host(keys), ramp)
        np.testing.assert_array_equal(to_host(values), ramp)
        provider.Dispose()


def _random_keys(tname, n, seed):
    rng = np.random.default_rng(seed)
    t = NP[tname]
    bits = rng.integers(0, 2 ** (8 * np.dtype(t).itemsize), size=n, dtype=np.uint64, endpoint=False) \
        if np.dtype(t).itemsize < 8 else rng.integers(0, 2 ** 64, size=n, dtype=np.uint64, endpoint=False)
    raw = bits.astype({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[np.dtype(t).itemsize])
    return raw.view(t)


@pytest.mark.parametrize("tname", ALL_KEYS)
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
def test_random_keys_every_type(accelerator, tname, direction):
    # Random bit patterns: for float types this includes negatives, NaNs, infinities and
    # denormals; comparison is on the bit patterns.
    op = getattr(Ops, direction + tname)
    for n in [1027, 8193, 300_007]:
        keys = _random_keys(tname, n, n)
        expected = oracle.radix_sort(keys, descending=op.descending)[0]
        got = _sort_keys(accelerator, op, keys)
        np.testing.assert_array_equal(_bits(got), _bits(expected))


@pytest.mark.parametrize("n", EDGE_SIZES + [(1 << 22) + 11])
def test_uint32_sizes(accelerator, n):
    keys = _random_keys("UInt32", n, n)
    got = _sort_keys(accelerator, Ops.AscendingUInt32, keys)
    np.testing.assert_array_equal(got, np.sort(keys, kind="stable"))


@pytest.mark.parametrize("key_t,val_t", [("UInt64", "UInt32"), ("UInt32", "UInt32"), ("Int32", "Int64"),
                                          ("Float", "UInt32"), ("UInt8", "UInt16"), ("Int16", "UInt8"),
                                          ("Double", "Double")])
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
def test_pairs_stable_with_duplicates(accelerator, key_t, val_t, direction):
    op = getattr(Ops, direction + key_t)
    for n in [4097, 250_003]:
        rng = np.random.default_rng(n)
        keys = rng.integers(0, 50, size=n).astype(NP[key_t])   # heavy duplicates
        if key_t in ("Int32", "Int16", "Float", "Double"):
            keys = (keys - 25).astype(NP[key_t])
        values = np.arange(n).astype(NP[val_t])                 # payload = original index (mod range)
        ek, ev = oracle.radix_sort(keys, values, descending=op.descending)
        dk, dv = to_device(keys), to_device(values)
        temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, dv.dtype, n), torch.int32)
        accelerator.CreateRadixSortPairs(op)(None, dk, dv, temp)
        accelerator.CheckDeviceStatus(None, temp)
        np.testing.assert_array_equal(_bits(to_host(dk)), _bits(ek))
        np.testing.assert_array_equal(to_host(dv), ev)


def test_pairs_16_byte_values(accelerator):
    n = 70_001
    rng = np.random.default_rng(3)
    keys = rng.integers(0, 1000, size=n).astype(np.uint32)
    values = rng.integers(0, 2 ** 63, size=(n, 2)).astype(np.int64)
    order = np.argsort(keys, kind="stable")
    dk = to_device(keys)
    dv = to_device(values.reshape(-1)).view(torch.complex128)  # any 16-byte element type
    op = Ops.AscendingUInt32
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, dv.dtype, n), torch.int32)
    accelerator.CreateRadixSortPairs(op)(None, dk, dv, temp)
    np.testing.assert_array_equal(to_host(dk), keys[order])
    np.testing.assert_array_equal(to_host(dv.view(torch.float64).view(torch.int64)).reshape(n, 2), values[order])


def test_zipf_pairs_skips_constant_digits(accelerator):
    # 64-bit keys whose upper four bytes are all zero: half of the digit passes are skipped.
    from ilgpu_b200 import synthetic
    n = 1 << 20
    keys = synthetic.zipf_uint64(n, seed=4)
    values = np.arange(n, dtype=np.uint32)
    ek, ev = oracle.radix_sort(keys, values)
    dk, dv = to_device(keys), to_device(values)
    op = Ops.AscendingUInt64
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, dv.dtype, n), torch.int32)
    accelerator.CreateRadixSortPairs(op)(None, dk, dv, temp)
    np.testing.assert_array_equal(to_host(dk), ek)
    np.testing.assert_array_equal(to_host(dv), ev)


def test_float_total_order_opt_in(accelerator):
    x = np.asarray([3.5, -1.0, 0.0, -0.0, -7.25, 2.0, np.inf, -np.inf, 1e-40, -1e-40] * 300, dtype=np.float32)
    dev = to_device(x)
    op = Ops.AscendingFloat
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortTempStorageSize(op, x.size), torch.int32)
    accelerator.CreateRadixSort(op, float_total_order=True)(None, dev, temp)
    np.testing.assert_array_equal(to_host(dev), np.sort(x, kind="stable"))


def test_strided_keys(accelerator):
    n, stride = 20_011, 3
    storage = _random_keys("UInt32", n * stride, 99)
    got = _sort_keys(accelerator, Ops.AscendingUInt32, storage, stride=stride)
    expected = storage.copy()
    expected[::stride] = np.sort(storage[::stride])
    np.testing.assert_array_equal(got, expected)   # elements between the strides untouched


def test_literal_two_bit_restatement_agrees(accelerator):
    # the 2-bit, two-kernel CPU path itself (not only its closed form) on a small case
    keys = _random_keys("Int32", 1027, 5)
    literal = oracle.radix_sort(keys, literal=True)[0]
    np.testing.assert_array_equal(_sort_keys(accelerator, Ops.AscendingInt32, keys), literal)


@pytest.mark.parametrize("key_t,seq_name,np_val", [
    ("UInt64", "IndexSequencer", np.int32), ("UInt32", "UInt32Sequencer", np.uint32), ("Int32", "Int64Sequencer", np.int64),
    ("Float", "FloatSequencer", np.float32), ("UInt8", "UInt16Sequencer", np.uint16), ("Int16", "UInt8Sequencer", np.uint8),
    ("Double", "DoubleSequencer", np.float64), ("UInt16", "HalfSequencer", np.float16)])
@pytest.mark.parametrize("direction", ["Ascending", "Descending"])
def test_pairs_with_sequencer_values(accelerator, key_t, seq_name, np_val, direction):
    """The sequencer overload (RadixSortExtensions.cs:1017-1074): the value of element i is
    sequencer.ComputeSequenceElement(i) = the index converted to the value type; the value
    view only receives the result and starts out as garbage here."""
    import ilgpu_b200 as ib
    op = getattr(Ops, direction + key_t)
    seq = getattr(ib.Sequencers, seq_name)
    for n in [1, 4097, 250_003]:
        rng = np.random.default_rng(n)
        keys = rng.integers(0, 50, size=n).astype(NP[key_t])
        if key_t in ("Int32", "Int16", "Float", "Double"):
            keys = (keys - 25).astype(NP[key_t])
        values = np.arange(n).astype(np_val)        # what the sequencer yields (wraps / rounds like the cast)
        ek, ev = oracle.radix_sort(keys, values, descending=op.descending)
        dk = to_device(keys)
        dv = to_device(rng.integers(0, 255, size=n * np.dtype(np_val).itemsize).astype(np.uint8)).view(seq.dtype)
        temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, dv.dtype, n), torch.int32)
        accelerator.CreateRadixSortPairs(op, sequencer=ib.Sequencers)(None, dk, dv, seq, temp)
        accelerator.CheckDeviceStatus(None, temp)
        np.testing.assert_array_equal(_bits(to_host(dk)), _bits(ek))
        np.testing.assert_array_equal(_bits(to_host(dv)), _bits(ev))


def test_pairs_with_sequencer_when_every_key_is_equal(accelerator):
    """No digit pass runs (all keys equal): the values still have to be produced."""
    import ilgpu_b200 as ib
    n = 100_003
    dk = to_device(np.full(n, 7, dtype=np.uint32))
    dv = to_device(np.full(n, 99, dtype=np.int32))
    op = Ops.AscendingUInt32
    temp = accelerator.Allocate1D(accelerator.ComputeRadixSortPairsTempStorageSize(op, dv.dtype, n), torch.int32)
    accelerator.CreateRadixSortPairs(op, sequencer=ib.Sequencers)(None, dk, dv, ib.Sequencers.IndexSequencer, temp)
    np.testing.assert_array_equal(to_host(dv), np.arange(n, dtype=np.int32))
    np.testing.assert_array_equal(to_host(dk), np.full(n, 7, dtype=np.uint32))


@pytest.mark.parametrize("key_t,val_t", [("UInt32", None), ("UInt64", "UInt32"), ("Int16", "Int64"), ("UInt8", None)])
@pytest.mark.parametrize("n,count", [(1, 1), (4097, 4097), (250_003, 250_003), (250_003, 99_999), (250_003, 0), (8192, 8191)])
def test_out_of_place_sort_with_a_device_side_count(accelerator, key_t, val_t, n, count):
    """b200alg_radix_sort_out_of_place: the input stays untouched, only the first *n_device
    elements are sorted into the output, and nothing beyond them is written."""
    import ctypes
    from ilgpu_b200 import _native as N
    from ilgpu_b200.algorithms import dtype_code
    L = N.lib()
    rng = np.random.default_rng(n + count)
    span = 50 if val_t else 2 ** 16
    keys = rng.integers(0, min(span, np.iinfo(NP[key_t]).max), size=n).astype(NP[key_t])
    if key_t == "Int16":
        keys = (keys - 25).astype(NP[key_t])
    values = None if val_t is None else rng.integers(0, 2 ** 31, size=n).astype(NP[val_t])
    dk = to_device(keys)
    dv = None if values is None else to_device(values)
    sentinel_k = np.full(n, 0x5A, dtype=np.uint8).repeat(keys.itemsize).view(NP[key_t])[:n]
    ok = to_device(sentinel_k.copy())
    ov = None if values is None else to_device(np.full(n, 77).astype(NP[val_t]))
    dn = torch.tensor([count], dtype=torch.int64, device="cuda")
    vb = 0 if values is None else values.itemsize
    need = ctypes.c_int64(0)
    assert L.b200alg_radix_sort_temp_bytes(dtype_code(dk.dtype), n, vb, ctypes.byref(need)) == N.OK
    temp = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    rc = L.b200alg_radix_sort_out_of_place(None, p(dk), p(dv), p(ok), p(ov), n, p(dn), dtype_code(dk.dtype), vb, 0,
                                           p(temp), need.value)
    assert rc == N.OK
    assert L.b200alg_device_status(None, p(temp)) == N.OK
    ek, ev = oracle.radix_sort(keys[:count], None if values is None else values[:count])
    np.testing.assert_array_equal(to_host(dk), keys)                       # input untouched
    np.testing.assert_array_equal(to_host(ok)[:count], ek)
    np.testing.assert_array_equal(to_host(ok)[count:], sentinel_k[count:])  # nothing written past the count
    if values is not None:
        np.testing.assert_array_equal(to_host(dv), values)
        np.testing.assert_array_equal(to_host(ov)[:count], ev)
        np.testing.assert_array_equal(to_host(ov)[count:], np.full(n - count, 77).astype(NP[val_t]))
