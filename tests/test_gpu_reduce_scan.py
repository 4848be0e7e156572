"""GPU parity of reduce and scan against the CPU oracle (through the C ABI).

Mirrors ILGPU.Algorithms.Tests/ReductionExtensionTests.tt:119-198 and
ScanExtensionTests.tt:122-282: ramps, constants, every operation and element type, the
provider API and strided views; then seeded random data at sizes around the tile edges.
Integer results must be bit-exact.  Float tolerance: |gpu - ref| <= 1e-5 * log2(n) * sum|x|.
"""
import math

import numpy as np
import pytest
import torch

from ilgpu_b200 import ScanKind, ScanReduceOperations as Ops
from ilgpu_b200 import ArgumentOutOfRangeException, ArgumentNullException
from oracle import cpu_oracle as oracle
from tests.helpers import ATOMIC, EDGE_SIZES, NP, REFERENCE_SIZES, compute_sequence, to_device, to_host

pytestmark = pytest.mark.gpu

OPS = ["Add", "Max", "Min"]


def _float_tol(x: np.ndarray) -> float:
    n = max(2, x.size)
    return 1e-5 * math.log2(n) * float(np.abs(x.astype(np.float64)).sum()) + 1e-30


def _check(got: np.ndarray, ref: np.ndarray, src: np.ndarray, op: str):
    if got.dtype.kind in "iu":
        np.testing.assert_array_equal(got, ref)
    elif op == "Add":
        assert np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64))) <= _float_tol(src)
    else:  # max / min never round
        np.testing.assert_array_equal(got, ref)


def _sequences(tname, size):
    t = NP[tname]
    yield "ascending", compute_sequence(t, 0, 1, size)
    if not tname.startswith("U"):
        yield "descending", compute_sequence(t, 0, -1, size)
        yield "const-1", compute_sequence(t, -1, 0, size)
    yield "const0", compute_sequence(t, 0, 0, size)
    yield "const1", compute_sequence(t, 1, 0, size)


@pytest.mark.parametrize("tname", ATOMIC)
@pytest.mark.parametrize("op", OPS)
def test_reduce_reference_cases(accelerator, tname, op):
    operation = getattr(Ops, op + tname)
    for size in REFERENCE_SIZES:
        if tname == "Float" and size > 1000:
            continue  # the reference skips these (ReductionExtensionTests.tt:51)
        for label, seq in _sequences(tname, size):
            ref = oracle.reduce(seq, op.lower())
            got = accelerator.Reduce(None, to_device(seq), operation)
            out = accelerator.Allocate1D(1, operation.dtype)
            accelerator.Reduce(None, to_device(seq), operation, out)
            accelerator.Synchronize()
            for g in (np.asarray(got, dtype=seq.dtype), to_host(out)[0]):
                _check(np.asarray([g]), np.asarray([ref]), seq, op)


@pytest.mark.parametrize("tname", ATOMIC)
@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("kind", [ScanKind.Inclusive, ScanKind.Exclusive])
def test_scan_reference_cases(accelerator, tname, op, kind):
    operation = getattr(Ops, op + tname)
    scan = accelerator.CreateScan(operation, kind)
    for size in REFERENCE_SIZES:
        if tname == "Float" and size > 1000:
            continue  # ScanExtensionTests.tt:52
        temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(operation.dtype, size), torch.int32)
        for label, seq in _sequences(tname, size):
            ref = oracle.scan(seq, op.lower(), kind == ScanKind.Inclusive)
            src = to_device(seq)
            dst = torch.zeros_like(src)
            scan(None, src, dst, temp)
            accelerator.CheckDeviceStatus(None, temp)
            _check(to_host(dst), ref, seq, op)


def _random(tname, n, seed):
    rng = np.random.default_rng(seed)
    t = NP[tname]
    if tname in ("Float", "Double"):
        return (rng.random(n) * 2 - 0.5).astype(t)
    info = np.iinfo(t)
    return rng.integers(info.min, info.max, size=n, dtype=t, endpoint=True)


@pytest.mark.parametrize("tname", ATOMIC)
@pytest.mark.parametrize("op", OPS)
def test_reduce_random_edges(accelerator, tname, op):
    operation = getattr(Ops, op + tname)
    for n in EDGE_SIZES + [1 << 20, (1 << 22) + 5]:
        x = _random(tname, n, n)
        ref = oracle.reduce(x, op.lower())
        got = np.asarray([accelerator.Reduce(None, to_device(x), operation)], dtype=x.dtype)
        _check(got, np.asarray([ref]), x, op)
        if x.dtype.kind == "f" and op == "Add":  # also against float64 truth
            assert abs(float(got[0]) - float(x.astype(np.float64).sum())) <= _float_tol(x)


@pytest.mark.parametrize("tname", ATOMIC)
@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("kind", [ScanKind.Inclusive, ScanKind.Exclusive])
def test_scan_random_edges(accelerator, tname, op, kind):
    operation = getattr(Ops, op + tname)
    scan = accelerator.CreateScan(operation, kind)
    for n in EDGE_SIZES + [(1 << 20) + 3]:
        x = _random(tname, n, n + 1)
        ref = oracle.scan(x, op.lower(), kind == ScanKind.Inclusive)
        src = to_device(x)
        dst = torch.empty_like(src)
        temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(operation.dtype, n), torch.int32)
        scan(None, src, dst, temp)
        accelerator.CheckDeviceStatus(None, temp)
        _check(to_host(dst), ref, x, op)


def test_scan_in_place_and_provider(accelerator):
    n = 50_001
    x = _random("Int32", n, 7)
    provider = accelerator.CreateScanProvider(torch.int32, n)
    scan = provider.CreateScan(Ops.AddInt32, ScanKind.Exclusive)
    buf = to_device(x)
    scan(None, buf, buf)
    accelerator.Synchronize()
    np.testing.assert_array_equal(to_host(buf), oracle.scan(x, "add", False))
    provider.Dispose()


@pytest.mark.parametrize("tname", ["Int32", "Double"])
def test_strided_views(accelerator, tname):
    # Stride1D.General views as in ScanExtensionTests.tt:148-154
    n, stride = 10_007, 3
    x = _random(tname, n * stride, 11)
    storage = to_device(x)
    view = storage[::stride]
    assert view.stride(0) == stride
    op = getattr(Ops, "Add" + tname)
    ref_red = oracle.reduce(x, "add", stride=stride)
    got_red = np.asarray([accelerator.Reduce(None, view, op)], dtype=x.dtype)
    _check(got_red, np.asarray([ref_red]), x[::stride], "Add")
    out_storage = torch.zeros(n * 2, dtype=storage.dtype, device="cuda")
    out_view = out_storage[::2]
    temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(op.dtype, n), torch.int32)
    accelerator.CreateScan(op, ScanKind.Inclusive)(None, view, out_view, temp)
    ref = oracle.scan(x, "add", True, in_stride=stride, out_stride=2)
    _check(to_host(out_storage)[: ref.size], ref, x[::stride], "Add")


def test_unaligned_dense_views(accelerator):
    # A sub-view that starts 4 bytes into an allocation is dense but not 16-byte aligned.
    n = 70_001
    x = _random("Int32", n + 1, 13)
    storage = to_device(x)
    view = storage[1:]
    assert accelerator.Reduce(None, view, Ops.AddInt32) == oracle.reduce(x[1:], "add")
    out = torch.empty(n + 3, dtype=torch.int32, device="cuda")[3:]
    temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(torch.int32, n), torch.int32)
    accelerator.CreateScan(Ops.AddInt32, ScanKind.Inclusive)(None, view, out, temp)
    np.testing.assert_array_equal(to_host(out), oracle.scan(x[1:], "add", True))


def test_scan_carry_in(accelerator):
    n = 33_333
    x = _random("Int64", n, 5)
    carry = to_device(np.asarray([12345], dtype=np.int64))
    src = to_device(x)
    dst = torch.empty_like(src)
    temp = accelerator.Allocate1D(accelerator.ComputeScanTempStorageSize(torch.int64, n), torch.int32)
    accelerator.CreateScan(Ops.AddInt64, ScanKind.Exclusive)(None, src, dst, temp, carry_in=carry)
    ref = oracle.scan(x, "add", False) + np.int64(12345)
    np.testing.assert_array_equal(to_host(dst), ref)


def test_argument_errors(accelerator):
    x = to_device(np.arange(8, dtype=np.int32))
    temp = accelerator.Allocate1D(1024, torch.int32)
    scan = accelerator.CreateScan(Ops.AddInt32, ScanKind.Inclusive)
    with pytest.raises(ArgumentNullException):
        scan(None, None, x, temp)
    with pytest.raises(ArgumentOutOfRangeException):
        scan(None, x, x[:4], temp)
    with pytest.raises(ArgumentOutOfRangeException):
        scan(None, x, x, temp[:2])
    with pytest.raises(ArgumentOutOfRangeException):
        accelerator.CreateReduction(Ops.AddInt32)(None, x[:0], x)
    with pytest.raises(ArgumentNullException):
        accelerator.CreateReduction(Ops.AddInt32)(None, x, None)
