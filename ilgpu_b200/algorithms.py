"""Host-side mirror of the ILGPU.Algorithms surface for radix sort, scan, reduce and
histogram, bound to the native B200 library.

Names, argument meaning and error behaviour follow the reference (paths inside the ILGPU
source tree, ``Src/ILGPU.Algorithms``):

* ``Accelerator.CreateRadixSort`` / ``CreateRadixSortPairs`` / ``CreateRadixSortProvider``
  and the temp-size helpers - RadixSortExtensions.cs:37-160, :168-300, :384-447, :1017-1437
* ``Accelerator.CreateScan`` / ``CreateScanProvider`` / ``ComputeScanTempStorageSize`` and
  ``ScanKind`` - ScanExtensions.cs:27-170, :930-991
* ``Accelerator.CreateReduction`` / ``Reduce`` - ReductionExtensions.cs:135-309
* ``Accelerator.CreateHistogram`` / ``Histogram`` / ``HistogramUnchecked`` -
  HistogramExtensions.cs:293-508, HistogramLaunchers.tt:52-101
* operation types ``Add/Max/Min{Int32,Int64,UInt32,UInt64,Float,Double}`` -
  ScanReduceOperations.tt:20-74; ``Ascending*/Descending*`` - RadixSortOperations.tt:26-125

An ``ArrayView1D<T, TStride>`` is a one-dimensional ``torch`` CUDA tensor (its stride is
the view's stride; dense = 1); ``ArrayView<int>`` temp views are int32 tensors.  A stream
argument is a ``torch.cuda.Stream`` or ``None`` (= the current stream).  PyTorch only
supplies device memory and streams; all computing is done by the CUDA library.
"""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass

import torch

from . import _native as N


# ---- exceptions (C# names kept so that tests read like the reference's) -----------------
class ArgumentNullException(ValueError):
    pass


class ArgumentOutOfRangeException(ValueError):
    pass


class NotSupportedException(RuntimeError):
    pass


class InvalidOperationException(RuntimeError):
    pass


class B200AlgException(RuntimeError):
    """A non-zero status from the native library (pattern: CuRandException.ThrowIfFailed,
    Runtime/Cuda/CuRandException.cs:98-103)."""

    def __init__(self, status: int):
        self.status = status
        msg = N.status_string(status)
        if status == N.CUDA_ERROR:
            msg += f" [cudaError {N.lib().b200alg_last_cuda_error()}]"
        super().__init__(f"b200alg status {status}: {msg}")

    @staticmethod
    def ThrowIfFailed(status: int) -> None:
        if status == N.OK:
            return
        if status == N.TOO_LARGE:
            raise NotSupportedException("NotSupportedArrayView64")
        if status == N.TEMP_TOO_SMALL:
            raise ArgumentOutOfRangeException("temp")
        if status == N.UNSUPPORTED:
            raise NotSupportedException(N.status_string(status))
        raise B200AlgException(status)


# ---- element types ------------------------------------------------------------------------
_TORCH_TO_CODE = {
    torch.int8: N.I8, torch.uint8: N.U8, torch.int16: N.I16, torch.uint16: N.U16,
    torch.int32: N.I32, torch.uint32: N.U32, torch.int64: N.I64, torch.uint64: N.U64,
    torch.float16: N.F16, torch.float32: N.F32, torch.float64: N.F64,
}
_TYPE_NAMES = {
    "Int8": torch.int8, "UInt8": torch.uint8, "Int16": torch.int16, "UInt16": torch.uint16,
    "Int32": torch.int32, "UInt32": torch.uint32, "Int64": torch.int64, "UInt64": torch.uint64,
    "Half": torch.float16, "Float": torch.float32, "Double": torch.float64,
}
_ATOMIC_NUMERIC = ("Int32", "Int64", "UInt32", "UInt64", "Float", "Double")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _TORCH_TO_CODE[dtype]
    except KeyError:
        raise NotSupportedException(f"element type {dtype}") from None


@dataclass(frozen=True)
class ScanReduceOperation:
    """IScanReduceOperation<T> restricted to the built-in structs."""
    name: str
    dtype: torch.dtype
    op: int

    @property
    def Identity(self):
        info = torch.finfo(self.dtype) if self.dtype.is_floating_point else torch.iinfo(self.dtype)
        return {N.ADD: 0, N.MAX: info.min, N.MIN: info.max}[self.op]


@dataclass(frozen=True)
class RadixSortOperation:
    """IRadixSortOperation<T> restricted to the built-in Ascending*/Descending* structs."""
    name: str
    dtype: torch.dtype
    descending: bool

    @property
    def NumBits(self) -> int:
        return self.dtype.itemsize * 8


class ScanReduceOperations:
    pass


class RadixSortOperations:
    pass


for _tn in _ATOMIC_NUMERIC:
    for _on, _oc in (("Add", N.ADD), ("Max", N.MAX), ("Min", N.MIN)):
        setattr(ScanReduceOperations, _on + _tn, ScanReduceOperation(_on + _tn, _TYPE_NAMES[_tn], _oc))
for _tn, _td in _TYPE_NAMES.items():
    setattr(RadixSortOperations, "Ascending" + _tn, RadixSortOperation("Ascending" + _tn, _td, False))
    setattr(RadixSortOperations, "Descending" + _tn, RadixSortOperation("Descending" + _tn, _td, True))


@dataclass(frozen=True)
class Sequencer:
    """ISequencer<T> restricted to the reference's built-in, stateless sequencers
    (Sequencer.cs:37-72, Sequencers.tt:26-38): element i is the index converted to T."""
    name: str
    dtype: torch.dtype


class Sequencers:
    IndexSequencer = Sequencer("IndexSequencer", torch.int32)
    HalfSequencer = Sequencer("HalfSequencer", torch.float16)
    FloatSequencer = Sequencer("FloatSequencer", torch.float32)
    DoubleSequencer = Sequencer("DoubleSequencer", torch.float64)


for _tn in ("Int8", "UInt8", "Int16", "UInt16", "Int32", "UInt32", "Int64", "UInt64"):
    setattr(Sequencers, _tn + "Sequencer", Sequencer(_tn + "Sequencer", _TYPE_NAMES[_tn]))


class ScanKind(enum.Enum):
    """ScanExtensions.cs:27-38."""
    Inclusive = 0
    Exclusive = 1


@dataclass(frozen=True)
class EqualWidthClampLocator:
    """Named bin locator: equal-width bins over [lo, hi), values outside clamp to the edge
    bins, NaN goes to bin 0 (see include/b200alg.h)."""
    lo: float
    hi: float
    code: int = N.LOCATOR_EQUAL_WIDTH_CLAMP


@dataclass(frozen=True)
class ModuloLocator:
    """The reference tests' ModuloBin*Operation (ILGPU.Algorithms.Tests/HistogramTests.tt:83-94)."""
    lo: float = 0.0
    hi: float = 1.0
    code: int = N.LOCATOR_MODULO


# ---- helpers --------------------------------------------------------------------------------
def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _check_view(view, name: str, dtype: torch.dtype | None = None) -> None:
    if view is None or not isinstance(view, torch.Tensor):
        raise ArgumentNullException(name)
    if view.dim() != 1:
        raise ArgumentOutOfRangeException(f"{name}: one-dimensional view expected")
    if not view.is_cuda:
        raise InvalidOperationException(f"{name}: the view is not in CUDA device memory")
    if dtype is not None and view.dtype != dtype:
        raise InvalidOperationException(f"{name}: element type {view.dtype}, expected {dtype}")
    if view.numel() > 1 and view.stride(0) < 1:
        raise ArgumentOutOfRangeException(f"{name}: stride")


def _stride(view: torch.Tensor) -> int:
    return view.stride(0) if view.numel() > 1 else 1


def _ptr(view: torch.Tensor | None):
    return None if view is None else ctypes.c_void_p(view.data_ptr())


def _check_temp(temp, required_ints: int) -> None:
    # TempViewManager (TempViewManager.cs:36-37, :84-112): a valid int view that is large enough.
    _check_view(temp, "temp", torch.int32)
    if _stride(temp) != 1:
        raise ArgumentOutOfRangeException("temp: dense view expected")
    if temp.numel() < required_ints:
        raise ArgumentOutOfRangeException("temp")
    if temp.data_ptr() % 256:
        raise InvalidOperationException("temp: the temporary view must start on a 256-byte boundary")


def _ints(nbytes: int) -> int:
    n = (nbytes + 3) // 4
    if n > 2**31 - 1:
        raise NotSupportedException("temporary storage exceeds the Index1D range")
    return n


# ---- providers ------------------------------------------------------------------------------
class RadixSortProvider:
    """RadixSortExtensions.cs:168-300: owns a temp buffer, hands out sort delegates bound to it."""

    def __init__(self, accelerator: "Accelerator", temp_ints: int):
        self.Accelerator = accelerator
        self._temp = accelerator.Allocate1D(max(int(temp_ints), 64), torch.int32)

    @property
    def TempView(self) -> torch.Tensor:
        return self._temp

    def CreateRadixSort(self, operation: RadixSortOperation):
        sort = self.Accelerator.CreateRadixSort(operation)
        return lambda stream, view: sort(stream, view, self._temp)

    def CreateRadixSortPairs(self, operation: RadixSortOperation):
        sort = self.Accelerator.CreateRadixSortPairs(operation)
        return lambda stream, keys, values: sort(stream, keys, values, self._temp)

    def Dispose(self) -> None:
        self._temp = None


class ScanProvider:
    """ScanExtensions.cs:84-142."""

    def __init__(self, accelerator: "Accelerator", temp_ints: int):
        self.Accelerator = accelerator
        self._temp = accelerator.Allocate1D(max(int(temp_ints), 64), torch.int32)

    @property
    def TempView(self) -> torch.Tensor:
        return self._temp

    def CreateScan(self, operation: ScanReduceOperation, kind: ScanKind):
        scan = self.Accelerator.CreateScan(operation, kind)
        return lambda stream, input, output: scan(stream, input, output, self._temp)

    def Dispose(self) -> None:
        self._temp = None


# ---- the accelerator -------------------------------------------------------------------------
class Accelerator:
    """A CUDA accelerator with the algorithm extensions bound to the native library."""

    def __init__(self, device: int | str | torch.device = 0):
        N.lib()  # fail loudly when the CUDA library is not built
        if not torch.cuda.is_available():
            raise InvalidOperationException("no CUDA device: this path has no CPU fallback")
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.L = N.lib()

    # -- memory / streams (plumbing) --
    def Allocate1D(self, length: int, dtype: torch.dtype) -> torch.Tensor:
        return torch.empty(int(length), dtype=dtype, device=self.device)

    def Synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def Bind(self):
        """Makes this accelerator's device current (CudaAccelerator.cs:422-424)."""
        return torch.cuda.device(self.device)

    # -- temp sizing: RadixSortExtensions.cs:384-447, ScanExtensions.cs:158-170 --
    def ComputeRadixSortTempStorageSize(self, operation: RadixSortOperation, dataLength: int) -> int:
        out = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(self.L.b200alg_radix_sort_temp_bytes(
            dtype_code(operation.dtype), int(dataLength), 0, ctypes.byref(out)))
        return _ints(out.value)

    def ComputeRadixSortPairsTempStorageSize(self, operation: RadixSortOperation, value_dtype: torch.dtype,
                                             dataLength: int) -> int:
        out = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(self.L.b200alg_radix_sort_temp_bytes(
            dtype_code(operation.dtype), int(dataLength), value_dtype.itemsize, ctypes.byref(out)))
        return _ints(out.value)

    def ComputeScanTempStorageSize(self, dtype: torch.dtype, dataLength: int) -> int:
        out = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(self.L.b200alg_scan_temp_bytes(dtype_code(dtype), int(dataLength), ctypes.byref(out)))
        return _ints(out.value)

    # -- radix sort --
    def CreateRadixSort(self, operation: RadixSortOperation, float_total_order: bool = False):
        """Returns ``sort(stream, view, temp)`` (RadixSort<T, TStride> delegate,
        RadixSortExtensions.cs:37-52)."""
        code = dtype_code(operation.dtype)
        order = (N.SORT_DESCENDING if operation.descending else 0) | (N.SORT_FLOAT_TOTAL_ORDER if float_total_order else 0)

        def sort(stream, view, temp):
            _check_view(view, "view", operation.dtype)
            n = view.numel()
            if n > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            _check_temp(temp, self.ComputeRadixSortTempStorageSize(operation, n))
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_radix_sort_keys(
                    _stream_ptr(stream), _ptr(view), n, _stride(view), code, order, _ptr(temp), temp.numel() * 4))

        return sort

    def CreateRadixSortPairs(self, operation: RadixSortOperation, float_total_order: bool = False,
                             sequencer: type | None = None):
        """Returns ``sort(stream, keys, values, temp)`` (RadixSortPairs delegate,
        RadixSortExtensions.cs:54-108); keys and values are reordered together, stably.
        With ``sequencer=Sequencers`` the sequencer overload (:1017-1074) is returned instead:
        ``sort(stream, keys, values, sequencer, temp)``, where the values entering the sort
        are ``sequencer.ComputeSequenceElement(i)`` and ``values`` only receives the result."""
        code = dtype_code(operation.dtype)
        order = (N.SORT_DESCENDING if operation.descending else 0) | (N.SORT_FLOAT_TOTAL_ORDER if float_total_order else 0)

        def sort_sequenced(stream, keys, values, seq, temp):
            if not isinstance(seq, Sequencer):
                raise NotSupportedException("only the built-in sequencers cross the native boundary")
            _check_view(keys, "keys", operation.dtype)
            _check_view(values, "values", seq.dtype)
            n = keys.numel()
            if n > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            if values.numel() != n:
                raise ArgumentOutOfRangeException("values")
            if _stride(keys) != 1 or _stride(values) != 1:
                raise NotSupportedException("pairs are sorted from dense views")
            _check_temp(temp, self.ComputeRadixSortPairsTempStorageSize(operation, values.dtype, n))
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_radix_sort_pairs_sequence(
                    _stream_ptr(stream), _ptr(keys), _ptr(values), n, code, dtype_code(seq.dtype), order,
                    _ptr(temp), temp.numel() * 4))

        if sequencer is not None:
            return sort_sequenced

        def sort(stream, keys, values, temp):
            _check_view(keys, "keys", operation.dtype)
            _check_view(values, "values")
            n = keys.numel()
            if n > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            if values.numel() < n:
                raise ArgumentOutOfRangeException("values")
            if _stride(keys) != 1 or _stride(values) != 1:
                raise NotSupportedException("pairs are sorted from dense views")
            _check_temp(temp, self.ComputeRadixSortPairsTempStorageSize(operation, values.dtype, n))
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_radix_sort_pairs(
                    _stream_ptr(stream), _ptr(keys), _ptr(values), n, code, values.dtype.itemsize, order,
                    _ptr(temp), temp.numel() * 4))

        return sort

    def CreateRadixSortProvider(self, operation: RadixSortOperation, dataLength: int,
                                value_dtype: torch.dtype | None = None) -> RadixSortProvider:
        """RadixSortExtensions.cs:1378-1437."""
        if value_dtype is None:
            ints = self.ComputeRadixSortTempStorageSize(operation, dataLength)
        else:
            ints = self.ComputeRadixSortPairsTempStorageSize(operation, value_dtype, dataLength)
        return RadixSortProvider(self, ints)

    # -- scan --
    def CreateScan(self, operation: ScanReduceOperation, kind: ScanKind):
        """Returns ``scan(stream, input, output, temp)`` (Scan<T, TStrideIn, TStrideOut>
        delegate, ScanExtensions.cs:52-63)."""
        code = dtype_code(operation.dtype)
        inclusive = 1 if kind == ScanKind.Inclusive else 0

        def scan(stream, input, output, temp, carry_in=None):
            # order and kinds of the checks: ScanExtensions.cs:675-689
            _check_view(input, "input", operation.dtype)
            _check_view(output, "output", operation.dtype)
            n = input.numel()
            if output.numel() < n:
                raise ArgumentOutOfRangeException("output")
            if n > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            _check_temp(temp, self.ComputeScanTempStorageSize(operation.dtype, n))
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_scan_carry(
                    _stream_ptr(stream), _ptr(input), _stride(input), _ptr(output), _stride(output), n, code,
                    operation.op, inclusive, _ptr(carry_in), _ptr(temp), temp.numel() * 4))

        return scan

    def CreateScanProvider(self, dtype: torch.dtype, dataLength: int) -> ScanProvider:
        """ScanExtensions.cs:968-991."""
        return ScanProvider(self, self.ComputeScanTempStorageSize(dtype, dataLength))

    # -- reduce --
    def CreateReduction(self, operation: ScanReduceOperation):
        """Returns ``reduce(stream, input, output)`` (Reduction<T, TStride> delegate,
        ReductionExtensions.cs:30-35)."""
        code = dtype_code(operation.dtype)

        def reduce(stream, input, output):
            # ReductionExtensions.cs:146-153
            if input is None:
                raise ArgumentNullException("input")
            _check_view(input, "input", operation.dtype)
            if input.numel() < 1:
                raise ArgumentOutOfRangeException("input")
            if output is None:
                raise ArgumentNullException("output")
            _check_view(output, "output", operation.dtype)
            if output.numel() < 1:
                raise ArgumentOutOfRangeException("output")
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_reduce(
                    _stream_ptr(stream), _ptr(input), _stride(input), input.numel(), code, operation.op, _ptr(output)))

        return reduce

    def Reduce(self, stream, input: torch.Tensor, operation: ScanReduceOperation, output: torch.Tensor | None = None):
        """With ``output``: asynchronous (ReductionExtensions.cs:180-196).  Without: allocates
        one element, reduces, copies it to the CPU - that synchronises - and returns the
        value (ReductionExtensions.cs:198-216)."""
        reduce = self.CreateReduction(operation)
        if output is not None:
            reduce(stream, input, output)
            return None
        out = self.Allocate1D(1, operation.dtype)
        reduce(stream, input, out)
        return out.cpu()[0].item()

    # -- histogram --
    def CreateHistogram(self, locator, checked: bool = True):
        """Returns ``histogram(stream, view, histogram, histogramOverflow)``
        (HistogramExtensions.cs:293-354); the unchecked variant (:371-427) takes no overflow view."""
        def run(stream, view, histogram, histogramOverflow=None):
            # HistogramExtensions.cs:322-338
            _check_view(view, "view")
            _check_view(histogram, "histogram")
            if checked:
                _check_view(histogramOverflow, "histogramOverflow", torch.int32)
                if histogramOverflow.numel() < 1:
                    raise ArgumentOutOfRangeException("histogramOverflow")
            if view.numel() > 2**31 - 1 or histogram.numel() > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            if histogram.numel() < 1:
                raise ArgumentOutOfRangeException("histogram")
            if _stride(histogram) != 1:
                raise NotSupportedException("histogram bins are a dense view")
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_histogram(
                    _stream_ptr(stream), _ptr(view), _stride(view), view.numel(), dtype_code(view.dtype), locator.code,
                    float(locator.lo), float(locator.hi), _ptr(histogram), histogram.numel(),
                    dtype_code(histogram.dtype), _ptr(histogramOverflow) if checked else None))

        return run

    def Histogram(self, stream, view, histogram, histogramOverflow, locator) -> None:
        """HistogramLaunchers.tt:52-69."""
        self.CreateHistogram(locator, checked=True)(stream, view, histogram, histogramOverflow)

    def HistogramUnchecked(self, stream, view, histogram, locator) -> None:
        """HistogramLaunchers.tt:71-87."""
        self.CreateHistogram(locator, checked=False)(stream, view, histogram)

    # -- unique (the step after a sort) --
    def ComputeUniqueTempStorageSize(self, dtype: torch.dtype, dataLength: int) -> int:
        """UniqueExtensions.cs:114-121; here the temp holds the survivors, so it grows with n."""
        out = ctypes.c_int64(0)
        B200AlgException.ThrowIfFailed(self.L.b200alg_unique_temp_bytes(dtype_code(dtype), int(dataLength), ctypes.byref(out)))
        return _ints(out.value)

    def CreateUnique(self, dtype: torch.dtype):
        """Returns ``unique(stream, input, output, temp)`` (Unique<T> delegate, UniqueExtensions.cs:25-30):
        removes consecutive duplicates in place; ``output[0]`` (int64) receives the new length."""
        code = dtype_code(dtype)

        def unique(stream, input, output, temp):
            # UniqueExtensions.cs:150-172
            _check_view(input, "input", dtype)
            _check_view(output, "output", torch.int64)
            if temp is None:
                raise ArgumentNullException("temp")
            if output.numel() < 1:
                raise ArgumentOutOfRangeException("output")
            if _stride(input) != 1:
                raise NotSupportedException("dense view expected")
            _check_temp(temp, self.ComputeUniqueTempStorageSize(dtype, input.numel()))
            if input.numel() > 2**31 - 1:
                raise NotSupportedException("NotSupportedArrayView64")
            with self.Bind():
                B200AlgException.ThrowIfFailed(self.L.b200alg_unique(
                    _stream_ptr(stream), _ptr(input), input.numel(), code, _ptr(output), _ptr(temp), temp.numel() * 4))

        return unique

    def Unique(self, stream, input: torch.Tensor) -> int:
        """Allocates output and temp, runs, copies the count back - which synchronises
        (UniqueExtensions.cs:200-220)."""
        output = self.Allocate1D(1, torch.int64)
        temp = self.Allocate1D(self.ComputeUniqueTempStorageSize(input.dtype, input.numel()), torch.int32)
        self.CreateUnique(input.dtype)(stream, input, output, temp)
        return int(output.cpu()[0])

    # -- edges of the path --
    def Initialize(self, stream, view: torch.Tensor, value) -> None:
        """InitializeExtensions.cs: fills the view with one value."""
        _check_view(view, "view")
        host = torch.tensor([value], dtype=view.dtype)
        with self.Bind():
            B200AlgException.ThrowIfFailed(self.L.b200alg_initialize(
                _stream_ptr(stream), _ptr(view), _stride(view), view.numel(), view.dtype.itemsize,
                ctypes.c_void_p(host.data_ptr())))

    def Sequence(self, stream, view: torch.Tensor, start: int = 0, step: int = 1) -> None:
        """SequenceExtensions.cs with an integer sequencer: view[i] = start + i * step."""
        _check_view(view, "view")
        if _stride(view) != 1:
            raise NotSupportedException("dense view expected")
        with self.Bind():
            B200AlgException.ThrowIfFailed(self.L.b200alg_sequence(
                _stream_ptr(stream), _ptr(view), view.numel(), dtype_code(view.dtype), int(start), int(step)))

    def CheckDeviceStatus(self, stream, temp: torch.Tensor) -> None:
        """Synchronises and raises if a bounded device-side wait ran out during a call that
        used ``temp``."""
        with self.Bind():
            B200AlgException.ThrowIfFailed(self.L.b200alg_device_status(_stream_ptr(stream), _ptr(temp)))
