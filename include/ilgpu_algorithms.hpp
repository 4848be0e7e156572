// C++ host-side mirror of the ILGPU.Algorithms surface for radix sort, scan, reduce and
// histogram, bound to the C ABI of b200alg.h.  Header only; link with libb200alg and the CUDA
// runtime.
//
// The reference is C#; this mirror keeps its names, argument meaning, argument checks and
// exception kinds so that calling code reads like code written against ILGPU.Algorithms
// (paths inside the ILGPU source tree, Src/ILGPU.Algorithms):
//   delegates RadixSort / RadixSortPairs / Scan / Reduction / Histogram
//       RadixSortExtensions.cs:37-160, ScanExtensions.cs:52-76, ReductionExtensions.cs:30-35,
//       HistogramExtensions.cs:35-59
//   CreateRadixSort / CreateRadixSortPairs / CreateRadixSortProvider, temp-size helpers
//       RadixSortExtensions.cs:384-447, :1017-1437
//   CreateScan / CreateScanProvider / ComputeScanTempStorageSize, ScanKind
//       ScanExtensions.cs:27-38, :158-170, :930-991
//   CreateReduction / Reduce            ReductionExtensions.cs:135-309
//   Histogram / HistogramUnchecked      HistogramLaunchers.tt:52-101
//   operation structs                   ScanReduceOperations.tt, RadixSortOperations.tt
//   ArrayView / ArrayView1D / Stride1D  Src/ILGPU/ArrayView.cs, Runtime/ArrayViews.tt, Stride.cs
// There is no fallback path: every call ends in the CUDA library.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <limits>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "b200alg.h"

namespace ILGPU {

// ---- exceptions (names of the .NET types the reference throws) ----------------------------
struct ArgumentNullException : std::invalid_argument { using std::invalid_argument::invalid_argument; };
struct ArgumentOutOfRangeException : std::out_of_range { using std::out_of_range::out_of_range; };
struct NotSupportedException : std::runtime_error { using std::runtime_error::runtime_error; };
struct InvalidOperationException : std::logic_error { using std::logic_error::logic_error; };

// Status of the native library -> exception (pattern: CuRandException.ThrowIfFailed,
// Runtime/Cuda/CuRandException.cs:98-103).
struct B200AlgException : std::runtime_error {
    int Status;
    explicit B200AlgException(int status)
        : std::runtime_error(std::string("b200alg: ") + b200alg_status_string(status) +
                             (status == B200ALG_CUDA_ERROR ? " [cudaError " + std::to_string(b200alg_last_cuda_error()) + "]" : "")),
          Status(status) {}
    static void ThrowIfFailed(int status) {
        switch (status) {
        case B200ALG_OK: return;
        case B200ALG_TOO_LARGE: throw NotSupportedException("NotSupportedArrayView64");
        case B200ALG_TEMP_TOO_SMALL: throw ArgumentOutOfRangeException("temp");
        case B200ALG_UNSUPPORTED: throw NotSupportedException(b200alg_status_string(status));
        default: throw B200AlgException(status);
        }
    }
};

// ---- element types ---------------------------------------------------------------------------
template <typename T> struct DTypeOf;
template <> struct DTypeOf<int8_t> { static constexpr int value = B200ALG_I8; };
template <> struct DTypeOf<uint8_t> { static constexpr int value = B200ALG_U8; };
template <> struct DTypeOf<int16_t> { static constexpr int value = B200ALG_I16; };
template <> struct DTypeOf<uint16_t> { static constexpr int value = B200ALG_U16; };
template <> struct DTypeOf<int32_t> { static constexpr int value = B200ALG_I32; };
template <> struct DTypeOf<uint32_t> { static constexpr int value = B200ALG_U32; };
template <> struct DTypeOf<int64_t> { static constexpr int value = B200ALG_I64; };
template <> struct DTypeOf<uint64_t> { static constexpr int value = B200ALG_U64; };
template <> struct DTypeOf<float> { static constexpr int value = B200ALG_F32; };
template <> struct DTypeOf<double> { static constexpr int value = B200ALG_F64; };

// ---- views -----------------------------------------------------------------------------------
namespace Stride1D {
struct Dense { static constexpr int64_t StrideExtent = 1; };
struct General { int64_t StrideExtent = 1; };
}  // namespace Stride1D

// ArrayView<T>: a dense span of device memory (Src/ILGPU/ArrayView.cs).
template <typename T> struct ArrayView {
    T *Pointer = nullptr;
    int64_t Length = 0;
    ArrayView() = default;
    ArrayView(T *pointer, int64_t length) : Pointer(pointer), Length(length) {}
    bool IsValid() const { return Pointer != nullptr; }
    int64_t LengthInBytes() const { return Length * (int64_t)sizeof(T); }
    ArrayView SubView(int64_t index, int64_t length) const {
        if (index < 0 || length < 0 || index + length > Length) throw ArgumentOutOfRangeException("index");
        return ArrayView(Pointer + index, length);
    }
    T *LoadEffectiveAddressAsPtr() const { return Pointer; }
};

// ArrayView1D<T, TStride>: `Length` elements, StrideExtent elements apart.
template <typename T, typename TStride = Stride1D::Dense> struct ArrayView1D {
    ArrayView<T> BaseView;
    TStride Stride;
    int64_t Length = 0;
    ArrayView1D() = default;
    ArrayView1D(ArrayView<T> base, int64_t length, TStride stride = TStride()) : BaseView(base), Stride(stride), Length(length) {}
    // dense views convert from ArrayView<T>
    template <typename S = TStride, typename = typename std::enable_if<std::is_same<S, Stride1D::Dense>::value>::type>
    ArrayView1D(ArrayView<T> base) : BaseView(base), Length(base.Length) {}
    bool IsValid() const { return BaseView.IsValid(); }
    int64_t StrideExtent() const { return Stride.StrideExtent; }
};

template <typename T> ArrayView1D<T, Stride1D::General> AsGeneral(ArrayView<T> base, int64_t stride) {
    const int64_t n = base.Length == 0 ? 0 : (base.Length - 1) / stride + 1;
    return ArrayView1D<T, Stride1D::General>(base, n, Stride1D::General{stride});
}

// ---- runtime plumbing: device, stream, buffers ---------------------------------------------------
class AcceleratorStream {
public:
    AcceleratorStream() : stream_(nullptr), owned_(false) {}  // default stream
    static AcceleratorStream Create() {
        AcceleratorStream s;
        if (cudaStreamCreateWithFlags(&s.stream_, cudaStreamNonBlocking) != cudaSuccess)
            throw InvalidOperationException("cudaStreamCreate failed");
        s.owned_ = true;
        return s;
    }
    AcceleratorStream(AcceleratorStream &&o) noexcept : stream_(o.stream_), owned_(o.owned_) { o.owned_ = false; }
    AcceleratorStream(const AcceleratorStream &) = delete;
    ~AcceleratorStream() { if (owned_) cudaStreamDestroy(stream_); }
    void *StreamPtr() const { return stream_; }  // CudaStream.StreamPtr
    void Synchronize() const { cudaStreamSynchronize(stream_); }
private:
    cudaStream_t stream_;
    bool owned_;
};

template <typename T> class MemoryBuffer1D {
public:
    explicit MemoryBuffer1D(int64_t length) : length_(length) {
        if (cudaMalloc(&ptr_, (size_t)(length < 1 ? 1 : length) * sizeof(T)) != cudaSuccess)
            throw InvalidOperationException("cudaMalloc failed");
    }
    MemoryBuffer1D(const MemoryBuffer1D &) = delete;
    ~MemoryBuffer1D() { cudaFree(ptr_); }
    ArrayView<T> View() const { return ArrayView<T>((T *)ptr_, length_); }
    int64_t Length() const { return length_; }
    void CopyFromCPU(const T *src) { cudaMemcpy(ptr_, src, (size_t)length_ * sizeof(T), cudaMemcpyHostToDevice); }
    void CopyToCPU(T *dst) const { cudaMemcpy(dst, ptr_, (size_t)length_ * sizeof(T), cudaMemcpyDeviceToHost); }
    void MemSetToZero() { cudaMemset(ptr_, 0, (size_t)length_ * sizeof(T)); }
private:
    void *ptr_ = nullptr;
    int64_t length_;
};

class Accelerator {
public:
    explicit Accelerator(int device = 0) : device_(device) {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count)
            throw InvalidOperationException("no such CUDA device: this path has no CPU fallback");
    }
    void Bind() const { cudaSetDevice(device_); }  // CudaAccelerator.cs:422-424
    void Synchronize() const { Bind(); cudaDeviceSynchronize(); }
    template <typename T> std::unique_ptr<MemoryBuffer1D<T>> Allocate1D(int64_t length) const {
        Bind();
        return std::unique_ptr<MemoryBuffer1D<T>>(new MemoryBuffer1D<T>(length));
    }
    int Device() const { return device_; }
private:
    int device_;
};

namespace Algorithms {

// ---- operations ------------------------------------------------------------------------------
enum class ScanKind { Inclusive, Exclusive };  // ScanExtensions.cs:27-38

namespace ScanReduceOperations {
template <typename TT, int OP> struct Operation {
    using T = TT;
    static constexpr int Op = OP;
    static T Identity() {
        return OP == B200ALG_ADD ? T(0) : (OP == B200ALG_MAX ? std::numeric_limits<T>::lowest() : std::numeric_limits<T>::max());
    }
};
#define B200ALG_DECLARE_SR_OPS(Name, Type)                      \
    using Add##Name = Operation<Type, B200ALG_ADD>;              \
    using Max##Name = Operation<Type, B200ALG_MAX>;              \
    using Min##Name = Operation<Type, B200ALG_MIN>;
B200ALG_DECLARE_SR_OPS(Int32, int32_t)
B200ALG_DECLARE_SR_OPS(Int64, int64_t)
B200ALG_DECLARE_SR_OPS(UInt32, uint32_t)
B200ALG_DECLARE_SR_OPS(UInt64, uint64_t)
B200ALG_DECLARE_SR_OPS(Float, float)
B200ALG_DECLARE_SR_OPS(Double, double)
#undef B200ALG_DECLARE_SR_OPS
}  // namespace ScanReduceOperations

namespace RadixSortOperations {
template <typename TT, bool DESCENDING> struct Operation {
    using T = TT;
    static constexpr int Order = DESCENDING ? B200ALG_SORT_DESCENDING : B200ALG_SORT_ASCENDING;
    static constexpr int NumBits = sizeof(TT) * 8;
};
#define B200ALG_DECLARE_SORT_OPS(Name, Type)            \
    using Ascending##Name = Operation<Type, false>;      \
    using Descending##Name = Operation<Type, true>;
B200ALG_DECLARE_SORT_OPS(Int8, int8_t)
B200ALG_DECLARE_SORT_OPS(UInt8, uint8_t)
B200ALG_DECLARE_SORT_OPS(Int16, int16_t)
B200ALG_DECLARE_SORT_OPS(UInt16, uint16_t)
B200ALG_DECLARE_SORT_OPS(Int32, int32_t)
B200ALG_DECLARE_SORT_OPS(UInt32, uint32_t)
B200ALG_DECLARE_SORT_OPS(Int64, int64_t)
B200ALG_DECLARE_SORT_OPS(UInt64, uint64_t)
B200ALG_DECLARE_SORT_OPS(Float, float)
B200ALG_DECLARE_SORT_OPS(Double, double)
#undef B200ALG_DECLARE_SORT_OPS
}  // namespace RadixSortOperations

// Named bin locators (the reference leaves the locator to user structs; see b200alg.h).
struct ModuloBinOperation {
    static constexpr int Locator = B200ALG_LOCATOR_MODULO;
    double Lo = 0.0, Hi = 1.0;
};
struct EqualWidthClampLocator {
    static constexpr int Locator = B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP;
    double Lo, Hi;
    EqualWidthClampLocator(double lo, double hi) : Lo(lo), Hi(hi) {}
};

// ---- delegates -----------------------------------------------------------------------------------
template <typename T, typename TStride = Stride1D::Dense>
using RadixSort = std::function<void(const AcceleratorStream &, ArrayView1D<T, TStride>, ArrayView<int>)>;
template <typename TKey, typename TValue>
using RadixSortPairs = std::function<void(const AcceleratorStream &, ArrayView1D<TKey>, ArrayView1D<TValue>, ArrayView<int>)>;
template <typename T, typename TStrideIn = Stride1D::Dense, typename TStrideOut = Stride1D::Dense>
using Scan = std::function<void(const AcceleratorStream &, ArrayView1D<T, TStrideIn>, ArrayView1D<T, TStrideOut>, ArrayView<int>)>;
template <typename T, typename TStride = Stride1D::Dense>
using Reduction = std::function<void(const AcceleratorStream &, ArrayView1D<T, TStride>, ArrayView<T>)>;

namespace detail {
inline int64_t IntsFor(int64_t bytes) {
    const int64_t ints = (bytes + 3) / 4;
    if (ints > std::numeric_limits<int32_t>::max()) throw NotSupportedException("temporary storage exceeds the Index1D range");
    return ints;
}
inline void CheckTemp(const ArrayView<int> &temp, int64_t required_ints) {
    // TempViewManager (TempViewManager.cs:36-37, :84-112)
    if (!temp.IsValid()) throw ArgumentNullException("temp");
    if (temp.Length < required_ints) throw ArgumentOutOfRangeException("temp");
}
}  // namespace detail

// ---- temp sizing (in 32-bit ints, like the reference) --------------------------------------------
template <typename T, typename TRadixSortOperation>
inline int64_t ComputeRadixSortTempStorageSize(const Accelerator &, int64_t dataLength) {
    int64_t bytes = 0;
    B200AlgException::ThrowIfFailed(b200alg_radix_sort_temp_bytes(DTypeOf<T>::value, dataLength, 0, &bytes));
    return detail::IntsFor(bytes);
}
template <typename TKey, typename TValue, typename TRadixSortOperation>
inline int64_t ComputeRadixSortPairsTempStorageSize(const Accelerator &, int64_t dataLength) {
    int64_t bytes = 0;
    B200AlgException::ThrowIfFailed(b200alg_radix_sort_temp_bytes(DTypeOf<TKey>::value, dataLength, (int)sizeof(TValue), &bytes));
    return detail::IntsFor(bytes);
}
template <typename T> inline int64_t ComputeScanTempStorageSize(const Accelerator &, int64_t dataLength) {
    int64_t bytes = 0;
    B200AlgException::ThrowIfFailed(b200alg_scan_temp_bytes(DTypeOf<T>::value, dataLength, &bytes));
    return detail::IntsFor(bytes);
}

// ---- radix sort ------------------------------------------------------------------------------------
template <typename T, typename TStride, typename TRadixSortOperation>
inline RadixSort<T, TStride> CreateRadixSort(const Accelerator &accelerator) {
    static_assert(std::is_same<T, typename TRadixSortOperation::T>::value, "operation and element type differ");
    return [accelerator](const AcceleratorStream &stream, ArrayView1D<T, TStride> view, ArrayView<int> temp) {
        if (!view.IsValid()) throw ArgumentNullException("view");
        if (view.Length > std::numeric_limits<int32_t>::max()) throw NotSupportedException("NotSupportedArrayView64");
        detail::CheckTemp(temp, ComputeRadixSortTempStorageSize<T, TRadixSortOperation>(accelerator, view.Length));
        accelerator.Bind();
        B200AlgException::ThrowIfFailed(b200alg_radix_sort_keys(stream.StreamPtr(), view.BaseView.Pointer, view.Length,
                                                                view.StrideExtent(), DTypeOf<T>::value,
                                                                TRadixSortOperation::Order, temp.Pointer, temp.LengthInBytes()));
    };
}

template <typename TKey, typename TValue, typename TRadixSortOperation>
inline RadixSortPairs<TKey, TValue> CreateRadixSortPairs(const Accelerator &accelerator) {
    static_assert(std::is_same<TKey, typename TRadixSortOperation::T>::value, "operation and key type differ");
    return [accelerator](const AcceleratorStream &stream, ArrayView1D<TKey> keys, ArrayView1D<TValue> values, ArrayView<int> temp) {
        if (!keys.IsValid()) throw ArgumentNullException("keys");
        if (!values.IsValid()) throw ArgumentNullException("values");
        if (values.Length < keys.Length) throw ArgumentOutOfRangeException("values");
        if (keys.Length > std::numeric_limits<int32_t>::max()) throw NotSupportedException("NotSupportedArrayView64");
        detail::CheckTemp(temp, ComputeRadixSortPairsTempStorageSize<TKey, TValue, TRadixSortOperation>(accelerator, keys.Length));
        accelerator.Bind();
        B200AlgException::ThrowIfFailed(b200alg_radix_sort_pairs(stream.StreamPtr(), keys.BaseView.Pointer, values.BaseView.Pointer,
                                                                 keys.Length, DTypeOf<TKey>::value, (int)sizeof(TValue),
                                                                 TRadixSortOperation::Order, temp.Pointer, temp.LengthInBytes()));
    };
}

// Sequencers (Sequencer.cs:20-72, Sequencers.tt:26-38): element i is the index converted to T.
// Only these built-in, stateless ones cross the native boundary.
template <typename TValue> struct ISequencer { using T = TValue; };
struct IndexSequencer : ISequencer<int32_t> {};
struct Int8Sequencer : ISequencer<int8_t> {};
struct UInt8Sequencer : ISequencer<uint8_t> {};
struct Int16Sequencer : ISequencer<int16_t> {};
struct UInt16Sequencer : ISequencer<uint16_t> {};
struct Int32Sequencer : ISequencer<int32_t> {};
struct UInt32Sequencer : ISequencer<uint32_t> {};
struct Int64Sequencer : ISequencer<int64_t> {};
struct UInt64Sequencer : ISequencer<uint64_t> {};
struct FloatSequencer : ISequencer<float> {};
struct DoubleSequencer : ISequencer<double> {};

// The sequencer overload of CreateRadixSortPairs (RadixSortExtensions.cs:1017-1074): values
// entering the sort are sequencer.ComputeSequenceElement(i); `values` receives the result.
template <typename TKey, typename TValue, typename TSequencer>
using RadixSortPairsSequenced =
    std::function<void(const AcceleratorStream &, ArrayView1D<TKey>, ArrayView1D<TValue>, TSequencer, ArrayView<int>)>;
template <typename TKey, typename TValue, typename TSequencer, typename TRadixSortOperation>
inline RadixSortPairsSequenced<TKey, TValue, TSequencer> CreateRadixSortPairs(const Accelerator &accelerator) {
    static_assert(std::is_same<TKey, typename TRadixSortOperation::T>::value, "operation and key type differ");
    static_assert(std::is_same<TValue, typename TSequencer::T>::value, "sequencer and value type differ");
    return [accelerator](const AcceleratorStream &stream, ArrayView1D<TKey> keys, ArrayView1D<TValue> values, TSequencer,
                         ArrayView<int> temp) {
        if (!keys.IsValid()) throw ArgumentNullException("keys");
        if (!values.IsValid()) throw ArgumentNullException("values");
        if (keys.Length != values.Length) throw ArgumentOutOfRangeException("values");
        if (keys.Length > std::numeric_limits<int32_t>::max()) throw NotSupportedException("NotSupportedArrayView64");
        detail::CheckTemp(temp, ComputeRadixSortPairsTempStorageSize<TKey, TValue, TRadixSortOperation>(accelerator, keys.Length));
        accelerator.Bind();
        B200AlgException::ThrowIfFailed(b200alg_radix_sort_pairs_sequence(
            stream.StreamPtr(), keys.BaseView.Pointer, values.BaseView.Pointer, keys.Length, DTypeOf<TKey>::value,
            DTypeOf<TValue>::value, TRadixSortOperation::Order, temp.Pointer, temp.LengthInBytes()));
    };
}

// RadixSortProvider (RadixSortExtensions.cs:168-300): owns the temp buffer.
class RadixSortProvider {
public:
    RadixSortProvider(const Accelerator &accelerator, int64_t temp_ints)
        : accelerator_(accelerator), temp_(accelerator.Allocate1D<int>(temp_ints < 64 ? 64 : temp_ints)) {}
    template <typename T, typename TStride, typename TRadixSortOperation>
    std::function<void(const AcceleratorStream &, ArrayView1D<T, TStride>)> CreateRadixSort() {
        auto sort = Algorithms::CreateRadixSort<T, TStride, TRadixSortOperation>(accelerator_);
        ArrayView<int> temp = temp_->View();
        return [sort, temp](const AcceleratorStream &stream, ArrayView1D<T, TStride> view) { sort(stream, view, temp); };
    }
    template <typename TKey, typename TValue, typename TRadixSortOperation>
    std::function<void(const AcceleratorStream &, ArrayView1D<TKey>, ArrayView1D<TValue>)> CreateRadixSortPairs() {
        auto sort = Algorithms::CreateRadixSortPairs<TKey, TValue, TRadixSortOperation>(accelerator_);
        ArrayView<int> temp = temp_->View();
        return [sort, temp](const AcceleratorStream &stream, ArrayView1D<TKey> keys, ArrayView1D<TValue> values) {
            sort(stream, keys, values, temp);
        };
    }
private:
    Accelerator accelerator_;
    std::unique_ptr<MemoryBuffer1D<int>> temp_;
};
template <typename T, typename TRadixSortOperation>
inline RadixSortProvider CreateRadixSortProvider(const Accelerator &accelerator, int64_t dataLength) {
    return RadixSortProvider(accelerator, ComputeRadixSortTempStorageSize<T, TRadixSortOperation>(accelerator, dataLength));
}
template <typename TKey, typename TValue, typename TRadixSortOperation>
inline RadixSortProvider CreateRadixSortPairsProvider(const Accelerator &accelerator, int64_t dataLength) {
    return RadixSortProvider(accelerator, ComputeRadixSortPairsTempStorageSize<TKey, TValue, TRadixSortOperation>(accelerator, dataLength));
}

// ---- scan --------------------------------------------------------------------------------------------
template <typename T, typename TStrideIn, typename TStrideOut, typename TScanOperation>
inline Scan<T, TStrideIn, TStrideOut> CreateScan(const Accelerator &accelerator, ScanKind kind) {
    static_assert(std::is_same<T, typename TScanOperation::T>::value, "operation and element type differ");
    return [accelerator, kind](const AcceleratorStream &stream, ArrayView1D<T, TStrideIn> input,
                               ArrayView1D<T, TStrideOut> output, ArrayView<int> temp) {
        // order of the checks: ScanExtensions.cs:675-689
        if (!input.IsValid()) throw ArgumentNullException("input");
        if (!output.IsValid()) throw ArgumentNullException("output");
        if (output.Length < input.Length) throw ArgumentOutOfRangeException("output");
        if (input.Length > std::numeric_limits<int32_t>::max()) throw NotSupportedException("NotSupportedArrayView64");
        detail::CheckTemp(temp, ComputeScanTempStorageSize<T>(accelerator, input.Length));
        accelerator.Bind();
        B200AlgException::ThrowIfFailed(b200alg_scan(stream.StreamPtr(), input.BaseView.Pointer, input.StrideExtent(),
                                                     output.BaseView.Pointer, output.StrideExtent(), input.Length,
                                                     DTypeOf<T>::value, TScanOperation::Op, kind == ScanKind::Inclusive ? 1 : 0,
                                                     temp.Pointer, temp.LengthInBytes()));
    };
}

// ScanProvider (ScanExtensions.cs:84-142).
class ScanProvider {
public:
    ScanProvider(const Accelerator &accelerator, int64_t temp_ints)
        : accelerator_(accelerator), temp_(accelerator.Allocate1D<int>(temp_ints < 64 ? 64 : temp_ints)) {}
    template <typename T, typename TStrideIn, typename TStrideOut, typename TScanOperation>
    std::function<void(const AcceleratorStream &, ArrayView1D<T, TStrideIn>, ArrayView1D<T, TStrideOut>)> CreateScan(ScanKind kind) {
        auto scan = Algorithms::CreateScan<T, TStrideIn, TStrideOut, TScanOperation>(accelerator_, kind);
        ArrayView<int> temp = temp_->View();
        return [scan, temp](const AcceleratorStream &stream, ArrayView1D<T, TStrideIn> input, ArrayView1D<T, TStrideOut> output) {
            scan(stream, input, output, temp);
        };
    }
private:
    Accelerator accelerator_;
    std::unique_ptr<MemoryBuffer1D<int>> temp_;
};
template <typename T> inline ScanProvider CreateScanProvider(const Accelerator &accelerator, int64_t dataLength) {
    return ScanProvider(accelerator, ComputeScanTempStorageSize<T>(accelerator, dataLength));
}

// ---- reduce ------------------------------------------------------------------------------------------
template <typename T, typename TStride, typename TReduction>
inline Reduction<T, TStride> CreateReduction(const Accelerator &accelerator) {
    static_assert(std::is_same<T, typename TReduction::T>::value, "operation and element type differ");
    return [accelerator](const AcceleratorStream &stream, ArrayView1D<T, TStride> input, ArrayView<T> output) {
        // ReductionExtensions.cs:146-153
        if (!input.IsValid()) throw ArgumentNullException("input");
        if (input.Length < 1) throw ArgumentOutOfRangeException("input");
        if (!output.IsValid()) throw ArgumentNullException("output");
        if (output.Length < 1) throw ArgumentOutOfRangeException("output");
        accelerator.Bind();
        B200AlgException::ThrowIfFailed(b200alg_reduce(stream.StreamPtr(), input.BaseView.Pointer, input.StrideExtent(),
                                                       input.Length, DTypeOf<T>::value, TReduction::Op, output.Pointer));
    };
}

// Asynchronous overload with an output view (ReductionExtensions.cs:180-196).
template <typename T, typename TStride, typename TReduction>
inline void Reduce(const Accelerator &accelerator, const AcceleratorStream &stream, ArrayView1D<T, TStride> input, ArrayView<T> output) {
    CreateReduction<T, TStride, TReduction>(accelerator)(stream, input, output);
}
// Value-returning overload: allocates one element, reduces, copies back - which synchronises
// (ReductionExtensions.cs:198-216).
template <typename T, typename TStride, typename TReduction>
inline T Reduce(const Accelerator &accelerator, const AcceleratorStream &stream, ArrayView1D<T, TStride> input) {
    auto cell = accelerator.Allocate1D<T>(1);
    CreateReduction<T, TStride, TReduction>(accelerator)(stream, input, cell->View());
    T result;
    stream.Synchronize();
    cell->CopyToCPU(&result);
    return result;
}

// ---- histogram ---------------------------------------------------------------------------------------
template <typename T, typename TStride, typename TBinType, typename TLocator>
inline void Histogram(const Accelerator &accelerator, const AcceleratorStream &stream, ArrayView1D<T, TStride> view,
                      ArrayView<TBinType> histogram, ArrayView<int> histogramOverflow, const TLocator &locator) {
    // HistogramExtensions.cs:322-338
    if (!view.IsValid()) throw ArgumentNullException("view");
    if (!histogram.IsValid()) throw ArgumentNullException("histogram");
    if (!histogramOverflow.IsValid()) throw ArgumentNullException("histogramOverflow");
    if (view.Length > std::numeric_limits<int32_t>::max() || histogram.Length > std::numeric_limits<int32_t>::max())
        throw NotSupportedException("NotSupportedArrayView64");
    if (histogram.Length < 1) throw ArgumentOutOfRangeException("histogram");
    if (histogramOverflow.Length < 1) throw ArgumentOutOfRangeException("histogramOverflow");
    accelerator.Bind();
    B200AlgException::ThrowIfFailed(b200alg_histogram(stream.StreamPtr(), view.BaseView.Pointer, view.StrideExtent(), view.Length,
                                                      DTypeOf<T>::value, TLocator::Locator, locator.Lo, locator.Hi, histogram.Pointer,
                                                      histogram.Length, DTypeOf<TBinType>::value, histogramOverflow.Pointer));
}

template <typename T, typename TStride, typename TBinType, typename TLocator>
inline void HistogramUnchecked(const Accelerator &accelerator, const AcceleratorStream &stream, ArrayView1D<T, TStride> view,
                               ArrayView<TBinType> histogram, const TLocator &locator) {
    if (!view.IsValid()) throw ArgumentNullException("view");
    if (!histogram.IsValid()) throw ArgumentNullException("histogram");
    if (view.Length > std::numeric_limits<int32_t>::max() || histogram.Length > std::numeric_limits<int32_t>::max())
        throw NotSupportedException("NotSupportedArrayView64");
    if (histogram.Length < 1) throw ArgumentOutOfRangeException("histogram");
    accelerator.Bind();
    B200AlgException::ThrowIfFailed(b200alg_histogram(stream.StreamPtr(), view.BaseView.Pointer, view.StrideExtent(), view.Length,
                                                      DTypeOf<T>::value, TLocator::Locator, locator.Lo, locator.Hi, histogram.Pointer,
                                                      histogram.Length, DTypeOf<TBinType>::value, nullptr));
}

}  // namespace Algorithms
}  // namespace ILGPU
