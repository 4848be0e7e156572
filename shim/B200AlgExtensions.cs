// Not compiled in this repository: no .NET SDK on the build machines (see README.md).
// The lambdas that CreateRadixSort / CreateRadixSortPairs / CreateScan / CreateReduction /
// CreateHistogram return on a CudaAccelerator, rewritten to call libb200alg.  The hook in the
// reference is the accelerator-type switch each Create* method already has
// (ScanExtensions.cs:942-958, RadixSortExtensions.cs:1157): `AcceleratorType.Cuda =>` these.
// Argument checks are the reference's own, in the reference's order; they throw before the
// native call.
using ILGPU.Algorithms;
using ILGPU.Algorithms.HistogramOperations;
using ILGPU.Algorithms.RadixSortOperations;
using ILGPU.Algorithms.ScanReduceOperations;
using ILGPU.Algorithms.Sequencers;
using System;

namespace ILGPU.Runtime.Cuda
{
    public static class B200AlgExtensions
    {
        private static IntPtr StreamPtr(AcceleratorStream stream) =>
            stream is CudaStream cudaStream
                ? cudaStream.StreamPtr                       // Src/ILGPU/Runtime/Cuda/CudaStream.cs:70
                : throw new NotSupportedException("A CUDA stream is required");

        private static IntPtr Ptr<T>(ArrayView<T> view) where T : unmanaged =>
            view.LoadEffectiveAddressAsPtr();                // Src/ILGPU/Runtime/ArrayViewExtensions.cs:48-50

        private static Index1D IntsFor(long bytes)
        {
            long ints = (bytes + 3) / 4;
            return ints <= int.MaxValue
                ? (Index1D)(int)ints
                : throw new NotSupportedException("Temporary storage exceeds int.MaxValue ints");
        }

        #region Temp-storage sizes (RadixSortExtensions.cs:384-447, ScanExtensions.cs:158-170)

        public static Index1D ComputeRadixSortTempStorageSizeNative<T, TRadixSortOperation>(
            this CudaAccelerator accelerator, Index1D dataLength)
            where T : unmanaged
            where TRadixSortOperation : struct, IRadixSortOperation<T>
        {
            B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_radix_sort_temp_bytes(
                (int)B200AlgTypes.DTypeOf<T>(), dataLength, 0, out long bytes));
            return IntsFor(bytes);
        }

        public static Index1D ComputeRadixSortPairsTempStorageSizeNative<TKey, TValue, TRadixSortOperation>(
            this CudaAccelerator accelerator, Index1D dataLength)
            where TKey : unmanaged
            where TValue : unmanaged
            where TRadixSortOperation : struct, IRadixSortOperation<TKey>
        {
            B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_radix_sort_temp_bytes(
                (int)B200AlgTypes.DTypeOf<TKey>(), dataLength, Interop.SizeOf<TValue>(), out long bytes));
            return IntsFor(bytes);
        }

        public static LongIndex1D ComputeScanTempStorageSizeNative<T>(
            this CudaAccelerator accelerator, LongIndex1D dataLength)
            where T : unmanaged
        {
            B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_scan_temp_bytes(
                (int)B200AlgTypes.DTypeOf<T>(), dataLength, out long bytes));
            return (bytes + 3) / 4;
        }

        #endregion

        #region Radix sort (RadixSortExtensions.cs:1130-1337, 1017-1118)

        public static RadixSort<T, TStride> CreateRadixSortNative<T, TStride, TRadixSortOperation>(
            this CudaAccelerator accelerator)
            where T : unmanaged
            where TStride : struct, IStride1D
            where TRadixSortOperation : struct, IRadixSortOperation<T>
        {
            var (dtype, order) = B200AlgTypes.SortOperationOf<TRadixSortOperation>();
            return (stream, view, temp) =>
            {
                if (!view.IsValid)
                    throw new ArgumentNullException(nameof(view));
                if (!temp.IsValid)
                    throw new ArgumentNullException(nameof(temp));
                if (view.Length > int.MaxValue)
                    throw new NotSupportedException("NotSupportedArrayView64");
                accelerator.Bind();                          // CudaAccelerator.cs:422-424, as CuBlas does
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_radix_sort_keys(
                    StreamPtr(stream), Ptr(view.BaseView), view.Length, view.Stride.StrideExtent,
                    (int)dtype, order, Ptr(temp), temp.Length * sizeof(int)));
            };
        }

        public static RadixSortPairs<TKey, TKeyStride, TValue, TValueStride>
            CreateRadixSortPairsNative<TKey, TKeyStride, TValue, TValueStride, TRadixSortOperation>(
            this CudaAccelerator accelerator)
            where TKey : unmanaged
            where TKeyStride : struct, IStride1D
            where TValue : unmanaged
            where TValueStride : struct, IStride1D
            where TRadixSortOperation : struct, IRadixSortOperation<TKey>
        {
            var (dtype, order) = B200AlgTypes.SortOperationOf<TRadixSortOperation>();
            return (stream, keys, values, temp) =>
            {
                if (!keys.IsValid)
                    throw new ArgumentNullException(nameof(keys));
                if (!values.IsValid)
                    throw new ArgumentNullException(nameof(values));
                if (keys.Length != values.Length)
                    throw new ArgumentOutOfRangeException(nameof(values));
                if (keys.Stride.StrideExtent != 1 || values.Stride.StrideExtent != 1)
                    throw new NotSupportedException("Pairs are sorted from dense views");
                accelerator.Bind();
                // structure of arrays: no RadixSortPair<TKey, TValue> gather / scatter (:605-645)
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_radix_sort_pairs(
                    StreamPtr(stream), Ptr(keys.BaseView), Ptr(values.BaseView), keys.Length,
                    (int)dtype, Interop.SizeOf<TValue>(), order, Ptr(temp), temp.Length * sizeof(int)));
            };
        }

        /// <summary>
        /// The sequencer overload (:1017-1074).  Only the stateless built-in sequencers
        /// (IndexSequencer, {Int8..UInt64}Sequencer, HalfSequencer, FloatSequencer,
        /// DoubleSequencer) are produced natively; a ViewSourceSequencer is the view overload.
        /// </summary>
        public static RadixSortPairs<TKey, TKeyStride, TValue, TValueStride, TSequencer>
            CreateRadixSortPairsNative<TKey, TKeyStride, TValue, TValueStride, TSequencer, TRadixSortOperation>(
            this CudaAccelerator accelerator)
            where TKey : unmanaged
            where TKeyStride : struct, IStride1D
            where TValue : unmanaged
            where TValueStride : struct, IStride1D
            where TSequencer : struct, ISequencer<TValue>
            where TRadixSortOperation : struct, IRadixSortOperation<TKey>
        {
            var (dtype, order) = B200AlgTypes.SortOperationOf<TRadixSortOperation>();
            var sequencerType = typeof(TSequencer);
            bool builtIn = sequencerType == typeof(IndexSequencer) || sequencerType == typeof(HalfSequencer) ||
                sequencerType == typeof(FloatSequencer) || sequencerType == typeof(DoubleSequencer) ||
                (sequencerType.Namespace == typeof(IndexSequencer).Namespace &&
                 sequencerType.Name.EndsWith("Sequencer", StringComparison.Ordinal) && !sequencerType.IsGenericType);
            if (!builtIn)
                throw new NotSupportedException($"Sequencer {sequencerType} has no native implementation");
            return (stream, keys, values, sequencer, temp) =>
            {
                if (!keys.IsValid)
                    throw new ArgumentNullException(nameof(keys));
                if (!values.IsValid)
                    throw new ArgumentNullException(nameof(values));
                if (keys.Length != values.Length)
                    throw new ArgumentOutOfRangeException(nameof(values));
                accelerator.Bind();
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_radix_sort_pairs_sequence(
                    StreamPtr(stream), Ptr(keys.BaseView), Ptr(values.BaseView), keys.Length,
                    (int)dtype, (int)B200AlgTypes.DTypeOf<TValue>(), order, Ptr(temp), temp.Length * sizeof(int)));
            };
        }

        #endregion

        #region Scan (ScanExtensions.cs:930-959) and reduce (ReductionExtensions.cs:135-167)

        public static Scan<T, TStrideIn, TStrideOut> CreateScanNative<T, TStrideIn, TStrideOut, TScanOperation>(
            this CudaAccelerator accelerator, ScanKind kind)
            where T : unmanaged
            where TStrideIn : struct, IStride1D
            where TStrideOut : struct, IStride1D
            where TScanOperation : struct, IScanReduceOperation<T>
        {
            var (dtype, op) = B200AlgTypes.ScanReduceOperationOf<TScanOperation>();
            return (stream, input, output, temp) =>
            {
                if (!input.IsValid)
                    throw new ArgumentNullException(nameof(input));
                if (!output.IsValid)
                    throw new ArgumentNullException(nameof(output));
                if (output.Length < input.Length)
                    throw new ArgumentOutOfRangeException(nameof(output));
                if (input.Length > int.MaxValue)
                    throw new NotSupportedException("NotSupportedArrayView64");
                accelerator.Bind();
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_scan(
                    StreamPtr(stream), Ptr(input.BaseView), input.Stride.StrideExtent,
                    Ptr(output.BaseView), output.Stride.StrideExtent, input.Length,
                    (int)dtype, (int)op, kind == ScanKind.Inclusive ? 1 : 0, Ptr(temp), temp.Length * sizeof(int)));
            };
        }

        public static Reduction<T, TStride> CreateReductionNative<T, TStride, TReduction>(
            this CudaAccelerator accelerator)
            where T : unmanaged
            where TStride : struct, IStride1D
            where TReduction : struct, IScanReduceOperation<T>
        {
            var (dtype, op) = B200AlgTypes.ScanReduceOperationOf<TReduction>();
            return (stream, input, output) =>
            {
                if (!input.IsValid)
                    throw new ArgumentNullException(nameof(input));
                if (input.Length < 1)
                    throw new ArgumentOutOfRangeException(nameof(input));
                if (!output.IsValid)
                    throw new ArgumentNullException(nameof(output));
                if (output.Length < 1)
                    throw new ArgumentOutOfRangeException(nameof(output));
                accelerator.Bind();
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_reduce(
                    StreamPtr(stream), Ptr(input.BaseView), input.Stride.StrideExtent, input.Length,
                    (int)dtype, (int)op, Ptr(output)));
            };
        }

        #endregion

        #region Histogram (HistogramExtensions.cs:293-427, HistogramLaunchers.tt:52-101)

        public static Histogram<T, TStride, TBinType> CreateHistogramNative<T, TStride, TBinType, TLocator>(
            this CudaAccelerator accelerator, bool checkedVariant)
            where T : unmanaged
            where TStride : struct, IStride1D
            where TBinType : unmanaged
            where TLocator : struct, IComputeSingleBinOperation<T, Index1D>
        {
            if (default(TLocator) is not IB200AlgLocator locator)
                throw new NotSupportedException(
                    $"Bin locator {typeof(TLocator)} has no native implementation (see IB200AlgLocator)");
            int inDtype = (int)B200AlgTypes.DTypeOf<T>(), binDtype = (int)B200AlgTypes.DTypeOf<TBinType>();
            return (stream, view, histogram, histogramOverflow) =>
            {
                if (!view.IsValid)
                    throw new ArgumentNullException(nameof(view));
                if (!histogram.IsValid)
                    throw new ArgumentNullException(nameof(histogram));
                if (checkedVariant && !histogramOverflow.IsValid)
                    throw new ArgumentNullException(nameof(histogramOverflow));
                if (view.Length > int.MaxValue || histogram.Length > int.MaxValue)
                    throw new NotSupportedException("NotSupportedArrayView64");
                accelerator.Bind();
                B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_histogram(
                    StreamPtr(stream), Ptr(view.BaseView), view.Stride.StrideExtent, view.Length, inDtype,
                    locator.NativeLocator, locator.Lo, locator.Hi, Ptr(histogram), histogram.Length, binDtype,
                    checkedVariant ? Ptr(histogramOverflow) : IntPtr.Zero));
            };
        }

        #endregion

        /// <summary>
        /// Synchronises the stream and throws B200AlgException(WaitLimit) if a bounded device-side
        /// wait ran out during a call that used this temp view.
        /// </summary>
        public static void CheckNativeStatus(this CudaAccelerator accelerator, AcceleratorStream stream, ArrayView<int> temp)
        {
            accelerator.Bind();
            B200AlgException.ThrowIfFailed(B200AlgAPI.b200alg_device_status(StreamPtr(stream), Ptr(temp)));
        }
    }
}
