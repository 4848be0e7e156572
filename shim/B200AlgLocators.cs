// Not compiled in this repository: no .NET SDK on the build machines (see README.md).
// Named bin locators.  The reference leaves the locator to a user struct
// (IComputeSingleBinOperation<T, Index1D>, IHistogramOperations.cs:19-33) that is instantiated
// as default(TLocator) inside the kernel (HistogramLaunchers.tt:95-96), so its logic cannot
// cross a C ABI.  These structs are ordinary locators in C# - they run unchanged on the
// CPUAccelerator and on the JIT path - and in addition tell the native path which of its
// built-in locators they are (include/b200alg.h, b200alg_locator).
using ILGPU.Algorithms.HistogramOperations;
using System;

namespace ILGPU.Runtime.Cuda
{
    /// <summary>Implemented by locators the native histogram knows.</summary>
    public interface IB200AlgLocator
    {
        /// <summary>b200alg_locator.</summary>
        int NativeLocator { get; }
        /// <summary>Lower / upper end of the binned range (ignored by the modulo locator).</summary>
        double Lo { get; }
        double Hi { get; }
    }

    /// <summary>A constant range, supplied as a type argument because locators carry no instance state.</summary>
    public interface IBinRange
    {
        double Lo { get; }
        double Hi { get; }
    }

    /// <summary>
    /// Equal-width bins over [Lo, Hi); values outside go to the edge bins, NaN to bin 0:
    /// t = (x - lo) * (numBins / (hi - lo)) in float, bin = clamp(floor(t), 0, numBins - 1).
    /// </summary>
    public readonly struct EqualWidthClampLocatorFloat<TRange> :
        IComputeSingleBinOperation<float, Index1D>, IB200AlgLocator
        where TRange : struct, IBinRange
    {
        public int NativeLocator => 0;  // B200ALG_LOCATOR_EQUAL_WIDTH_CLAMP
        public double Lo => default(TRange).Lo;
        public double Hi => default(TRange).Hi;

        public Index1D ComputeHistogramBin(float value, Index1D numBins)
        {
            float lo = (float)default(TRange).Lo, hi = (float)default(TRange).Hi;
            float scale = (float)numBins.X / (hi - lo);
            float t = (value - lo) * scale;
            // clamp in floating point, then truncate (t >= 0 here, so truncation is floor);
            // the comparisons are false for NaN, which therefore lands in bin 0
            float top = numBins.X - 1;
            t = t > 0.0f ? t : 0.0f;
            t = t < top ? t : top;
            return (Index1D)(int)t;
        }
    }

    /// <summary>The same locator for double input.</summary>
    public readonly struct EqualWidthClampLocatorDouble<TRange> :
        IComputeSingleBinOperation<double, Index1D>, IB200AlgLocator
        where TRange : struct, IBinRange
    {
        public int NativeLocator => 0;
        public double Lo => default(TRange).Lo;
        public double Hi => default(TRange).Hi;

        public Index1D ComputeHistogramBin(double value, Index1D numBins)
        {
            double lo = default(TRange).Lo, hi = default(TRange).Hi;
            double t = (value - lo) * (numBins.X / (hi - lo));
            double top = numBins.X - 1;
            t = t > 0.0 ? t : 0.0;
            t = t < top ? t : top;
            return (Index1D)(int)t;
        }
    }

    /// <summary>
    /// |x % numBins|: the ModuloBin{T}Operation of the reference's tests
    /// (ILGPU.Algorithms.Tests/HistogramTests.tt:83-94), here for int; the other element types
    /// follow the same two lines.
    /// </summary>
    public readonly struct ModuloLocatorInt32 : IComputeSingleBinOperation<int, Index1D>, IB200AlgLocator
    {
        public int NativeLocator => 1;  // B200ALG_LOCATOR_MODULO
        public double Lo => 0.0;
        public double Hi => 1.0;
        public Index1D ComputeHistogramBin(int value, Index1D numBins) => Math.Abs(value % numBins.X);
    }
}
