// Not compiled in this repository: no .NET SDK on the build machines (see README.md).
// Generic arguments of the ILGPU.Algorithms API -> the closed sets of codes that cross the
// native boundary (include/b200alg.h: b200alg_dtype, b200alg_op, B200ALG_SORT_*).
using ILGPU.Algorithms.RadixSortOperations;
using ILGPU.Algorithms.ScanReduceOperations;
using System;
using System.Collections.Generic;

namespace ILGPU.Runtime.Cuda
{
    /// <summary>b200alg_dtype.</summary>
    internal enum B200AlgDType : int
    {
        I8 = 0, U8 = 1, I16 = 2, U16 = 3, I32 = 4, U32 = 5, I64 = 6, U64 = 7, F16 = 8, F32 = 9, F64 = 10,
    }

    /// <summary>b200alg_op.</summary>
    internal enum B200AlgOp : int { Add = 0, Max = 1, Min = 2 }

    /// <summary>
    /// Put on a user struct that only forwards to one of the built-in operations (the test
    /// suite's Xunit{Op}{T} wrappers, Generic/AlgorithmsTestData.tt:142-160, are the model):
    /// it names the built-in whose native implementation may stand in for the wrapper.
    /// Operations without this attribute that are not built-ins raise NotSupportedException:
    /// arbitrary C# logic cannot cross a C ABI and there is no fallback on this path.
    /// </summary>
    [AttributeUsage(AttributeTargets.Struct)]
    public sealed class B200AlgEquivalentAttribute : Attribute
    {
        public B200AlgEquivalentAttribute(Type builtInOperation) { BuiltInOperation = builtInOperation; }
        public Type BuiltInOperation { get; }
    }

    internal static class B200AlgTypes
    {
        private static readonly Dictionary<Type, B200AlgDType> DTypes = new()
        {
            { typeof(sbyte), B200AlgDType.I8 }, { typeof(byte), B200AlgDType.U8 },
            { typeof(short), B200AlgDType.I16 }, { typeof(ushort), B200AlgDType.U16 },
            { typeof(int), B200AlgDType.I32 }, { typeof(uint), B200AlgDType.U32 },
            { typeof(long), B200AlgDType.I64 }, { typeof(ulong), B200AlgDType.U64 },
            { typeof(Half), B200AlgDType.F16 }, { typeof(float), B200AlgDType.F32 },
            { typeof(double), B200AlgDType.F64 },
            { typeof(Index1D), B200AlgDType.I32 }, { typeof(LongIndex1D), B200AlgDType.I64 },
        };

        // The 22 structs of RadixSortOperations.tt:26-125: (key type, descending)
        private static readonly Dictionary<Type, (B200AlgDType, bool)> SortOperations = new()
        {
            { typeof(AscendingInt8), (B200AlgDType.I8, false) }, { typeof(DescendingInt8), (B200AlgDType.I8, true) },
            { typeof(AscendingUInt8), (B200AlgDType.U8, false) }, { typeof(DescendingUInt8), (B200AlgDType.U8, true) },
            { typeof(AscendingInt16), (B200AlgDType.I16, false) }, { typeof(DescendingInt16), (B200AlgDType.I16, true) },
            { typeof(AscendingUInt16), (B200AlgDType.U16, false) }, { typeof(DescendingUInt16), (B200AlgDType.U16, true) },
            { typeof(AscendingInt32), (B200AlgDType.I32, false) }, { typeof(DescendingInt32), (B200AlgDType.I32, true) },
            { typeof(AscendingUInt32), (B200AlgDType.U32, false) }, { typeof(DescendingUInt32), (B200AlgDType.U32, true) },
            { typeof(AscendingInt64), (B200AlgDType.I64, false) }, { typeof(DescendingInt64), (B200AlgDType.I64, true) },
            { typeof(AscendingUInt64), (B200AlgDType.U64, false) }, { typeof(DescendingUInt64), (B200AlgDType.U64, true) },
            { typeof(AscendingHalf), (B200AlgDType.F16, false) }, { typeof(DescendingHalf), (B200AlgDType.F16, true) },
            { typeof(AscendingFloat), (B200AlgDType.F32, false) }, { typeof(DescendingFloat), (B200AlgDType.F32, true) },
            { typeof(AscendingDouble), (B200AlgDType.F64, false) }, { typeof(DescendingDouble), (B200AlgDType.F64, true) },
        };

        // The 18 structs of ScanReduceOperations.tt:20-74: (element type, operation)
        private static readonly Dictionary<Type, (B200AlgDType, B200AlgOp)> ScanReduceOperations = new()
        {
            { typeof(AddInt32), (B200AlgDType.I32, B200AlgOp.Add) }, { typeof(MaxInt32), (B200AlgDType.I32, B200AlgOp.Max) }, { typeof(MinInt32), (B200AlgDType.I32, B200AlgOp.Min) },
            { typeof(AddInt64), (B200AlgDType.I64, B200AlgOp.Add) }, { typeof(MaxInt64), (B200AlgDType.I64, B200AlgOp.Max) }, { typeof(MinInt64), (B200AlgDType.I64, B200AlgOp.Min) },
            { typeof(AddUInt32), (B200AlgDType.U32, B200AlgOp.Add) }, { typeof(MaxUInt32), (B200AlgDType.U32, B200AlgOp.Max) }, { typeof(MinUInt32), (B200AlgDType.U32, B200AlgOp.Min) },
            { typeof(AddUInt64), (B200AlgDType.U64, B200AlgOp.Add) }, { typeof(MaxUInt64), (B200AlgDType.U64, B200AlgOp.Max) }, { typeof(MinUInt64), (B200AlgDType.U64, B200AlgOp.Min) },
            { typeof(AddFloat), (B200AlgDType.F32, B200AlgOp.Add) }, { typeof(MaxFloat), (B200AlgDType.F32, B200AlgOp.Max) }, { typeof(MinFloat), (B200AlgDType.F32, B200AlgOp.Min) },
            { typeof(AddDouble), (B200AlgDType.F64, B200AlgOp.Add) }, { typeof(MaxDouble), (B200AlgDType.F64, B200AlgOp.Max) }, { typeof(MinDouble), (B200AlgDType.F64, B200AlgOp.Min) },
        };

        private static Type Resolve(Type operation)
        {
            var attribute = (B200AlgEquivalentAttribute?)Attribute.GetCustomAttribute(
                operation, typeof(B200AlgEquivalentAttribute));
            return attribute?.BuiltInOperation ?? operation;
        }

        internal static B200AlgDType DTypeOf<T>() where T : unmanaged =>
            DTypes.TryGetValue(typeof(T), out var dtype)
                ? dtype
                : throw new NotSupportedException($"Element type {typeof(T)} is not supported by the native path");

        /// <summary>(key dtype, B200ALG_SORT_* flags) of a radix-sort operation type.</summary>
        internal static (B200AlgDType DType, int Order) SortOperationOf<TOperation>()
            where TOperation : struct =>
            SortOperations.TryGetValue(Resolve(typeof(TOperation)), out var entry)
                ? (entry.Item1, entry.Item2 ? 1 : 0)
                : throw new NotSupportedException(
                    $"Radix-sort operation {typeof(TOperation)} has no native implementation");

        /// <summary>(dtype, op) of a scan / reduce operation type.</summary>
        internal static (B200AlgDType DType, B200AlgOp Op) ScanReduceOperationOf<TOperation>()
            where TOperation : struct =>
            ScanReduceOperations.TryGetValue(Resolve(typeof(TOperation)), out var entry)
                ? entry
                : throw new NotSupportedException(
                    $"Scan / reduce operation {typeof(TOperation)} has no native implementation");
    }
}
