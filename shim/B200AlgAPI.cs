// Not compiled in this repository: no .NET SDK on the build machines (see README.md).
// One declaration per export of include/b200alg.h, in the shape that
// Src/ILGPU/Static/DllImporter.ttinclude:169-226 generates for the cuRAND / cuBLAS bindings:
// blittable arguments only (IntPtr pointers and streams, long counts, int enums, double scalars).
using System;
using System.Runtime.InteropServices;

namespace ILGPU.Runtime.Cuda
{
    internal static unsafe partial class B200AlgAPI
    {
        /// <summary>libb200alg.so / b200alg.dll; override with the B200ALG_LIBRARY variable.</summary>
        private const string LibName = "b200alg";

#if NET7_0_OR_GREATER
        [LibraryImport(LibName)] internal static partial int b200alg_version();
        [LibraryImport(LibName)] internal static partial IntPtr b200alg_status_string(int status);
        [LibraryImport(LibName)] internal static partial int b200alg_last_cuda_error();

        // radix sort: RadixSortExtensions.cs:384-447 (temp sizes), :1130-1337 (keys), :1017-1118 (pairs)
        [LibraryImport(LibName)] internal static partial int b200alg_radix_sort_temp_bytes(
            int keyDtype, long n, int valueBytes, out long bytes);
        [LibraryImport(LibName)] internal static partial int b200alg_radix_sort_keys(
            IntPtr stream, IntPtr keys, long n, long stride, int keyDtype, int order, IntPtr temp, long tempBytes);
        [LibraryImport(LibName)] internal static partial int b200alg_radix_sort_pairs(
            IntPtr stream, IntPtr keys, IntPtr values, long n, int keyDtype, int valueBytes, int order,
            IntPtr temp, long tempBytes);
        [LibraryImport(LibName)] internal static partial int b200alg_radix_sort_pairs_sequence(
            IntPtr stream, IntPtr keys, IntPtr values, long n, int keyDtype, int valueDtype, int order,
            IntPtr temp, long tempBytes);
        [LibraryImport(LibName)] internal static partial int b200alg_radix_sort_out_of_place(
            IntPtr stream, IntPtr inKeys, IntPtr inValues, IntPtr outKeys, IntPtr outValues, long n,
            IntPtr nDevice, int keyDtype, int valueBytes, int order, IntPtr temp, long tempBytes);

        // scan: ScanExtensions.cs:158-170 (temp size), :930-959 (CreateScan)
        [LibraryImport(LibName)] internal static partial int b200alg_scan_temp_bytes(int dtype, long n, out long bytes);
        [LibraryImport(LibName)] internal static partial int b200alg_scan(
            IntPtr stream, IntPtr input, long inStride, IntPtr output, long outStride, long n,
            int dtype, int op, int inclusive, IntPtr temp, long tempBytes);
        [LibraryImport(LibName)] internal static partial int b200alg_scan_carry(
            IntPtr stream, IntPtr input, long inStride, IntPtr output, long outStride, long n,
            int dtype, int op, int inclusive, IntPtr carryIn, IntPtr temp, long tempBytes);
        [LibraryImport(LibName)] internal static partial int b200alg_scan_static(
            IntPtr stream, IntPtr input, long inStride, IntPtr output, long outStride, long n,
            int dtype, int op, int inclusive);

        // reduce: ReductionExtensions.cs:135-167
        [LibraryImport(LibName)] internal static partial int b200alg_reduce(
            IntPtr stream, IntPtr input, long stride, long n, int dtype, int op, IntPtr output);

        // histogram: HistogramExtensions.cs:293-427
        [LibraryImport(LibName)] internal static partial int b200alg_histogram(
            IntPtr stream, IntPtr input, long stride, long n, int inDtype, int locator, double lo, double hi,
            IntPtr bins, long numBins, int binDtype, IntPtr overflowOrNull);

        // edges of the path: InitializeExtensions.cs, SequenceExtensions.cs, UniqueExtensions.cs:59-220
        [LibraryImport(LibName)] internal static partial int b200alg_initialize(
            IntPtr stream, IntPtr view, long stride, long n, int elemBytes, void* value);
        [LibraryImport(LibName)] internal static partial int b200alg_sequence(
            IntPtr stream, IntPtr view, long n, int dtype, long start, long step);
        [LibraryImport(LibName)] internal static partial int b200alg_unique_temp_bytes(int dtype, long n, out long bytes);
        [LibraryImport(LibName)] internal static partial int b200alg_unique(
            IntPtr stream, IntPtr data, long n, int dtype, IntPtr outCount, IntPtr temp, long tempBytes);

        [LibraryImport(LibName)] internal static partial int b200alg_device_status(IntPtr stream, IntPtr temp);
#else
        [DllImport(LibName)] internal static extern int b200alg_version();
        [DllImport(LibName)] internal static extern IntPtr b200alg_status_string(int status);
        [DllImport(LibName)] internal static extern int b200alg_last_cuda_error();
        [DllImport(LibName)] internal static extern int b200alg_radix_sort_temp_bytes(
            int keyDtype, long n, int valueBytes, out long bytes);
        [DllImport(LibName)] internal static extern int b200alg_radix_sort_keys(
            IntPtr stream, IntPtr keys, long n, long stride, int keyDtype, int order, IntPtr temp, long tempBytes);
        [DllImport(LibName)] internal static extern int b200alg_radix_sort_pairs(
            IntPtr stream, IntPtr keys, IntPtr values, long n, int keyDtype, int valueBytes, int order,
            IntPtr temp, long tempBytes);
        [DllImport(LibName)] internal static extern int b200alg_radix_sort_pairs_sequence(
            IntPtr stream, IntPtr keys, IntPtr values, long n, int keyDtype, int valueDtype, int order,
            IntPtr temp, long tempBytes);
        [DllImport(LibName)] internal static extern int b200alg_scan_temp_bytes(int dtype, long n, out long bytes);
        [DllImport(LibName)] internal static extern int b200alg_scan(
            IntPtr stream, IntPtr input, long inStride, IntPtr output, long outStride, long n,
            int dtype, int op, int inclusive, IntPtr temp, long tempBytes);
        [DllImport(LibName)] internal static extern int b200alg_reduce(
            IntPtr stream, IntPtr input, long stride, long n, int dtype, int op, IntPtr output);
        [DllImport(LibName)] internal static extern int b200alg_histogram(
            IntPtr stream, IntPtr input, long stride, long n, int inDtype, int locator, double lo, double hi,
            IntPtr bins, long numBins, int binDtype, IntPtr overflowOrNull);
        [DllImport(LibName)] internal static extern int b200alg_device_status(IntPtr stream, IntPtr temp);
#endif
    }
}
