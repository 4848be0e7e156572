// Not compiled in this repository: no .NET SDK on the build machines (see README.md).
// Follows Src/ILGPU.Algorithms/Runtime/Cuda/CuRandException.cs.
using System;
using System.Runtime.CompilerServices;
using System.Runtime.InteropServices;

namespace ILGPU.Runtime.Cuda
{
    /// <summary>Status codes of libb200alg (include/b200alg.h, b200alg_status).</summary>
    public enum B200AlgStatus : int
    {
        Success = 0,
        InvalidArgument = 1,
        Unsupported = 2,
        TempTooSmall = 3,
        CudaError = 4,
        WaitLimit = 5,
        Misaligned = 6,
        TooLarge = 7,
        StaticLimit = 8,
        NcclError = 9,
    }

    /// <summary>An error reported by libb200alg.</summary>
    [Serializable]
    public sealed class B200AlgException : Exception
    {
        public B200AlgException(B200AlgStatus error)
            : base(Marshal.PtrToStringAnsi(B200AlgAPI.b200alg_status_string((int)error)) +
                   (error == B200AlgStatus.CudaError
                       ? $" [cudaError {B200AlgAPI.b200alg_last_cuda_error()}]"
                       : string.Empty))
        {
            Error = error;
        }

        /// <summary>Returns the error.</summary>
        public B200AlgStatus Error { get; }

        /// <summary>
        /// Throws on failure.  Argument errors keep the exception kinds the reference's own
        /// checks use (ScanExtensions.cs:675-689, TempViewManager.cs:36-37, 88-89).
        /// </summary>
        [MethodImpl(MethodImplOptions.AggressiveInlining)]
        public static void ThrowIfFailed(int status)
        {
            switch ((B200AlgStatus)status)
            {
                case B200AlgStatus.Success:
                    return;
                case B200AlgStatus.TooLarge:
                    throw new NotSupportedException(
                        "The current array view is too large (NotSupportedArrayView64)");
                case B200AlgStatus.TempTooSmall:
                    throw new ArgumentOutOfRangeException("temp");
                case B200AlgStatus.Unsupported:
                    throw new NotSupportedException(
                        Marshal.PtrToStringAnsi(B200AlgAPI.b200alg_status_string(status)));
                default:
                    throw new B200AlgException((B200AlgStatus)status);
            }
        }
    }
}
