"""ctypes binding of ``libb200alg.so`` (the C ABI declared in ``include/b200alg.h``).

There is no fallback: if the shared library is missing or fails to load, importing the
algorithms raises.  Build it with ``python -c "import __graft_entry__ as g; g.build()"``
or ``make -C ilgpu_b200/csrc``.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200ALG_LIBRARY overrides the path of the shared library (e.g. a differently tuned build).
LIB_PATH = os.environ.get("B200ALG_LIBRARY") or os.path.join(_HERE, "libb200alg.so")

# status codes (include/b200alg.h)
OK, INVALID_ARGUMENT, UNSUPPORTED, TEMP_TOO_SMALL, CUDA_ERROR, WAIT_LIMIT, MISALIGNED, TOO_LARGE, STATIC_LIMIT = range(9)

# dtype codes
I8, U8, I16, U16, I32, U32, I64, U64, F16, F32, F64 = range(11)
ADD, MAX, MIN = range(3)
SORT_ASCENDING, SORT_DESCENDING, SORT_FLOAT_TOTAL_ORDER = 0, 1, 2
LOCATOR_EQUAL_WIDTH_CLAMP, LOCATOR_MODULO = 0, 1

_i64, _int, _vp, _dbl = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_double

# name -> (restype, argtypes); every symbol include/b200alg.h declares
SIGNATURES = {
    "b200alg_version": (_int, []),
    "b200alg_status_string": (ctypes.c_char_p, [_int]),
    "b200alg_last_cuda_error": (_int, []),
    "b200alg_radix_sort_temp_bytes": (_int, [_int, _i64, _int, ctypes.POINTER(_i64)]),
    "b200alg_radix_sort_keys": (_int, [_vp, _vp, _i64, _i64, _int, _int, _vp, _i64]),
    "b200alg_radix_sort_pairs": (_int, [_vp, _vp, _vp, _i64, _int, _int, _int, _vp, _i64]),
    "b200alg_radix_sort_pairs_sequence": (_int, [_vp, _vp, _vp, _i64, _int, _int, _int, _vp, _i64]),
    "b200alg_radix_sort_out_of_place": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _int, _int, _int, _vp, _i64]),
    "b200alg_bucket_partition_temp_bytes": (_int, [_int, _i64, ctypes.POINTER(_i64)]),
    "b200alg_bucket_partition": (_int, [_vp, _vp, _vp, _i64, _int, _int, _int, _vp, _vp, _int, _i64, _vp, _vp, _vp, _vp, _i64]),
    "b200alg_bucket_count": (_int, [_vp, _vp, _i64, _int, _int, _vp, _vp, _int, _i64, _vp, _vp, _i64]),
    "b200alg_bucket_scatter": (_int, [_vp, _vp, _vp, _i64, _int, _int, _int, _vp, _vp, _int, _i64, _vp, _vp, _vp, _i64]),
    "b200alg_select_splitters": (_int, [_vp, _vp, _vp, _i64, _vp, _int, _int, _int, _vp, _vp, _vp, _i64]),
    "b200alg_scan_temp_bytes": (_int, [_int, _i64, ctypes.POINTER(_i64)]),
    "b200alg_scan": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _int, _int, _int, _vp, _i64]),
    "b200alg_scan_carry": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _int, _int, _int, _vp, _vp, _i64]),
    "b200alg_scan_static": (_int, [_vp, _vp, _i64, _vp, _i64, _i64, _int, _int, _int]),
    "b200alg_reduce": (_int, [_vp, _vp, _i64, _i64, _int, _int, _vp]),
    "b200alg_histogram": (_int, [_vp, _vp, _i64, _i64, _int, _int, _dbl, _dbl, _vp, _i64, _int, _vp]),
    "b200alg_initialize": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "b200alg_sequence": (_int, [_vp, _vp, _i64, _int, _i64, _i64]),
    "b200alg_unique_temp_bytes": (_int, [_int, _i64, ctypes.POINTER(_i64)]),
    "b200alg_unique": (_int, [_vp, _vp, _i64, _int, _vp, _vp, _i64]),
    "b200alg_run_length_encode_temp_bytes": (_int, [_int, _i64, ctypes.POINTER(_i64)]),
    "b200alg_run_length_encode": (_int, [_vp, _vp, _i64, _int, _vp, _vp, _vp, _vp, _i64]),
    "b200alg_device_status": (_int, [_vp, _vp]),
}

# multi-GPU layer (include/b200alg_mg.h): libb200alg_mg.so, loaded on first use
MG_LIB_PATH = os.environ.get("B200ALG_MG_LIBRARY") or os.path.join(_HERE, "libb200alg_mg.so")
NCCL_ERROR = 9
UNIQUE_ID_BYTES = 128
_pp = ctypes.POINTER(ctypes.c_void_p)
MG_SIGNATURES = {
    "b200alg_comm_unique_id": (_int, [_vp]),
    "b200alg_comm_create_rank": (_int, [_vp, _int, _int, _i64, _pp]),
    "b200alg_comm_create": (_int, [_int, ctypes.POINTER(_int), _i64, _pp]),
    "b200alg_comm_destroy": (_int, [_vp]),
    "b200alg_comm_rank": (_int, [_vp, ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "b200alg_comm_status": (_int, [_vp, _vp]),
    "b200alg_comm_last_nccl_error": (_int, [_vp]),
    "b200alg_reduce_mg": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _vp]),
    "b200alg_histogram_mg": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _int, _dbl, _dbl, _vp, _i64, _int, _vp]),
    "b200alg_scan_mg": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _int, _int, _vp, _i64]),
    "b200alg_sort_mg": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _int, _int, _vp, _vp, _i64, _vp]),
}

_lib = None
_mg_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def mg_lib() -> ctypes.CDLL:
    """Loads the multi-GPU library once (it needs NCCL and libb200alg.so); raises
    NativeLibraryMissing when it is not built."""
    global _mg_lib
    if _mg_lib is None:
        lib()  # the single-GPU library first: the multi-GPU one links against it
        if not os.path.exists(MG_LIB_PATH):
            raise NativeLibraryMissing(f"{MG_LIB_PATH} not found; build it with `make -C ilgpu_b200/csrc`")
        L = ctypes.CDLL(MG_LIB_PATH)
        for name, (res, args) in MG_SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _mg_lib = L
    return _mg_lib


def lib() -> ctypes.CDLL:
    """Loads the library once; raises NativeLibraryMissing when it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryMissing(
                f"{LIB_PATH} not found: the CUDA library is required (there is no CPU or "
                "PyTorch fallback); build it with `make -C ilgpu_b200/csrc`")
        L = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().b200alg_status_string(status).decode()
