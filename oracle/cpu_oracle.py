"""ctypes/numpy front end of the CPU oracle (``ilgpu_cpu_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libilgpu_cpu_oracle.so")

# dtype codes shared with include/b200alg.h
DTYPES = {
    "i8": 0, "u8": 1, "i16": 2, "u16": 3, "i32": 4, "u32": 5,
    "i64": 6, "u64": 7, "f16": 8, "f32": 9, "f64": 10,
}
NP_DTYPES = {
    "i8": np.int8, "u8": np.uint8, "i16": np.int16, "u16": np.uint16, "i32": np.int32,
    "u32": np.uint32, "i64": np.int64, "u64": np.uint64, "f16": np.float16,
    "f32": np.float32, "f64": np.float64,
}
OPS = {"add": 0, "max": 1, "min": 2}
LOCATORS = {"equal_width_clamp": 0, "modulo": 1}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "ilgpu_cpu_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libilgpu_cpu_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, i32, vp, dbl, u64 = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_double, ctypes.c_uint64
        L.oracle_key_bits.restype = u64
        L.oracle_key_bits.argtypes = [i32, u64]
        L.oracle_extract_radix_bits.restype = i32
        L.oracle_extract_radix_bits.argtypes = [i32, u64, i32, i32, i32]
        L.oracle_radix_sort_literal.argtypes = [i32, vp, vp, i32, i64, i32, i32]
        L.oracle_radix_sort_literal_mt.argtypes = [i32, vp, i64, i32, i32, i32]
        L.oracle_radix_sort.argtypes = [i32, vp, vp, i32, i64, i32]
        L.oracle_scan.argtypes = [i32, i32, i32, vp, i64, vp, i64, i64, i32]
        L.oracle_reduce.argtypes = [i32, i32, vp, i64, i64, vp, i32, i32, i32]
        L.oracle_locate_bin.restype = i64
        L.oracle_locate_bin.argtypes = [i32, u64, i32, dbl, dbl, i64]
        L.oracle_unique.restype = i64
        L.oracle_unique.argtypes = [i32, vp, i64]
        L.oracle_histogram.argtypes = [i32, vp, i64, i64, i32, dbl, dbl, i32, vp, i64, vp]
        _lib = L
    return _lib


def _code(np_dtype) -> tuple[str, int]:
    for name, t in NP_DTYPES.items():
        if np.dtype(t) == np.dtype(np_dtype):
            return name, DTYPES[name]
    raise TypeError(f"unsupported dtype {np_dtype}")


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def key_bits(dtype: str, raw: int) -> int:
    return int(lib().oracle_key_bits(DTYPES[dtype], ctypes.c_uint64(raw)))


def extract_radix_bits(dtype: str, raw: int, shift: int, mask: int, descending: bool) -> int:
    return int(lib().oracle_extract_radix_bits(DTYPES[dtype], ctypes.c_uint64(raw), shift, mask, int(descending)))


def radix_sort(keys: np.ndarray, values: np.ndarray | None = None, descending: bool = False,
               literal: bool = False, num_groups: int = 16):
    """Returns sorted copies ``(keys, values)``.  ``literal`` runs the two-kernel 2-bit
    restatement (slow, small n); otherwise the equivalent stable LSD closed form."""
    _, code = _code(keys.dtype)
    k = np.ascontiguousarray(keys).copy()
    v = None if values is None else np.ascontiguousarray(values).copy()
    vb = 0 if v is None else v.dtype.itemsize
    vp = None if v is None else _ptr(v)
    if literal:
        rc = lib().oracle_radix_sort_literal(code, _ptr(k), vp, vb, k.size, int(descending), num_groups)
    else:
        rc = lib().oracle_radix_sort(code, _ptr(k), vp, vb, k.size, int(descending))
    assert rc == 0
    return k, v


def radix_sort_literal_mt(keys: np.ndarray, descending: bool, num_groups: int, num_threads: int) -> np.ndarray:
    _, code = _code(keys.dtype)
    k = np.ascontiguousarray(keys).copy()
    rc = lib().oracle_radix_sort_literal_mt(code, _ptr(k), k.size, int(descending), num_groups, num_threads)
    assert rc == 0
    return k


def scan(values: np.ndarray, op: str = "add", inclusive: bool = True, group_size: int = 16,
         in_stride: int = 1, out_stride: int = 1) -> np.ndarray:
    """``values`` holds the strided input storage; returns the strided output storage
    (untouched slots are zero)."""
    _, code = _code(values.dtype)
    src = np.ascontiguousarray(values)
    n = 0 if src.size == 0 else (src.size - 1) // in_stride + 1
    out = np.zeros(max(0, (n - 1) * out_stride + 1) if n else 0, dtype=src.dtype)
    rc = lib().oracle_scan(code, OPS[op], int(inclusive), _ptr(src), in_stride, _ptr(out), out_stride, n, group_size)
    assert rc == 0
    return out


def reduce(values: np.ndarray, op: str = "add", grid_dim: int = 1, group_dim: int = 16,
           warp_size: int = 4, stride: int = 1):
    _, code = _code(values.dtype)
    src = np.ascontiguousarray(values)
    n = (src.size - 1) // stride + 1
    out = np.zeros(1, dtype=src.dtype)
    rc = lib().oracle_reduce(code, OPS[op], _ptr(src), stride, n, _ptr(out), grid_dim, group_dim, warp_size)
    assert rc == 0
    return out[0]


def locate_bin(dtype: str, raw: int, locator: str, lo: float, hi: float, num_bins: int) -> int:
    return int(lib().oracle_locate_bin(DTYPES[dtype], ctypes.c_uint64(raw), LOCATORS[locator], lo, hi, num_bins))


def histogram(values: np.ndarray, bins: np.ndarray, locator: str = "equal_width_clamp",
              lo: float = 0.0, hi: float = 1.0, overflow: np.ndarray | None = None, stride: int = 1):
    """Accumulates into ``bins`` (in place) and ORs the overflow flag into
    ``overflow[0]`` (int32, in place); returns ``(bins, overflow)``."""
    _, in_code = _code(values.dtype)
    _, bin_code = _code(bins.dtype)
    src = np.ascontiguousarray(values)
    n = 0 if src.size == 0 else (src.size - 1) // stride + 1
    if overflow is None:
        overflow = np.zeros(1, dtype=np.int32)
    assert bins.flags.c_contiguous and overflow.dtype == np.int32
    rc = lib().oracle_histogram(in_code, _ptr(src), stride, n, LOCATORS[locator], lo, hi,
                                bin_code, _ptr(bins), bins.size, _ptr(overflow))
    assert rc == 0, rc
    return bins, overflow


def unique(values: np.ndarray) -> np.ndarray:
    """Consecutive duplicates removed (a copy, cut to the new length)."""
    _, code = _code(values.dtype)
    a = np.ascontiguousarray(values).copy()
    m = lib().oracle_unique(code, _ptr(a), a.size)
    return a[:m]
