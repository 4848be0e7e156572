"""The C-ABI library loads and exports every function include/b200alg.h declares (no
compute calls: this runs without a GPU)."""
import ctypes
import os
import re

from ilgpu_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200alg.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200alg_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared()
    assert len(declared) >= 14
    assert sorted(_native.SIGNATURES) == declared


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_native.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), name


def test_multi_gpu_library_exports_what_its_header_declares():
    text = open(os.path.join(ROOT, "include", "b200alg_mg.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = sorted(set(re.findall(r"\b(b200alg_[a-z0-9_]+)\s*\(", text)))
    assert sorted(_native.MG_SIGNATURES) == declared
    lib = _native.mg_lib()
    for name in declared:
        assert hasattr(lib, name), name
    # argument errors come back before any CUDA or NCCL call
    assert lib.b200alg_comm_unique_id(None) == _native.INVALID_ARGUMENT
    assert lib.b200alg_comm_status(None, None) == _native.INVALID_ARGUMENT


def test_host_only_entry_points():
    L = _native.lib()
    assert L.b200alg_version() == 100
    assert _native.status_string(0) == "success"
    assert "wait" in _native.status_string(_native.WAIT_LIMIT)
    out = ctypes.c_int64(0)
    assert L.b200alg_radix_sort_temp_bytes(_native.U32, 1 << 26, 0, ctypes.byref(out)) == 0
    assert out.value % 256 == 0 and out.value >= (1 << 26) * 4
    keys_only = out.value
    assert L.b200alg_radix_sort_temp_bytes(_native.U32, 1 << 26, 4, ctypes.byref(out)) == 0
    assert out.value >= keys_only + (1 << 26) * 4
    assert L.b200alg_radix_sort_temp_bytes(_native.U64, 1 << 28, 4, ctypes.byref(out)) == 0
    assert out.value // 4 < 2 ** 31          # fits the reference's Index1D count of ints
    assert L.b200alg_radix_sort_temp_bytes(_native.U32, 2 ** 31, 0, ctypes.byref(out)) == 0   # 64-bit lengths inside
    assert out.value >= 2 ** 33
    assert L.b200alg_radix_sort_temp_bytes(_native.U32, 2 ** 38 + 1, 0, ctypes.byref(out)) == _native.TOO_LARGE
    assert L.b200alg_radix_sort_temp_bytes(99, 10, 0, ctypes.byref(out)) == _native.UNSUPPORTED
    assert L.b200alg_scan_temp_bytes(_native.F32, 1 << 30, ctypes.byref(out)) == 0 and out.value > 0
    assert L.b200alg_scan_temp_bytes(_native.I8, 10, ctypes.byref(out)) == _native.UNSUPPORTED
    # argument errors are reported before any CUDA call
    assert L.b200alg_reduce(None, None, 1, 10, _native.I32, _native.ADD, None) == _native.INVALID_ARGUMENT
    assert L.b200alg_scan(None, None, 1, None, 1, 10, _native.I32, 0, 1, None, 0) == _native.INVALID_ARGUMENT
    assert L.b200alg_histogram(None, None, 1, 10, _native.F32, 0, 0.0, 1.0, None, 4, _native.I32, None) == _native.INVALID_ARGUMENT
    # a range that is fine in double but collapses in float is refused for float input (pointers are
    # only checked for null and alignment before that, never dereferenced on the host)
    fake = ctypes.c_void_p(4096)
    assert L.b200alg_histogram(None, fake, 1, 10, _native.F32, 0, 1.0, 1.0 + 1e-12, fake, 4, _native.I32, None) == _native.INVALID_ARGUMENT
    assert L.b200alg_histogram(None, fake, 1, 10, _native.F32, 0, -1e300, 1e300, fake, 4, _native.I32, None) == _native.INVALID_ARGUMENT


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "libb200alg.so"))
    with pytest.raises(_native.NativeLibraryMissing):
        _native.lib()
