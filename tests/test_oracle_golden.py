"""Pins the CPU oracle: every known-answer case the reference's unit tests hold for this
path (tests/golden/reference_kats.npz, written by tests/golden/make_golden.py) must come
out of the oracle exactly, and the oracle's fast closed forms must agree with its literal
restatements."""
import os

import numpy as np
import pytest

from oracle import cpu_oracle as oracle
from tests.helpers import NP

KATS = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.npz"))
KEYS = sorted(KATS.files)


def _cases(prefix, suffix):
    return [k[: -len(suffix)] for k in KEYS if k.startswith(prefix) and k.endswith(suffix)]


def test_sort_kats_literal_and_closed_form():
    cases = _cases("sort/", "/in")
    assert len(cases) >= 200
    for c in cases:
        descending = "/desc/" in c
        src, expected = KATS[c + "/in"], KATS[c + "/out"]
        for literal in (True, False):
            got, _ = oracle.radix_sort(src, descending=descending, literal=literal)
            np.testing.assert_array_equal(got, expected, err_msg=f"{c} literal={literal}")


def test_pairs_kats():
    for c in _cases("pairs/", "/in"):
        src, expected = KATS[c + "/in"], KATS[c + "/out"]
        for literal in (True, False):
            k, v = oracle.radix_sort(src, src.copy(), literal=literal)
            np.testing.assert_array_equal(k, expected)
            np.testing.assert_array_equal(v, expected)


def test_scan_kats():
    cases = _cases("scan/", "/in")
    assert len(cases) >= 200
    for c in cases:
        op = c.split("/")[2].lower()
        src = KATS[c + "/in"]
        for group in (16, 1024):   # default CPU device group size, and a GPU-like one
            np.testing.assert_array_equal(oracle.scan(src, op, True, group), KATS[c + "/incl"], err_msg=c)
            np.testing.assert_array_equal(oracle.scan(src, op, False, group), KATS[c + "/excl"], err_msg=c)


def test_reduce_kats():
    for c in _cases("reduce/", "/in"):
        op = c.split("/")[2].lower()
        src = KATS[c + "/in"]
        assert oracle.reduce(src, op) == KATS[c + "/out"][0], c
        assert oracle.reduce(src, op, grid_dim=3, group_dim=64, warp_size=32) == KATS[c + "/out"][0], c


def test_histogram_kats():
    for c in _cases("hist/", "/bins"):
        _, in_name, bin_name, num_bins = c.split("/")
        x = np.arange(1, 1025).astype(NP[in_name])
        bins, ov = oracle.histogram(x, np.zeros(int(num_bins), NP[bin_name]), "modulo")
        np.testing.assert_array_equal(bins, KATS[c + "/bins"], err_msg=c)
        np.testing.assert_array_equal(ov, KATS[c + "/overflow"], err_msg=c)


def test_histogram_overflow_kats():
    for c in _cases("histoverflow/", "/start"):
        _, in_name, bin_name = c.split("/")
        x = np.arange(1, 33).astype(NP[in_name])
        bins = KATS[c + "/start"].copy()
        _, ov = oracle.histogram(x, bins, "modulo")
        np.testing.assert_array_equal(bins, KATS[c + "/after1"])
        np.testing.assert_array_equal(ov, KATS[c + "/overflow1"])
        _, ov = oracle.histogram(x, bins, "modulo", overflow=ov)
        np.testing.assert_array_equal(bins, KATS[c + "/after2"])
        np.testing.assert_array_equal(ov, KATS[c + "/overflow2"])
        assert ov[0] == 1


@pytest.mark.parametrize("tname", list(NP.keys()))
@pytest.mark.parametrize("descending", [False, True])
def test_closed_form_sort_equals_literal_on_random_bits(tname, descending):
    rng = np.random.default_rng(17)
    t = np.dtype(NP[tname])
    raw = rng.integers(0, 2 ** 63, size=3001, dtype=np.uint64).astype(
        {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[t.itemsize])
    if t.itemsize == 8:
        raw ^= rng.integers(0, 2, size=raw.size, dtype=np.uint64) << np.uint64(63)
    keys = raw.view(t)
    values = np.arange(keys.size, dtype=np.uint32)
    lk, lv = oracle.radix_sort(keys, values, descending=descending, literal=True, num_groups=16)
    ck, cv = oracle.radix_sort(keys, values, descending=descending, literal=False)
    np.testing.assert_array_equal(lk.view(raw.dtype), ck.view(raw.dtype))
    np.testing.assert_array_equal(lv, cv)
    mt = oracle.radix_sort_literal_mt(keys, descending, 48, 3)
    np.testing.assert_array_equal(mt.view(raw.dtype), ck.view(raw.dtype))


def test_integer_key_order_is_numeric_and_stable():
    rng = np.random.default_rng(3)
    keys = rng.integers(-40, 40, size=5000).astype(np.int16)
    values = np.arange(keys.size, dtype=np.uint32)
    k, v = oracle.radix_sort(keys, values)
    order = np.argsort(keys, kind="stable")
    np.testing.assert_array_equal(k, keys[order])
    np.testing.assert_array_equal(v, values[order])
    k, v = oracle.radix_sort(keys, values, descending=True)
    order = np.argsort(-keys.astype(np.int32), kind="stable")
    np.testing.assert_array_equal(k, keys[order])
    np.testing.assert_array_equal(v, values[order])


def test_float_key_transform_literal_reading():
    # RadixSortOperations.tt:81-89 with an unsigned FloatAsInt: negative floats come first in
    # ascending magnitude; non-negative floats ascend except for a swapped mantissa LSB.
    import struct
    def bits(f):
        return struct.unpack("<I", struct.pack("<f", f))[0]
    assert oracle.key_bits("f32", bits(-1.0)) == bits(-1.0) ^ 0x80000000
    assert oracle.key_bits("f32", bits(1.0)) == bits(1.0) ^ 0x80000001
    assert oracle.key_bits("f64", 0x8000000000000000) == 0
    assert oracle.key_bits("f16", 0x3C00) == 0x3C00 ^ 0xFFFF
    assert oracle.key_bits("f16", 0xBC00) == 0xBC00 ^ 0xFFFE
    assert oracle.extract_radix_bits("i32", 0xFFFFFFFF, 30, 3, False) == 1   # -1 -> 0x7FFFFFFF
    assert oracle.extract_radix_bits("i32", 0xFFFFFFFF, 30, 3, True) == 2


def test_scan_chunk_association_for_floats():
    # chunked serial association (IL group scan): a different group size may change float
    # rounding but never integer results
    rng = np.random.default_rng(1)
    x = rng.integers(-1000, 1000, size=5000).astype(np.int64)
    np.testing.assert_array_equal(oracle.scan(x, "add", True, 16), np.cumsum(x))
    np.testing.assert_array_equal(oracle.scan(x, "add", False, 16)[1:], np.cumsum(x)[:-1])
    np.testing.assert_array_equal(oracle.scan(x, "max", True, 7), np.maximum.accumulate(x))
    f = rng.random(5000).astype(np.float32)
    a, b = oracle.scan(f, "add", True, 16), oracle.scan(f, "add", True, 64)
    assert np.allclose(a, b, rtol=1e-5)


def test_equal_width_locator_edges():
    f32 = lambda v: int(np.asarray([v], dtype=np.float32).view(np.uint32)[0])
    loc = lambda v: oracle.locate_bin("f32", f32(v), "equal_width_clamp", -4.0, 4.0, 256)
    assert loc(-4.0) == 0 and loc(-3.97) == 0 and loc(-3.96875) == 1
    assert loc(3.99) == 255 and loc(4.0) == 255 and loc(1e30) == 255 and loc(-1e30) == 0
    assert loc(float("nan")) == 0 and loc(float("inf")) == 255 and loc(float("-inf")) == 0
    assert loc(0.0) == 128 and loc(-0.0) == 128


def test_unique_reference_cases():
    # UniqueExtensionTests.tt:36-72: the expectation there drops an element equal to the last kept one
    for tname, t in NP.items():
        for repeat in (1, 317, 1025):
            length = 1025 if np.dtype(t).itemsize > 1 else 100
            host = np.repeat(np.arange(1, length + 1), repeat)[:length].astype(t)
            kept = [host[0]]
            for v in host[1:]:
                if kept[-1] != v:
                    kept.append(v)
            np.testing.assert_array_equal(oracle.unique(host), np.asarray(kept, dtype=t))
    f = np.asarray([0.0, -0.0, np.nan, np.nan, 1.0], dtype=np.float32)   # CompareTo: -0 == 0, NaN == NaN
    assert oracle.unique(f).size == 3
