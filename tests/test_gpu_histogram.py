"""GPU parity of the histogram against the CPU oracle (through the C ABI).

Mirrors ILGPU.Algorithms.Tests/HistogramTests.tt:101-203: inputs 1..1024 into 64 / 256
modulo bins for every input type x bin type, and the overflow scenario; then the
equal-width clamping locator on seeded normal data (bit-exact counts).
"""
import numpy as np
import pytest
import torch

from ilgpu_b200 import EqualWidthClampLocator, ModuloLocator
from ilgpu_b200 import synthetic
from oracle import cpu_oracle as oracle
from tests.helpers import ATOMIC, NP, to_device, to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in_t", ATOMIC)
@pytest.mark.parametrize("bin_t", ATOMIC)
@pytest.mark.parametrize("num_bins", [64, 256])
def test_modulo_bins_reference_case(accelerator, in_t, bin_t, num_bins):
    x = np.arange(1, 1025).astype(NP[in_t])
    expected, expected_of = oracle.histogram(x, np.zeros(num_bins, NP[bin_t]), "modulo")
    bins = torch.zeros(num_bins, dtype=to_device(expected).dtype, device="cuda")
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    accelerator.Histogram(None, to_device(x), bins, overflow, ModuloLocator())
    np.testing.assert_array_equal(to_host(bins), expected)
    np.testing.assert_array_equal(to_host(overflow), expected_of)


@pytest.mark.parametrize("in_t", ATOMIC)
@pytest.mark.parametrize("bin_t", ["Int32", "Int64", "UInt32", "UInt64"])
def test_overflow_reference_case(accelerator, in_t, bin_t):
    # HistogramTests.tt:146-203: one bin pre-loaded just below MaxValue, 32 inputs, twice.
    length = 32
    x = np.arange(1, length + 1).astype(NP[in_t])
    info = np.iinfo(NP[bin_t])
    start = np.asarray([info.max - length - 1], dtype=NP[bin_t])
    expected = start.copy()
    _, of1 = oracle.histogram(x, expected, "modulo")
    assert of1[0] == 0
    bins = to_device(expected.copy())
    _, of2 = oracle.histogram(x, expected, "modulo")
    assert of2[0] == 1
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    accelerator.Histogram(None, to_device(x), bins, overflow, ModuloLocator())
    np.testing.assert_array_equal(to_host(bins), expected)
    np.testing.assert_array_equal(to_host(overflow), of2)


@pytest.mark.parametrize("n", [1, 31, 4097, 1 << 20, (1 << 22) + 77])
def test_equal_width_normal_data(accelerator, n):
    x = synthetic.normal_float32(n, seed=3)
    x[::97] = np.float32(9.5)       # clamps to the last bin
    x[1::89] = np.float32(-1e30)    # clamps to the first bin
    if n > 10:
        x[5] = np.float32("nan")
        x[7] = np.float32("inf")
    expected, _ = oracle.histogram(x, np.zeros(256, np.int32), "equal_width_clamp", -4.0, 4.0)
    assert expected.sum() == n
    bins = torch.zeros(256, dtype=torch.int32, device="cuda")
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    accelerator.Histogram(None, to_device(x), bins, overflow, EqualWidthClampLocator(-4.0, 4.0))
    np.testing.assert_array_equal(to_host(bins), expected)
    assert to_host(overflow)[0] == 0
    # accumulates into the bins, never clears them
    accelerator.HistogramUnchecked(None, to_device(x), bins, EqualWidthClampLocator(-4.0, 4.0))
    np.testing.assert_array_equal(to_host(bins), expected * 2)


@pytest.mark.parametrize("in_t", ["Int32", "UInt64", "Double"])
@pytest.mark.parametrize("num_bins", [1, 7, 1000, 20_000])
def test_equal_width_other_types_and_bin_counts(accelerator, in_t, num_bins):
    rng = np.random.default_rng(num_bins)
    x = (rng.random(200_003) * 1200 - 100).astype(NP[in_t]) if in_t != "UInt64" else rng.integers(0, 1200, 200_003).astype(np.uint64)
    expected, _ = oracle.histogram(x, np.zeros(num_bins, np.int64), "equal_width_clamp", 0.0, 1000.0)
    bins = torch.zeros(num_bins, dtype=torch.int64, device="cuda")
    accelerator.HistogramUnchecked(None, to_device(x), bins, EqualWidthClampLocator(0.0, 1000.0))
    np.testing.assert_array_equal(to_host(bins), expected)


def test_strided_input(accelerator):
    x = synthetic.normal_float32(30_000, seed=8)
    view = to_device(x)[::3]
    expected, _ = oracle.histogram(x, np.zeros(64, np.uint32), "equal_width_clamp", -3.0, 3.0, stride=3)
    bins = torch.zeros(64, dtype=torch.uint32, device="cuda")
    accelerator.HistogramUnchecked(None, view, bins, EqualWidthClampLocator(-3.0, 3.0))
    np.testing.assert_array_equal(to_host(bins), expected)


def test_float_bins_beyond_2_pow_24_the_stated_exception(accelerator):
    """The one stated parity exception of the histogram.  The reference adds 1.0f per element, so
    a float bin stops growing at 2^24 (16777216.0f + 1.0f == 16777216.0f); here a block's count
    goes in with one atomic add, so the bin keeps counting.  Below 2^24 the two agree exactly
    (the cases above); this test pins the behaviour beyond it: 2^25 elements into one float bin
    give exactly 2^25, the overflow flag stays clear, and an int32 bin next to it agrees."""
    n = 1 << 25
    x = torch.zeros(n, dtype=torch.int32, device="cuda")          # modulo locator: everything lands in bin 0
    float_bins = torch.zeros(4, dtype=torch.float32, device="cuda")
    int_bins = torch.zeros(4, dtype=torch.int32, device="cuda")
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    accelerator.Histogram(None, x, float_bins, overflow, ModuloLocator())
    accelerator.Histogram(None, x, int_bins, overflow, ModuloLocator())
    assert float(float_bins[0]) == float(n) and float(float_bins[1:].abs().sum()) == 0.0
    assert int(int_bins[0]) == n
    assert int(overflow[0]) == 0
    assert np.float32(2 ** 24) + np.float32(1) == np.float32(2 ** 24)   # where the reference's bin would have stopped
