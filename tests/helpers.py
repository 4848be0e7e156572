"""Shared helpers of the GPU parity tests: ramps as the reference's test sequencers build
them (ILGPU.Algorithms.Tests/Generic/AlgorithmsTestData.tt:74-96) and dtype tables."""
import numpy as np
import torch

# sizes of the reference's algorithm tests (Generic/ConfigurationBase.tt:80) plus tile edges
REFERENCE_SIZES = [1, 31, 33, 127, 1027]
EDGE_SIZES = [2047, 2048, 2049, 4095, 4096, 4097, 8191, 8192, 8193, 100_003]

NP = {
    "Int8": np.int8, "UInt8": np.uint8, "Int16": np.int16, "UInt16": np.uint16, "Int32": np.int32,
    "UInt32": np.uint32, "Int64": np.int64, "UInt64": np.uint64, "Half": np.float16,
    "Float": np.float32, "Double": np.float64,
}
ATOMIC = ["Int32", "Int64", "UInt32", "UInt64", "Float", "Double"]


def compute_sequence(np_dtype, start, step, length):
    """{T}TestSequencer.ComputeSequence: sequence[i] = sequence[i-1] + stepSize."""
    with np.errstate(over="ignore"):
        return (np.arange(length, dtype=np.int64) * step + start).astype(np_dtype)


def compute_inverted_sequence(np_dtype, start, step, length):
    """{T}TestSequencer.ComputeInvertedSequence: the same ramp, last element first."""
    return compute_sequence(np_dtype, start, step, length)[::-1].copy()


def to_device(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_host(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy()
