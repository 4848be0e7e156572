"""B200-native radix sort, scan, reduce and histogram behind the ILGPU.Algorithms API.

The package needs its CUDA library (``ilgpu_b200/libb200alg.so``, built from
``ilgpu_b200/csrc``); there is no CPU or PyTorch fallback.
"""
from . import _native
from .algorithms import (
    Accelerator,
    ArgumentNullException,
    ArgumentOutOfRangeException,
    B200AlgException,
    EqualWidthClampLocator,
    InvalidOperationException,
    ModuloLocator,
    NotSupportedException,
    RadixSortOperations,
    RadixSortProvider,
    ScanKind,
    ScanProvider,
    ScanReduceOperations,
    Sequencer,
    Sequencers,
)

__all__ = [
    "Accelerator", "ArgumentNullException", "ArgumentOutOfRangeException", "B200AlgException",
    "EqualWidthClampLocator", "InvalidOperationException", "ModuloLocator", "NotSupportedException",
    "RadixSortOperations", "RadixSortProvider", "ScanKind", "ScanProvider", "ScanReduceOperations",
    "Sequencer", "Sequencers",
    "_native",
]
