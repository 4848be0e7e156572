"""Runs the compiled test programs under tests/cpp: the C++ host mirror replaying the
reference's unit-test cases through include/ilgpu_algorithms.hpp and the C ABI, the
device-side header, and the library inside a second CUDA context."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(name):
    exe = os.path.join(HERE, "cpp", name)
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-C", os.path.join(HERE, "cpp")])
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-4000:] + run.stderr[-2000:]
    assert "0 failures" in run.stdout


def test_cpp_host_mirror_passes_reference_cases():
    _run("host_mirror_test")


def test_device_side_header_sorts_and_permutes_like_the_reference_helpers():
    """tests/cpp/device_header_test.cu: include/b200alg_device.cuh against host computations."""
    _run("device_header_test")


def test_library_in_a_second_cuda_context():
    """tests/cpp/context_test.cpp: sort, scan and the scan with built-in scratch in the primary
    context and in a context created the way ILGPU creates its own."""
    _run("context_test")
