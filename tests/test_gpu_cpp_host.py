"""Runs the C++ host mirror's own test program (tests/cpp/host_mirror_test.cpp): the
reference's unit-test cases driven through include/ilgpu_algorithms.hpp and the C ABI."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_cpp_host_mirror_passes_reference_cases():
    exe = os.path.join(HERE, "cpp", "host_mirror_test")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-C", os.path.join(HERE, "cpp")])
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-4000:] + run.stderr[-2000:]
    assert "0 failures" in run.stdout
