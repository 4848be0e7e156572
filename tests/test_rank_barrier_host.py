"""The bounded flag barrier of the multi-GPU library, exercised on the CPU: two host threads
stand for two ranks (tests/cpp/barrier_host_test.cpp instantiates the same template the
device kernel uses).  One case has a rank that never arrives; the other rank must give up
after its poll limit and report it.  No GPU."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_rank_barrier_with_and_without_the_other_rank(tmp_path):
    exe = str(tmp_path / "barrier_host_test")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-pthread", "-I", os.path.join(ROOT, "ilgpu_b200", "csrc"),
                           os.path.join(HERE, "cpp", "barrier_host_test.cpp"), "-o", exe])
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "0 failures" in run.stdout
