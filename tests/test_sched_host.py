"""The host-side control around the attention step (include/battn_sched.h: slot pool with prefix affinity, the
batching step scheduler with chunked prompts, the prompt-lookup drafter, the speculative round, per-row-count
graphs) against a fake engine: compiled with g++ and run on the CPU."""
import os
import shutil
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_scheduler_drafter_and_spec_round_with_a_fake_engine():
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "sched_test")
        r = subprocess.run([gxx, "-std=c++17", "-O1", "-pthread", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"),
                            os.path.join(ROOT, "tests", "host", "sched_test.cpp"), "-o", exe], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and r.stdout.strip() == "OK", r.stdout + r.stderr


def test_work_cut_and_merge_ranges_on_the_host():
    """csrc/work_cut.h -- the integer logic the attention kernels and the merge share -- over many shapes."""
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "cut_test")
        r = subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Wextra", os.path.join(ROOT, "tests", "host", "cut_test.cpp"),
                            "-o", exe], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and r.stdout.strip() == "OK", r.stdout + r.stderr
