"""The GEMM kernels' tile scheduler (csrc/gemm_schedule.cuh, host/device code) on the host:
every element of C is produced exactly once for many shapes and both tile sizes
(tests/native/gemm_schedule_check.cc)."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_work_items_partition_the_output(tmp_path):
    exe = str(tmp_path / "sched")
    build = subprocess.run(["g++", "-std=c++17", "-O2", "-I",
                            os.path.join(ROOT, "bitscom_b200", "csrc"),
                            os.path.join(ROOT, "tests", "native", "gemm_schedule_check.cc"),
                            "-o", exe], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert run.stdout.startswith("ok:")
