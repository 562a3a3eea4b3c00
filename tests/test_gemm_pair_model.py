"""The barrier protocol of the CTA-pair GEMM (csrc/gemm_tcgen05_2cta.cu) as a host model
(tests/native/gemm_pair_model.cc): both CTAs' producers and epilogue warps, the leader's MMA
issuer, a tensor pipe and two copy engines as threads (both CTAs' loads complete on the leader's
barrier); ring stages and accumulator buffers tagged with what they hold.  The protocol must run clean for
1 to 8 tiles of 1 to 64 k-blocks; three seeded bugs must be noticed."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "gemm_pair_model.cc")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _run(tmp_path, flags, name):
    exe = str(tmp_path / name)
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread"] + flags + [SRC, "-o", exe],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    return subprocess.run([exe], capture_output=True, text=True, timeout=900)


def test_pair_protocol_runs_clean(tmp_path):
    run = _run(tmp_path, [], "pair")
    assert run.returncode == 0, (run.stdout[-300:], run.stderr[-2000:])
    assert run.stdout.startswith("ok: cta pair")


@pytest.mark.parametrize("bug", [1, 2, 3])
def test_a_protocol_bug_is_detected(tmp_path, bug):
    run = _run(tmp_path, [f"-DBUG={bug}"], f"bug{bug}")
    assert run.returncode == 3, "the seeded bug went unnoticed"
    assert "violation:" in run.stderr
