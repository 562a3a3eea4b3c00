"""The small-bucket form of the fused all-reduce ({word, epoch} pairs polled by the consumer,
no fence, no flag handshake, slots reused by the next launch without a barrier) as a
multi-threaded host model (tests/native/ll_protocol_model.cc), also under ThreadSanitizer.  Two
seeded bugs show that the model notices a rank that runs a launch ahead and an epoch that
repeats."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "ll_protocol_model.cc")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _build(tmp_path, flags, name):
    exe = str(tmp_path / name)
    out = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread"] + flags + [SRC, "-o", exe],
                         capture_output=True, text=True, timeout=300)
    if out.returncode != 0 and "sanitize" in out.stderr and "cannot find" in out.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert out.returncode == 0, out.stderr[-3000:]
    return exe


@pytest.mark.parametrize("flags", [[], ["-fsanitize=thread"]], ids=["plain", "tsan"])
def test_slots_can_be_reused_without_a_barrier(tmp_path, flags):
    exe = _build(tmp_path, flags, "ll_model")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1"))
    assert run.returncode == 0, (run.stdout[-500:], run.stderr[-4000:])
    assert run.stdout.startswith("ok:")


@pytest.mark.parametrize("bug", [1, 2])
def test_seeded_bugs_are_detected(tmp_path, bug):
    """A rank that does not wait in phase 3 runs ahead and overwrites pairs a slow peer still
    needs; an epoch that repeats lets a stale pair through."""
    exe = _build(tmp_path, [f"-DBUG={bug}"], f"ll_model_bug{bug}")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900)
    assert run.returncode != 0, "the seeded bug went unnoticed"
    assert "protocol violation" in run.stderr
