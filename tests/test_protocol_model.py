"""The fused collective's flag / counter protocol as a multi-threaded host model under
ThreadSanitizer (tests/native/protocol_model.cc): back-to-back collectives without any barrier
between ranks, plain-memory slots whose reads must be ordered by the flags alone.  Two seeded
protocol bugs show that the model notices when the ordering is wrong."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "protocol_model.cc")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _build(tmp_path, flags, name):
    exe = str(tmp_path / name)
    out = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread"] + flags + [SRC, "-o", exe],
                         capture_output=True, text=True, timeout=300)
    if out.returncode != 0 and "sanitize" in out.stderr and "cannot find" in out.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert out.returncode == 0, out.stderr[-3000:]
    return exe


def test_protocol_is_race_free_under_tsan(tmp_path):
    exe = _build(tmp_path, ["-fsanitize=thread"], "model_tsan")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1"))
    assert run.returncode == 0, (run.stdout[-500:], run.stderr[-4000:])
    assert run.stdout.startswith("ok:")


@pytest.mark.parametrize("bug", [1, 2])
def test_seeded_protocol_bugs_are_detected(tmp_path, bug):
    """Publishing before re-arming loses arrivals; reading before the phase-2 flags reads
    slots that are still being written.  Either the values or the sanitizer must object."""
    exe = _build(tmp_path, ["-fsanitize=thread", f"-DBUG={bug}"], f"model_bug{bug}")
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1"))
    assert run.returncode != 0, "the seeded bug went unnoticed"
