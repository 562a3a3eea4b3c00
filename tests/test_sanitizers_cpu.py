"""The C++ CPU codec under AddressSanitizer + UndefinedBehaviorSanitizer, and its thread
fan-out under ThreadSanitizer.  (The GPU kernels cannot be run under compute-sanitizer here;
the host runtime can be, and is, checked with the compiler's sanitizers.)"""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "bitscom_b200", "csrc", "cpu_codec.cc")
DRIVER = os.path.join(ROOT, "tests", "native", "cpu_codec_sanitize.cc")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _build_and_run(tmp_path, flags, env=None):
    exe = str(tmp_path / "codec_sanitize")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread", "-ffp-contract=off"] + flags + \
          [SRC, DRIVER, "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=900,
                         env=dict(os.environ, **(env or {})))
    assert run.returncode == 0, (run.stdout[-1000:], run.stderr[-4000:])
    assert run.stdout.startswith("ok ")


def test_cpu_codec_under_asan_and_ubsan(tmp_path):
    _build_and_run(tmp_path, ["-fsanitize=address,undefined", "-fno-sanitize-recover=all"],
                   env={"ASAN_OPTIONS": "detect_leaks=1"})


def test_cpu_codec_threads_under_tsan(tmp_path):
    _build_and_run(tmp_path, ["-fsanitize=thread", "-DBCOM_NO_CLONES"])
