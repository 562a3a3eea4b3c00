"""The tcgen05 instruction-descriptor encoder (a constexpr host/device function) against the
documented bit layout: D format f32 at bit 4, A / B format bf16 at bits 7 / 10, the
MN-major flags at bits 15 / 16, N >> 3 at bit 17, M >> 4 at bit 24."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _expect(m, n, a_mn, b_mn):
    return (1 << 4) | (1 << 7) | (1 << 10) | (int(a_mn) << 15) | (int(b_mn) << 16) | \
        ((n >> 3) << 17) | ((m >> 4) << 24)


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                    reason="needs nvcc")
def test_instruction_descriptors(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path / "descriptors")
    build = subprocess.run([nvcc, "-std=c++17", "-I", os.path.join(ROOT, "bitscom_b200", "csrc"),
                            "-gencode", "arch=compute_100a,code=sm_100a",
                            os.path.join(ROOT, "tests", "native", "descriptors.cu"), "-o", exe],
                           capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stderr
    got = [int(v) for v in run.stdout.split()]
    assert got == [_expect(128, 256, False, False), _expect(128, 256, True, True),
                   _expect(128, 64, False, False), _expect(128, 128, False, True)]
