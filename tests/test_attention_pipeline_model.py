"""The mbarrier protocol of the software-pipelined attention forward kernels as a host model
(tests/native/attention_pipeline_model.cc): issuer, tensor pipe, copy engine and softmax
warps as threads, parity waits as in the kernels, every buffer tagged with the key block it
holds.  Both kernels' protocols must run clean for 2 to 32 key blocks; two seeded bugs (a
missing wait each) must be noticed.

The backward kernel's query-block loop has a model of its own
(tests/native/attention_bwd_model.cc): the loads of the next Q / dO tiles after the whole
second MMA group or as soon as dV and dK are complete, the dQ staging tile that shares memory
with P^T / dS^T, and the bulk-group wait that protects it; three seeded bugs."""

import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "attention_pipeline_model.cc")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


BWD_SRC = os.path.join(ROOT, "tests", "native", "attention_bwd_model.cc")


def _run(tmp_path, flags, name, src=SRC):
    exe = str(tmp_path / name)
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread"] + flags + [src, "-o", exe],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    return subprocess.run([exe], capture_output=True, text=True, timeout=900)


@pytest.mark.parametrize("warps", [4])
def test_pipeline_protocol_runs_clean(tmp_path, warps):
    run = _run(tmp_path, [f"-DSOFTMAX_WARPS={warps}"], f"model{warps}")
    assert run.returncode == 0, (run.stdout[-300:], run.stderr[-2000:])
    assert run.stdout.startswith(f"ok: {warps} softmax warps")


@pytest.mark.parametrize("bug", [1, 2])
def test_a_missing_wait_is_detected(tmp_path, bug):
    run = _run(tmp_path, ["-DSOFTMAX_WARPS=4", f"-DBUG={bug}"], f"bug{bug}")
    assert run.returncode == 3, "the seeded bug went unnoticed"
    assert "violation:" in run.stderr


@pytest.mark.parametrize("early", [0])
def test_backward_protocol_runs_clean(tmp_path, early):
    run = _run(tmp_path, [f"-DEARLY={early}"], f"bwd{early}", BWD_SRC)
    assert run.returncode == 0, (run.stdout[-300:], run.stderr[-2000:])
    assert run.stdout.startswith(f"ok: early={early}")


@pytest.mark.parametrize("early,bug", [(0, 2), (0, 3)])
def test_backward_missing_wait_is_detected(tmp_path, early, bug):
    run = _run(tmp_path, [f"-DEARLY={early}", f"-DBUG={bug}"], f"bwdbug{early}{bug}", BWD_SRC)
    assert run.returncode == 3, "the seeded bug went unnoticed"
    assert "violation:" in run.stderr
