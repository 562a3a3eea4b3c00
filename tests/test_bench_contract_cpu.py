"""The output contract of bench.py, checked on CPU ranks with the tiny model (``--device cpu``):
one JSON line from rank 0 with the keys the benchmark driver reads, whole-job values, and the
reference arm's ``unavailable`` line when the reference cannot run."""

import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
            "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config", "e2e",
            "gpu_launches", "clocks"}


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _bench(nproc, *extra):
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    common = ["bench.py", "--gpus", str(nproc), "--steps", "2", "--warmup", "3", "--device", "cpu",
              "--model", "tiny", "--micro-batches", "2", "--micro-batch-size", "1", *extra]
    if nproc == 1:
        cmd = [sys.executable] + common
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node",
               str(nproc), "--master-addr", "127.0.0.1", "--master-port", str(_free_port())] + common
    run = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    lines = [line for line in run.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, lines      # ONE line, from rank 0 only
    return json.loads(lines[0])


def _check(row, n):
    assert REQUIRED <= set(row), REQUIRED - set(row)
    assert row["n_gpus"] == n and row["steps"] == 2 and row["warmup"] == 3
    assert row["higher_is_better"] is True and row["scaling"] == "weak"
    assert row["unit"] == "tokens/s" and row["dtype"] == "bf16" and "synthetic" in row["data"]
    assert row["value"] > 0 and row["ms_per_step"] > 0
    cfg, e2e = row["config"], row["e2e"]
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(cfg)
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(e2e)
    tokens_per_step = cfg["global_batch"] * cfg["seq_len"]
    # value is the whole job's tokens/s: tokens per step over the measured step time
    assert abs(row["value"] - tokens_per_step / (row["ms_per_step"] / 1e3)) < 1e-6 * row["value"]
    assert e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(row["clocks"])


def test_single_process_line():
    row = _bench(1)
    _check(row, 1)
    assert row["config"]["parallelism"] == "dp1xpp1" and row["config"]["global_batch"] == 2


def test_four_ranks_report_the_whole_job():
    row = _bench(4)
    _check(row, 4)
    assert row["config"]["parallelism"] == "dp2xpp2"
    assert row["config"]["global_batch"] == 2 * 2 * 1    # dp x micro-batches x sequences
    # --local-size 1 (the default) is the flat fused / host low-bit all-reduce, and says so
    assert "flat" in row["config"]["grad_sync"] and "4-bit" in row["config"]["grad_sync"]


def test_reference_arm_reports_unavailable_without_a_gpu():
    run = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0
    row = json.loads([line for line in run.stdout.splitlines() if line.startswith("{")][-1])
    assert row["impl"] == "reference" and isinstance(row.get("unavailable"), str)
