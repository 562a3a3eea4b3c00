"""The restart-based launcher (bitscom_b200/launch.py) with the elastic training example on CPU
ranks: a rank disappears at a given step (made on the host: the process exits), the others
stop between steps, the launcher starts a new generation without it, and training resumes
from the checkpoints and finishes."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(tmp_path, launcher_args, worker_args, timeout=600):
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "bitscom_b200.launch"] + launcher_args + [
        "--", sys.executable, os.path.join(ROOT, "examples", "elastic_training.py"),
        "--ckpt", str(tmp_path / "ckpt")] + worker_args
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=timeout)


def _rows(text):
    out = []
    for line in text.replace("}{", "}\n{").splitlines():   # ranks share one pipe
        line = line.strip()
        if line.startswith("{"):
            try:
                out.append(json.loads(line))
            except ValueError:
                pass
    return out


def test_job_without_failures_runs_one_generation(tmp_path):
    run = _launch(tmp_path, ["--nproc", "2"], ["--steps", "4"])
    assert run.returncode == 0, run.stderr[-3000:]
    done = [r for r in _rows(run.stdout) if r.get("finished")]
    assert done == [dict(done[0], generation=0, world=2, resumed_at=0, steps=4)]
    events = [r["launch"] for r in _rows(run.stderr) if "launch" in r]
    assert events == ["generation started", "finished"]


def test_lost_rank_leads_to_a_smaller_generation_that_resumes(tmp_path):
    run = _launch(tmp_path, ["--nproc", "3", "--min-nproc", "2", "--shrink", "--max-restarts",
                             "2", "--grace", "40"],
                  ["--steps", "10", "--fail-rank", "2", "--fail-step", "4"])
    assert run.returncode == 0, (run.stdout[-2000:], run.stderr[-3000:])
    rows = _rows(run.stdout)
    done = [r for r in rows if r.get("finished")]
    assert len(done) == 1
    assert done[0]["generation"] == 1 and done[0]["world"] == 2
    assert done[0]["resumed_at"] == 4 and done[0]["steps"] == 10
    stopped = [r for r in rows if "stopped" in r]
    assert {r["rank"] for r in stopped} == {0, 1} and all(r["generation"] == 0 for r in stopped)
    events = [r for r in _rows(run.stderr) if "launch" in r]
    failed = [r for r in events if r["launch"] == "generation failed"]
    assert len(failed) == 1 and failed[0]["lost"] == [2]
    assert failed[0]["exit_codes"] == {"0": 3, "1": 3, "2": 17}
    assert [r["world"] for r in events if r["launch"] == "generation started"] == [3, 2]


def test_restarts_are_bounded(tmp_path):
    # the failing rank is rank 1 of a two-rank job that may not shrink: generation 1 succeeds
    # only because the example fails in generation 0 alone; with no restarts allowed the
    # launcher gives up
    run = _launch(tmp_path, ["--nproc", "2", "--max-restarts", "0", "--grace", "40"],
                  ["--steps", "6", "--fail-rank", "1", "--fail-step", "2"])
    assert run.returncode == 1
    events = [r["launch"] for r in _rows(run.stderr) if "launch" in r]
    assert events == ["generation started", "generation failed"]


def test_llama_trainer_recovers_under_the_launcher(tmp_path):
    """The headline trainer itself (tiny model, CPU ranks): rank 1 disappears before step 3
    (host-side injection), rank 0's collective fails, the heartbeat monitor names the lost
    peer, rank 0 stops with exit code 3, the launcher restarts both ranks, and they resume from
    the periodic checkpoints at step 3 and finish step 5."""
    ckpt = str(tmp_path / "ckpt")
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1",
               BITSCOM_INJECT_EXIT="1:3")
    cmd = [sys.executable, "-m", "bitscom_b200.launch", "--nproc", "2", "--max-restarts", "1",
           "--grace", "40", "--", sys.executable, "-m", "bitscom_b200.trainer.llama_dp_pp",
           "--pg_timeout", "10",
           "--device", "cpu", "--model", "tiny", "--seq_length", "64", "--micro_batches", "2",
           "--batch_size", "2", "--max_steps", "6", "--lr", "1e-3", "--health_check",
           "--health_timeout", "3", "--output_dir", ckpt, "--resume", ckpt, "--save_every", "1"]
    run = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, (run.stdout[-2000:], run.stderr[-3000:])
    rows = _rows(run.stdout)
    steps = sorted(r["step"] for r in rows if "step_s" in r)
    assert steps == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5]      # each step once per rank, no repeats
    stopped = [r for r in rows if "stopped" in r]
    assert len(stopped) == 1 and stopped[0]["step"] == 3 and "rank 1" in stopped[0]["stopped"]
    events = [r for r in _rows(run.stderr) if "launch" in r]
    failed = [r for r in events if r["launch"] == "generation failed"]
    assert len(failed) == 1 and failed[0]["exit_codes"] == {"0": 3, "1": 17}
    assert failed[0]["lost"] == [1]
    assert events[-1]["launch"] == "finished" and events[-1]["generation"] == 1
