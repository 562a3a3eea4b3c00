"""The Llama DP x PP trainer (the headline benchmark's program) on CPU ranks over gloo, tiny
model, through the ops' host paths: own 1F1B schedule across two stages, bucketed low-bit
gradient sync through pipeline-A across two replicas, flat AdamW.  Run as a script this file is
the per-rank worker."""

import functools
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(pp: int, sync: str, steps: int, defer_wgrad: bool = False,
            untied: bool = False, local_size: int = 1, chunks: int = 1) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from bitscom_b200.models.llama import LlamaConfig
    from bitscom_b200.trainer.llama_dp_pp import LlamaTrainer, TrainerConfig

    mcfg = LlamaConfig.tiny(max_seq=64, num_layers=4, tie_embeddings=not untied)
    mcfg.attention = "sdpa"
    tcfg = TrainerConfig(pp_size=pp, micro_batches=4, micro_batch_size=2, seq_length=64,
                         bitwidth=4, error_feedback=True, dp_sync=sync, lr=1e-2, device="cpu",
                         defer_wgrad=defer_wgrad, local_size=local_size, pp_chunks=chunks)
    trainer = LlamaTrainer(mcfg, tcfg)
    losses = []
    for _ in range(steps):
        loss = trainer.train_step(trainer.synthetic_batch(0))  # one batch: the loss must fall
        if loss is not None:
            losses.append(float(loss))
    if losses:
        sys.stdout.write(json.dumps({"rank": trainer.rank, "dp_rank": trainer.dp_rank,
                                     "dp": trainer.dp, "pp": trainer.pp,
                                     "grad_sync": trainer.grad_sync_description(),
                                     "residual_keys": sorted(
                                         repr(k) for k in trainer.lowbit._ef_states)
                                     if trainer.sync is not None else [],
                                     "losses": losses}) + "\n")   # one write: a shared pipe
        sys.stdout.flush()
    if dist.is_initialized():
        dist.barrier()
        import bitscom_b200

        bitscom_b200.shutdown()
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


@functools.lru_cache(maxsize=None)   # the runs are deterministic: tests share them
def _run(nproc: int, pp: int, sync: str, steps: int = 6, defer_wgrad: bool = False,
         untied: bool = False, local_size: int = 1, chunks: int = 1):
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(nproc),
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         os.path.abspath(__file__), str(pp), sync, str(steps), str(int(defer_wgrad)),
         str(int(untied)), str(local_size), str(chunks)],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    text = run.stdout.replace("}{", "}\n{")
    rows = [json.loads(line) for line in text.splitlines() if line.startswith("{")]
    return sorted(rows, key=lambda r: r["rank"])


def test_pipeline_split_computes_what_the_unsplit_model_computes():
    """With an output head of its own (so that both variants are the same network) a model cut
    into two or four pipeline stages follows the unsplit model's loss curve exactly: stages
    exchange the bf16 activations and gradients the unsplit model passes between its layers,
    every parameter starts from the same value whichever stage owns it, and every gradient is
    accumulated in micro-batch order."""
    whole = _run(1, 1, "dense", untied=True)
    two = _run(2, 2, "dense", untied=True)
    four = _run(4, 4, "dense", untied=True)
    assert len(whole) == len(two) == len(four) == 1
    assert whole[0]["losses"][-1] < whole[0]["losses"][0] - 0.5
    assert two[0]["losses"] == whole[0]["losses"]
    assert four[0]["losses"] == whole[0]["losses"]


def test_interleaved_pipeline_computes_what_the_unsplit_model_computes():
    """Two chunks per rank (four virtual stages on two ranks, interleaved 1F1B): the same loss
    curve as the unsplit model, bit for bit, with and without deferred weight gradients; and
    with two replicas the per-chunk gradient buckets keep error-feedback residuals of their
    own."""
    whole = _run(1, 1, "dense", untied=True)
    inter = _run(2, 2, "dense", steps=3, untied=True, chunks=2)
    inter_deferred = _run(2, 2, "dense", steps=3, untied=True, chunks=2, defer_wgrad=True)
    assert inter[0]["losses"] == whole[0]["losses"][:3]
    assert inter_deferred[0]["losses"] == whole[0]["losses"][:3]
    low = _run(4, 2, "flat", steps=4, chunks=2, defer_wgrad=True)
    assert [r["dp_rank"] for r in low] == [0, 1]
    for a in low:
        assert a["losses"][-1] < a["losses"][0] - 0.3
    assert any("chunk" in k for k in low[0]["residual_keys"])


def test_dp2_pp2_behaves_like_dp2_pp1_with_dense_gradient_sync():
    """Two pipeline stages against the unsplit model, two replicas each.  The two are not the
    same network (a split model has an output head of its own on the last stage where the
    unsplit one ties it to the embedding), so the curves are compared loosely: same start, both
    fall, similar end."""
    split = [r for r in _run(4, 2, "dense") if r["dp_rank"] == 0]
    whole = [r for r in _run(2, 1, "dense") if r["dp_rank"] == 0]
    assert len(split) == 1 and split[0]["pp"] == 2 and split[0]["dp"] == 2
    assert len(whole) == 1 and whole[0]["pp"] == 1
    a, b = split[0]["losses"], whole[0]["losses"]
    assert abs(a[0] - b[0]) < 0.02 and abs(a[0] - 6.24) < 0.1     # ln(512) at initialisation
    assert a[-1] < a[0] - 0.5 and b[-1] < b[0] - 0.5
    assert abs(a[-1] - b[-1]) < 0.5, (a, b)


def test_dp2_pp2_trains_with_lowbit_pipeline_a_sync():
    """4-bit gradients with error feedback through the hierarchical pipeline-A path: the loss
    falls as with dense gradients, and both last-stage ranks report (one per replica)."""
    low = _run(4, 2, "pipeline_a")
    dense = _run(4, 2, "dense")
    assert [r["dp_rank"] for r in low] == [0, 1] and all(r["pp"] == 2 for r in low)
    for lo, de in zip(low, dense):
        assert lo["losses"][-1] < lo["losses"][0] - 0.5
        assert abs(lo["losses"][-1] - de["losses"][-1]) < 0.3, (lo["losses"], de["losses"])


_CLI_CACHE = {}


def _cli(tmp_path, port_tag, *extra):
    if "--output_dir" not in extra and "--resume" not in extra and extra in _CLI_CACHE:
        return _CLI_CACHE[extra]
    rows = _cli_run(*extra)
    _CLI_CACHE[extra] = rows
    return rows


def _cli_run(*extra):
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         "-m", "bitscom_b200.trainer.llama_dp_pp", "--device", "cpu", "--model", "tiny",
         "--seq_length", "64", "--micro_batches", "2", "--batch_size", "2", "--lr", "1e-3",
         *extra], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    text = run.stdout.replace("}{", "}\n{")   # two ranks may print on one line
    rows = [json.loads(line) for line in text.splitlines() if line.startswith('{"step"')]
    return sorted((r["step"], r["loss"]) for r in rows)


def test_trainer_cli_resumes_on_the_same_trajectory(tmp_path):
    """Six steps in one go against three steps, a checkpoint (weights, optimizer, residuals of
    the low-bit gradient sync, step counter) and three more steps from it: the same losses to
    the last bit, and the resumed run does not repeat or skip a batch."""
    ckpt = str(tmp_path / "ckpt")
    whole = _cli(tmp_path, 0, "--max_steps", "6")
    first = _cli(tmp_path, 1, "--max_steps", "3", "--output_dir", ckpt)
    _CLI_CACHE[("--max_steps", "3")] = first   # the same run without the checkpoint at its end
    second = _cli(tmp_path, 2, "--max_steps", "6", "--resume", ckpt)
    assert [s for s, _ in whole] == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5]
    assert first + second == whole


def test_stochastic_rounding_is_reproducible_through_the_trainer(tmp_path):
    """The rounding stream is keyed by the trainer's seed and a call counter, not drawn from
    a global generator: two runs give the same losses, and they differ from nearest rounding
    (so the flag does reach the quantizer)."""
    a = _cli(tmp_path, 0, "--max_steps", "3", "--stochastic_rounding")
    b = _cli_run("--max_steps", "3", "--stochastic_rounding")   # a second, real run
    nearest = _cli(tmp_path, 2, "--max_steps", "3")
    assert a == b
    assert a[:2] == nearest[:2] and a != nearest   # step 0 is before the first gradient sync


def test_flat_lowbit_sync_without_pipeline_stages():
    """dp2 x pp1 with the flat low-bit all-reduce per bucket (no hierarchy, no pipeline)."""
    rows = _run(2, 1, "flat")
    assert [r["dp_rank"] for r in rows] == [0, 1]
    assert all(r["losses"][-1] < r["losses"][0] - 0.5 for r in rows)


def test_deferred_weight_gradients_change_nothing_but_the_order_of_work():
    """With ``defer_wgrad`` a stage sends the input gradient before it runs the queued
    weight-gradient GEMMs; every gradient is still accumulated in micro-batch order, so the
    loss curve is the same to the last bit."""
    plain = _run(4, 2, "dense")
    deferred = _run(4, 2, "dense", defer_wgrad=True)
    assert [r["losses"] for r in plain] == [r["losses"] for r in deferred]
    # the same with the low-bit gradient buckets, which are then launched from the queue, each
    # behind the weight-gradient GEMMs of its layer
    low = _run(4, 2, "flat")
    low_deferred = _run(4, 2, "flat", defer_wgrad=True)
    assert [r["losses"] for r in low] == [r["losses"] for r in low_deferred]


def test_dp4_pp2_pipeline_a_with_local_pairs_on_strided_groups():
    """Real two-level pipeline-A through the trainer: data-parallel groups are strided subgroups
    of the (dp, pp) mesh (global ranks 0, 2, 4, 6 and 1, 3, 5, 7), local groups are pairs of
    them and the pairs' first ranks are the leaders.  The leaders' ranks must be translated to
    global ranks for the local reduce / broadcast, the leaders' inter phase keeps error-feedback
    residuals per (bucket, chunk), every replica ends on the same loss curve and it falls."""
    rows = _run(8, 2, "pipeline_a", steps=5, local_size=2)
    assert [r["dp_rank"] for r in rows] == [0, 1, 2, 3] and all(r["pp"] == 2 for r in rows)
    assert all("pipeline-A" in r["grad_sync"] for r in rows)
    # (every replica fits its own batch, four of them share the weights: after five steps the
    # first replica's loss has clearly fallen, and all of them track the dense run below)
    assert rows[0]["losses"][-1] < rows[0]["losses"][0] - 0.4, rows[0]["losses"]
    # leaders (dp ranks 0 and 2) hold residuals keyed by bucket and chunk; the others hold none
    assert any("chunk" in k for k in rows[0]["residual_keys"])
    assert any("chunk" in k for k in rows[2]["residual_keys"])
    assert rows[1]["residual_keys"] == [] and rows[3]["residual_keys"] == []
    dense = _run(8, 2, "dense", steps=5)
    for lo, de in zip(rows, dense):
        assert abs(lo["losses"][-1] - de["losses"][-1]) < 0.3, (lo["losses"], de["losses"])


if __name__ == "__main__":
    _worker(int(sys.argv[1]), sys.argv[2], int(sys.argv[3]), bool(int(sys.argv[4])),
            bool(int(sys.argv[5])), int(sys.argv[6]) if len(sys.argv) > 6 else 1,
            int(sys.argv[7]) if len(sys.argv) > 7 else 1)
