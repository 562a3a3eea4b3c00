"""The benchmark programs that run without a GPU: trace analyser, multi-model convergence
bench, collective comparison and the quantize latency curve (host columns)."""

import csv
import json
import os
import subprocess
import sys

import pytest
import torch

from bitscom_b200.bench import multimodel_e2e_curve as MM
from bitscom_b200.bench import quantize_perf_curve as QC
from bitscom_b200.bench import trace_stable_window as TW

def _assert_png(path):
    """Every bench CSV has a plot beside it (the reference writes one with matplotlib)."""
    with open(path, "rb") as f:
        head = f.read(8)
    assert head == b"\x89PNG\r\n\x1a\n", path


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port(hint):
    """A port nobody listens on right now (``hint`` is only used if the probe fails)."""
    import socket

    try:
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]
    except OSError:
        return hint


def _torchrun(module, args, port, nproc=2, timeout=600):
    port = _free_port(port)
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", module] + args
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    return [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]


# ------------------------------------------------------------------ trace analyser
def _trace(tmp_path, with_steps=True):
    ev = []
    if with_steps:
        for k in range(6):
            ev.append({"ph": "X", "name": f"ProfilerStep#{k}", "ts": 1000 * k, "dur": 1000})
    for k in range(6):
        base = 1000 * k
        ev.append({"ph": "X", "name": "aten::mm", "ts": base + 10, "dur": 300, "cat": "cpu_op"})
        ev.append({"ph": "X", "name": "nccl:all_reduce", "ts": base + 400, "dur": 100,
                   "cat": "user_annotation"})
        ev.append({"ph": "X", "name": "lowbit_collective_kernel<float, 4>", "ts": base + 500,
                   "dur": 50, "cat": "kernel"})
        ev.append({"ph": "X", "name": "gemm_kernel", "ts": base + 600, "dur": 150,
                   "cat": "kernel"})
        ev.append({"ph": "i", "name": "marker", "ts": base + 5})
    ev.append({"ph": "X", "name": "straddles", "ts": 2900, "dur": 300})  # crosses a boundary
    path = tmp_path / "trace.json"
    path.write_text(json.dumps({"traceEvents": ev}))
    return str(path)


def test_trace_window_by_profiler_steps(tmp_path):
    r = TW.analyze(_trace(tmp_path), skip_steps=3, keep_steps=2, topk=3)
    assert r["profiler_steps"] == 6 and r["window_by"] == "profiler_steps"
    assert r["window_us"] == [3000.0, 5000.0]
    assert r["events"] == 8                       # 2 steps x 4 ops, step ranges left out
    assert r["total_op_ms"] == pytest.approx(2 * 0.6)
    assert r["comm_op_ms"] == pytest.approx(2 * 0.15)
    assert r["device_comm_share"] == pytest.approx(50 / 200)
    assert r["top"][0]["name"] == "aten::mm" and r["top"][0]["count"] == 2
    with pytest.raises(RuntimeError):
        TW.analyze(_trace(tmp_path), skip_steps=6)
    all_rest = TW.analyze(_trace(tmp_path), skip_steps=3, keep_steps=0)
    assert all_rest["window_us"] == [3000.0, 6000.0] and all_rest["events"] == 12


def test_trace_window_falls_back_to_time_ratio(tmp_path, capsys):
    path = _trace(tmp_path, with_steps=False)
    r = TW.main(["--trace", path, "--fallback-skip-ratio", "0.5"])
    assert r["window_by"] == "time_ratio" and r["profiler_steps"] == 0
    first, last = 10.0, 5750.0
    assert r["window_us"][0] == pytest.approx(first + 0.5 * (last - first))
    assert "no ProfilerStep found" in capsys.readouterr().out


# ------------------------------------------------------------- multi-model helpers
def test_slice_batch_wraps_and_lr_schedule():
    data = {"a": torch.arange(10)}
    assert MM.slice_batch(data, 1, 4)["a"].tolist() == [0, 1, 2, 3]
    assert MM.slice_batch(data, 3, 4)["a"].tolist() == [8, 9, 0, 1]
    f = [MM.lr_factor(s, 100, 0.1, 0.1) for s in range(100)]
    assert f[0] == pytest.approx(0.1) and f[9] == pytest.approx(1.0)
    assert f[10] == pytest.approx(1.0) and f[99] < 0.11 and min(f[10:]) >= 0.1
    assert all(a >= b for a, b in zip(f[10:], f[11:]))


class _FakeGroup:
    def __init__(self):
        self.calls = []

    def all_reduce(self, flat, ef_key=None):
        self.calls.append((flat.numel(), ef_key))
        flat.mul_(2)  # as if two ranks held the same gradient


def test_bucketed_sync_groups_and_scatters_back():
    grads = [torch.full((n,), float(i + 1)) for i, n in enumerate((3, 4, 10, 2, 2))]
    g = _FakeGroup()
    n = MM.sync_grads_bucketed(grads, g, world=2, bucket_numel=8)
    assert n == 3 and [c[0] for c in g.calls] == [7, 10, 4]
    assert [c[1] for c in g.calls] == [("bucket", 0), ("bucket", 1), ("bucket", 2)]
    for i, t in enumerate(grads):
        assert torch.equal(t, torch.full_like(t, float(i + 1)))


def test_ef_mode_mapping():
    ap = MM.parser()
    args = ap.parse_args(["--ef-mode", "ef21_plus"])
    assert MM.EF_FLAGS["legacy"] == MM.EF_FLAGS["ef21"] == (True, False)
    assert MM.EF_FLAGS[args.ef_mode] == (True, True)
    with pytest.raises(ValueError):
        MM.make_group("bogus", args)


def test_multimodel_bench_two_cpu_ranks(tmp_path):
    out = str(tmp_path / "mm")
    recs = _torchrun("bitscom_b200.bench.multimodel_e2e_curve",
                     ["--device", "cpu", "--models", "bert", "resnet50", "--nlp-steps", "6",
                      "--steps", "3", "--bert-hidden", "32", "--bert-layers", "1",
                      "--bert-heads", "2", "--bert-seq-len", "8", "--resnet-image-size", "32",
                      "--resnet-depths", "1", "1", "1", "1", "--resnet-width", "8",
                      "--resnet-batch-size", "4", "--arms", "lowbit_sr", "no_compression",
                      "--ef-modes", "ef21_plus", "--out-dir", out, "--profile-trace",
                      "--profile-model", "bert", "--profile-arms", "lowbit_sr",
                      "--profile-steps", "4"], port=29641)
    arms = {(r["model"], r["arm"]) for r in recs}
    assert arms == {(m, a) for m in ("bert", "resnet50")
                    for a in ("lowbit_sr", "no_compression", "ef_ef21_plus")}
    assert all(r["final_loss"] == r["final_loss"] and r["throughput_samples_per_s"] > 0
               for r in recs)
    _assert_png(os.path.join(out, "bert_loss_curve_bw4.png"))
    with open(os.path.join(out, "bert_loss_curve_bw4.csv")) as f:
        rows = list(csv.reader(f))
    assert rows[0][:4] == ["step", "loss_lowbit_sr", "loss_no_compression", "loss_ef_ef21_plus"]
    assert len(rows) == 7
    table = MM.summarize(out, 4)
    base = next(r for r in table["bert"] if r["arm"] == "no_compression")
    assert base["throughput_vs_no_compression"] == pytest.approx(1.0)
    trace = os.path.join(out, "trace_bert_lowbit_sr_bw4.json")
    r = TW.analyze(trace, skip_steps=1)
    assert r["profiler_steps"] == 4 and r["comm_op_ms"] > 0


@pytest.mark.parametrize("kind", ["allreduce", "reduce_scatter", "all_gather"])
def test_collective_compare_two_cpu_ranks(kind, tmp_path):
    port = 29650 + ["allreduce", "reduce_scatter", "all_gather"].index(kind)
    recs = _torchrun("bitscom_b200.bench.collective_compare",
                     ["--collective", kind, "--bitwidths", "2", "4", "--device", "cpu",
                      "--steps", "4", "--numel", "8192", "--out-dir", str(tmp_path)], port=port)
    by_bits = {r["bitwidth"]: r for r in recs}
    assert set(by_bits) == {2, 4}
    assert 0 < by_bits[4]["rel_error_mean"] < by_bits[2]["rel_error_mean"] < 0.5
    assert by_bits[4]["rel_error_mean"] < 0.12
    _assert_png(tmp_path / f"{kind}_compare_bw4.png")
    with open(tmp_path / f"{kind}_compare_bw4.csv") as f:
        rows = list(csv.reader(f))
    assert rows[0] == ["step", "rel_error", "lowbit_ms", "baseline_ms"] and len(rows) == 5


def test_quantize_curve_host_columns(tmp_path):
    rows = QC.main(["--mode", "blockwise", "--min-pow2", "10", "--max-pow2", "12",
                    "--max-iters", "3", "--warmup", "1", "--device", "cpu",
                    "--out-dir", str(tmp_path)])
    assert [r["numel"] for r in rows] == [1024, 2048, 4096]
    assert all(r["cpu_torch_ms"] > 0 for r in rows)
    assert os.path.exists(tmp_path / "quantize_curve_blockwise_bw4.csv")
    _assert_png(tmp_path / "quantize_curve_blockwise_bw4.png")
    rows = QC.main(["--min-pow2", "10", "--max-pow2", "10", "--max-iters", "3", "--warmup", "1",
                    "--device", "cpu"])
    assert "gpu_ms" not in rows[0] and rows[0]["cpu_melems_per_s"] > 0


# ------------------------------------------------------------------------- examples
def _run_example(name, port):
    port = _free_port(port)
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "examples", name)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    return out.stdout


def test_quickstart_example_keeps_the_accumulated_error_small():
    out = _run_example("allreduce_quickstart.py", 29661)
    line = next(l for l in out.splitlines() if "relative error" in l)
    words = line.split()
    with_ef, without = float(words[words.index("feedback") + 1]), float(words[-1])
    assert with_ef < 0.6 * without and without < 0.5


def test_ddp_hook_example_trains():
    out = _run_example("ddp_comm_hook.py", 29662)
    line = next(l for l in out.splitlines() if l.startswith("loss "))
    first, last = (float(v) for v in line[5:].split(" -> "))
    assert last < 0.6 * first


def test_sharded_optimizer_example_trains():
    out = _run_example("sharded_optimizer.py", 29663)
    assert "each of 2 ranks keeps 2304 of 4608 fp32 master weights" in out
    line = next(l for l in out.splitlines() if l.startswith("loss "))
    first, last = (float(v) for v in line[5:].split(" -> "))
    assert last < 0.2 * first


def test_roofline_report_table():
    from bitscom_b200.bench import roofline_report as RR

    lines = [
        json.dumps({"case": "gemm_tcgen05", "M": 4096, "N": 4096, "K": 4096, "ms": 0.11,
                    "tflops": 1250.0, "frac_bf16_peak": 0.76, "peaks": "of measured"}),
        json.dumps({"case": "attention_tcgen05", "batch": 2, "seq": 2048, "heads": 32,
                    "head_dim": 128, "fwd_variant": "pipelined", "bwd_dq": "tma",
                    "fwd_ms": 0.137, "fwd_tflops": 503.0, "fwd_frac_bf16_peak": 0.30,
                    "bwd_ms": 0.673, "bwd_tflops": 255.0, "bwd_frac_bf16_peak": 0.15,
                    "peaks": "of measured"}),
        json.dumps({"case": "elementwise", "tokens": 8192, "peaks": "of fallback", "kernels": [
            {"name": "adamw_flat", "ms": 1.5, "gbs": 6071.0, "frac_hbm": 0.93}]}),
        json.dumps({"bytes": 1 << 30, "dtype": "fp32", "world": 8, "bits": 4, "lowbit_ms": 1.317,
                    "lowbit_fp32eq_gbs": 815.0, "roofline_frac": 0.59, "peaks": "measured"}),
        "not json", json.dumps({"something": "else"}),
    ]
    rows = RR.collect(lines)
    assert [r["kernel"] for r in rows] == [
        "gemm_tcgen05", "attention_tcgen05 fwd (pipelined)", "attention_tcgen05 bwd (dQ tma)",
        "adamw_flat", "low-bit all-reduce 4-bit"]
    table = RR.to_markdown(rows)
    assert "| gemm_tcgen05 | 4096 x 4096 x 4096 | 0.110 ms | 1250 TFLOP/s | 0.76 |" in table
    assert "8 GPUs, 1024 MB fp32" in table and "HBM copy, of fallback" in table


def test_resnet18_ddp_trainer_on_cpu_ranks(tmp_path):
    """Config-3 program end to end on CPU ranks: torch DDP buckets through the low-bit
    communication hook (2-bit + error feedback), loss reported, output row written."""
    out = str(tmp_path / "resnet.jsonl")
    recs = _torchrun("bitscom_b200.trainer.resnet18_ddp",
                     ["--device", "cpu", "--steps", "3", "--warmup", "1", "--batch", "8",
                      "--bucket-mb", "4", "--out", out], port=29663, timeout=900)
    row = recs[-1]
    assert row["workload"] == "resnet18_cifar_ddp" and row["world"] == 2 and row["bitwidth"] == 2
    assert row["loss_last"] == row["loss_last"] and row["samples_per_s"] > 0
    assert os.path.exists(out)


# ------------------------------------------------------------------ error-feedback benefit
def test_error_feedback_benefit_and_training_curves(tmp_path, capsys):
    """Both halves of the error-feedback comparison: the accumulated-error curve (error feedback
    must win by an order of magnitude at 4 bit) and the small MLP trained through the quantizer
    with and without residuals (same start, both learn, 8-bit runs indistinguishable); a CSV
    and a PNG per curve."""
    from bitscom_b200.bench import error_feedback_benefit as EF

    EF.main(["--bits", "4", "8", "--steps", "40", "--vec-size", "32768", "--train-steps", "60",
             "--out-dir", str(tmp_path)])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    curve4 = next(r for r in lines if r["bitwidth"] == 4 and "ef_rel_error" in r)
    assert curve4["ef_rel_error"] < curve4["no_ef_rel_error"] / 3
    for bits in (4, 8):
        run = next(r for r in lines if r["bitwidth"] == bits and "train_steps" in r)
        assert run["loss_no_ef_first"] == run["loss_ef_first"] > 1.5
        assert run["loss_no_ef_last"] < 0.1 and run["loss_ef_last"] < 0.1
        rows = list(csv.reader(open(tmp_path / f"ef_training_curve_bw{bits}.csv")))
        assert rows[0] == ["step", "loss_noef", "loss_ef"] and len(rows) == 61
        _assert_png(tmp_path / f"ef_training_curve_bw{bits}.png")
        _assert_png(tmp_path / f"ef_comparison_bw{bits}.png")
    run8 = next(r for r in lines if r["bitwidth"] == 8 and "train_steps" in r)
    assert abs(run8["loss_no_ef_last"] - run8["loss_ef_last"]) < 1e-3
    # the curves are deterministic
    a = EF.ef_training_curve(4, steps=5, use_ef=True)
    assert a == EF.ef_training_curve(4, steps=5, use_ef=True)
