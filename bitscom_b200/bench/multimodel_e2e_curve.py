"""Convergence and throughput of three small models trained data-parallel with low-bit
gradient all-reduce: ResNet-50 on prototype images, a 4-layer BERT classifier with a label
cue in token 0, and a 4-layer GPT-2 on arithmetic-progression sequences.

One program covers what the reference spreads over three scripts:

* rounding arms ``lowbit_no_sr`` / ``lowbit_sr`` / ``no_compression`` of
  ``benchmarks/multimodel_stochastic_e2e_curve.py`` (``--arms``);
* the error-feedback sweep ``none / legacy / ef21 / ef21_plus`` of
  ``benchmarks/multimodel_error_feedback_e2e_curve.py`` (``--ef-modes``; each mode is a
  nearest-rounding arm named ``ef_<mode>``);
* the table and combined curves of ``benchmarks/error_feedback_multimodel_summary.py``
  (``--summary`` reads the CSV files an earlier run left in ``--out-dir``).

Training recipe as in the reference (``multimodel_stochastic_e2e_curve.py:247-402``):
AdamW, linear warm-up then cosine decay to ``min_lr_ratio``, gradient clipping, gradients
concatenated into flat buckets of ``--grad-bucket-numel`` elements, one
``LowBitGroup.all_reduce`` per bucket, division by the world size, scatter back.  The
"no compression" arm is an 8-bit group, which is a dense all-reduce.  Differences: the
models are this package's own small implementations (no torchvision / transformers
download), error feedback works together with stochastic rounding, and with
``--profile-trace`` rank 0 exports a Chrome trace of the first ``--profile-steps`` steps
for ``bench.trace_stable_window``.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m bitscom_b200.bench.multimodel_e2e_curve --device cpu --models bert gpt2
"""

from __future__ import annotations

import argparse
import csv
import glob
import json
import math
import os
import time
from contextlib import nullcontext
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..api import LowBitGroup

MODELS = ("resnet50", "bert", "gpt2")
EF_FLAGS = {  # mode -> (stage 1, stage 2); "legacy" and "ef21" behave identically
    "none": (False, False), "legacy": (True, False), "ef21": (True, False),
    "ef21_plus": (True, True), "ef21+": (True, True),
}


# ----------------------------------------------------------------------------- data
def dataset_resnet50(rank: int, size: int, image: int, classes: int, seed: int):
    """Low-frequency class prototypes plus a little noise: an easy visual task."""
    g = torch.Generator().manual_seed(seed + rank * 10_000)
    coarse = torch.randn(classes, 3, 12, 12, generator=g) * 0.6
    proto = F.interpolate(coarse, size=(image, image), mode="bilinear", align_corners=False)
    y = torch.randint(0, classes, (size,), generator=g)
    x = proto[y] + torch.randn(size, 3, image, image, generator=g) * 0.01
    return {"x": x, "y": y}


def dataset_bert(rank: int, size: int, seq: int, labels: int, seed: int, vocab: int = 30522):
    """Random tokens; token 0 carries the label (offset 101), so the task is learnable."""
    g = torch.Generator().manual_seed(seed + rank * 20_000)
    ids = torch.randint(0, vocab, (size, seq), generator=g)
    y = torch.randint(0, labels, (size,), generator=g)
    ids[:, 0] = y + 101
    return {"ids": ids, "y": y}


def dataset_gpt2(rank: int, size: int, seq: int, seed: int, base_vocab: int = 512):
    """Arithmetic progressions modulo 512: next-token prediction is deterministic."""
    g = torch.Generator().manual_seed(seed + rank * 30_000)
    start = torch.randint(0, base_vocab, (size, 1), generator=g)
    return {"ids": (start + torch.arange(seq).unsqueeze(0)) % base_vocab}


def slice_batch(data: Dict[str, torch.Tensor], step: int, batch: int) -> Dict[str, torch.Tensor]:
    """Batch ``step`` (1-based) of a dataset walked in order, wrapping at the end."""
    n = next(iter(data.values())).shape[0]
    idx = (torch.arange(batch) + ((step - 1) * batch) % n) % n
    return {k: v[idx] for k, v in data.items()}


# ---------------------------------------------------------------------------- models
def build_model(name: str, args) -> torch.nn.Module:
    if name == "resnet50":
        from ..models.resnet import ResNet50
        return ResNet50(num_classes=args.resnet_num_classes, depths=tuple(args.resnet_depths),
                        base_width=args.resnet_width)
    from ..models.small_transformers import BertClassifier, GPT2LM
    if name == "bert":
        return BertClassifier(hidden=args.bert_hidden, layers=args.bert_layers,
                              heads=args.bert_heads, num_labels=args.bert_num_labels)
    if name == "gpt2":
        return GPT2LM(hidden=args.gpt2_hidden, layers=args.gpt2_layers, heads=args.gpt2_heads)
    raise ValueError(f"unsupported model: {name}")


def build_dataset(name: str, rank: int, cfg: Dict[str, float], args):
    n = int(cfg["dataset_size"])
    if name == "resnet50":
        return dataset_resnet50(rank, n, args.resnet_image_size, args.resnet_num_classes,
                                args.data_seed)
    if name == "bert":
        return dataset_bert(rank, n, args.bert_seq_len, args.bert_num_labels, args.data_seed)
    return dataset_gpt2(rank, n, args.gpt2_seq_len, args.data_seed)


def model_loss(name: str, model, batch) -> torch.Tensor:
    if name == "resnet50":
        return F.cross_entropy(model(batch["x"]), batch["y"])
    if name == "bert":
        return model(batch["ids"], batch["y"])
    return model(batch["ids"], batch["ids"])


def train_cfg(name: str, args) -> Dict[str, float]:
    """Per-family settings: the NLP models take more, smaller steps than ResNet."""
    pre = "nlp" if name in ("bert", "gpt2") else "resnet"

    def pick(field: str, default):
        v = getattr(args, f"{pre}_{field}")
        return default if v is None else v

    return {"steps": int(pick("steps", args.steps)),
            "batch_size": int(pick("batch_size", args.batch_size)),
            "dataset_size": int(pick("dataset_size", args.dataset_size)),
            "grad_clip_norm": float(pick("grad_clip_norm", args.grad_clip_norm)),
            "warmup_ratio": float(pick("warmup_ratio", args.warmup_ratio)),
            "min_lr_ratio": float(pick("min_lr_ratio", args.min_lr_ratio))}


def model_lr(name: str, arm: str, args) -> float:
    if name == "resnet50":
        return args.lr_resnet_sr if arm == "lowbit_sr" else args.lr_resnet
    return args.lr_bert if name == "bert" else args.lr_gpt2


# ------------------------------------------------------------------------ grad sync
def sync_grads_bucketed(grads: List[torch.Tensor], group: LowBitGroup, world: int,
                        bucket_numel: int) -> int:
    """All-reduce ``grads`` in flat buckets of at most ``bucket_numel`` elements (a tensor
    larger than that is a bucket of its own); returns the number of buckets."""
    bucket: List[torch.Tensor] = []
    filled, count = 0, 0

    def flush():
        nonlocal bucket, filled, count
        if not bucket:
            return
        flat = torch.cat([g.reshape(-1) for g in bucket])
        group.all_reduce(flat, ef_key=("bucket", count))
        flat.div_(world)
        off = 0
        for g in bucket:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
        bucket, filled = [], 0
        count += 1

    for g in grads:
        if bucket and filled + g.numel() > bucket_numel:
            flush()
        bucket.append(g)
        filled += g.numel()
    flush()
    return count


def make_group(arm: str, args) -> LowBitGroup:
    if arm == "no_compression":
        return LowBitGroup(bitwidth=8)
    if arm in ("lowbit_no_sr", "lowbit_sr"):
        s1, s2 = EF_FLAGS[args.ef_mode]
        sr = arm == "lowbit_sr"
    elif arm.startswith("ef_"):
        s1, s2 = EF_FLAGS[arm[3:]]
        sr = False
    else:
        raise ValueError(f"unknown arm: {arm}")
    return LowBitGroup(bitwidth=args.bitwidth, stochastic_rounding=sr, error_feedback=s1,
                       stage2_error_feedback=s2, sr_seed=args.seed if sr else None)


def lr_factor(step: int, total: int, warmup_ratio: float, min_ratio: float) -> float:
    warm = max(1, int(total * warmup_ratio))
    if step < warm:
        return (step + 1) / warm
    progress = (step - warm) / max(1, total - warm)
    return min_ratio + (1.0 - min_ratio) * 0.5 * (1.0 + math.cos(math.pi * progress))


# ---------------------------------------------------------------------------- train
def run_train(name: str, arm: str, args, rank: int, world: int, device) -> Dict[str, object]:
    cfg = train_cfg(name, args)
    torch.manual_seed(args.seed)
    model = build_model(name, args).to(device).train()
    data = build_dataset(name, rank, cfg, args)
    group = make_group(arm, args)
    opt = torch.optim.AdamW(model.parameters(), lr=model_lr(name, arm, args),
                            betas=(0.9, 0.999), eps=1e-8, weight_decay=args.weight_decay)
    steps, batch = cfg["steps"], cfg["batch_size"]
    sched = torch.optim.lr_scheduler.LambdaLR(
        opt, lambda s: lr_factor(s, steps, cfg["warmup_ratio"], cfg["min_lr_ratio"]))
    cuda = device.type == "cuda"
    profile = (args.profile_trace and rank == 0 and name == args.profile_model
               and arm in args.profile_arms and args.profile_steps > 0)
    ctx = nullcontext()
    if profile:
        acts = [torch.profiler.ProfilerActivity.CPU]
        if cuda:
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        os.makedirs(args.out_dir, exist_ok=True)
        trace_path = os.path.join(args.out_dir, f"trace_{name}_{arm}_bw{args.bitwidth}.json")
        # a schedule makes the profiler emit one "ProfilerStep#k" range per step, which is
        # what the stable-window analyser cuts on
        ctx = torch.profiler.profile(
            activities=acts, record_shapes=True,
            schedule=torch.profiler.schedule(wait=0, warmup=0,
                                             active=min(steps, args.profile_steps), repeat=1),
            on_trace_ready=lambda p: p.export_chrome_trace(trace_path))
    losses: List[float] = []
    elapsed = 0.0
    with ctx as prof:
        for step in range(1, steps + 1):
            if cuda:
                torch.cuda.synchronize(device)
            t0 = time.perf_counter()
            b = {k: v.to(device, non_blocking=True)
                 for k, v in slice_batch(data, step, batch).items()}
            opt.zero_grad(set_to_none=True)
            loss = model_loss(name, model, b)
            loss.backward()
            grads = [p.grad for p in model.parameters() if p.grad is not None]
            if args.grad_bucket_numel > 0 and not args.disable_grad_bucket:
                sync_grads_bucketed(grads, group, world, args.grad_bucket_numel)
            else:
                for i, g in enumerate(grads):
                    group.all_reduce(g, ef_key=("param", i))
                    g.div_(world)
            if cfg["grad_clip_norm"] > 0:
                torch.nn.utils.clip_grad_norm_(model.parameters(), cfg["grad_clip_norm"])
            opt.step()
            sched.step()
            t = loss.detach().float().view(1)
            dist.all_reduce(t)
            losses.append(float(t.item()) / world)  # .item() also drains the device
            elapsed += time.perf_counter() - t0
            if profile and step <= args.profile_steps:
                prof.step()
    if profile:
        print(f"saved trace: {trace_path}")
    safe = max(elapsed, 1e-9)
    return {"losses": losses, "avg_step_time_ms": safe / max(len(losses), 1) * 1e3,
            "throughput_samples_per_s": batch * len(losses) * world / safe}


def moving_average(values: List[float], window: int) -> List[float]:
    out, run = [], 0.0
    for i, v in enumerate(values):
        run += v
        if i >= window:
            run -= values[i - window]
        out.append(run / min(i + 1, max(window, 1)))
    return out if window > 1 else list(values)


# ---------------------------------------------------------------------------- output
def save_outputs(out_dir: str, name: str, bitwidth: int, window: int,
                 runs: Dict[str, Dict[str, object]]) -> Tuple[str, str]:
    os.makedirs(out_dir, exist_ok=True)
    arms = list(runs)
    curve = os.path.join(out_dir, f"{name}_loss_curve_bw{bitwidth}.csv")
    with open(curve, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["step"] + [f"loss_{a}" for a in arms] + [f"ma{window}_{a}" for a in arms])
        smooth = {a: moving_average(runs[a]["losses"], window) for a in arms}
        for i in range(max(len(runs[a]["losses"]) for a in arms)):
            row = [i + 1]
            row += [runs[a]["losses"][i] if i < len(runs[a]["losses"]) else "" for a in arms]
            row += [smooth[a][i] if i < len(smooth[a]) else "" for a in arms]
            w.writerow(row)
    from ..utils.plot import save_line_plot

    save_line_plot(curve[:-4] + ".png",
                   {a: (list(range(1, len(smooth[a]) + 1)), smooth[a]) for a in arms},
                   title=f"{name} loss (moving average {window}), {bitwidth}-bit",
                   xlabel="step", ylabel="loss")
    thr = os.path.join(out_dir, f"{name}_throughput_bw{bitwidth}.csv")
    with open(thr, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["model", "arm", "avg_step_time_ms", "throughput_samples_per_s",
                    "final_loss", "mean_last10_loss"])
        for a in arms:
            ls = runs[a]["losses"]
            w.writerow([name, a, runs[a]["avg_step_time_ms"],
                        runs[a]["throughput_samples_per_s"], ls[-1],
                        sum(ls[-10:]) / len(ls[-10:])])
    return curve, thr


def summarize(out_dir: str, bitwidth: int) -> Dict[str, List[Dict[str, object]]]:
    """Collect every ``*_throughput_bw<b>.csv`` in ``out_dir`` into one table (written to
    ``summary_bw<b>.csv`` and returned)."""
    rows: List[Dict[str, object]] = []
    for path in sorted(glob.glob(os.path.join(out_dir, f"*_throughput_bw{bitwidth}.csv"))):
        with open(path, newline="") as f:
            rows += list(csv.DictReader(f))
    by_model: Dict[str, List[Dict[str, object]]] = {}
    for r in rows:
        by_model.setdefault(r["model"], []).append(r)
    for model_rows in by_model.values():
        base = next((r for r in model_rows if r["arm"] == "no_compression"), None)
        for r in model_rows:
            r["throughput_vs_no_compression"] = (
                float(r["throughput_samples_per_s"]) / float(base["throughput_samples_per_s"])
                if base else "")
            r["final_loss_minus_no_compression"] = (
                float(r["final_loss"]) - float(base["final_loss"]) if base else "")
    if rows:
        with open(os.path.join(out_dir, f"summary_bw{bitwidth}.csv"), "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
            w.writeheader()
            w.writerows(rows)
    return by_model


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--models", nargs="+", default=list(MODELS), choices=MODELS)
    ap.add_argument("--arms", nargs="+", default=["lowbit_no_sr", "lowbit_sr", "no_compression"])
    ap.add_argument("--ef-mode", default="none", choices=sorted(EF_FLAGS),
                    help="error feedback used by the lowbit_no_sr / lowbit_sr arms")
    ap.add_argument("--ef-modes", nargs="*", default=[], choices=sorted(EF_FLAGS),
                    help="additional nearest-rounding arms, one per error-feedback mode")
    ap.add_argument("--bitwidth", type=int, default=4)
    ap.add_argument("--steps", type=int, default=80)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--dataset-size", type=int, default=512)
    ap.add_argument("--grad-clip-norm", type=float, default=1.0)
    ap.add_argument("--warmup-ratio", type=float, default=0.1)
    ap.add_argument("--min-lr-ratio", type=float, default=0.1)
    for pre, d in (("resnet", dict(steps=None, batch_size=16, dataset_size=None,
                                   grad_clip_norm=None, warmup_ratio=None, min_lr_ratio=None)),
                   ("nlp", dict(steps=160, batch_size=4, dataset_size=1024, grad_clip_norm=0.8,
                                warmup_ratio=0.08, min_lr_ratio=0.05))):
        for field, default in d.items():
            kind = int if field in ("steps", "batch_size", "dataset_size") else float
            ap.add_argument(f"--{pre}-{field.replace('_', '-')}", type=kind, default=default)
    ap.add_argument("--lr-resnet", type=float, default=2e-4)
    ap.add_argument("--lr-resnet-sr", type=float, default=1.5e-4)
    ap.add_argument("--lr-bert", type=float, default=2.5e-4)
    ap.add_argument("--lr-gpt2", type=float, default=2e-4)
    ap.add_argument("--weight-decay", type=float, default=1e-2)
    ap.add_argument("--seed", type=int, default=2026)
    ap.add_argument("--data-seed", type=int, default=17)
    ap.add_argument("--grad-bucket-numel", type=int, default=4_000_000)
    ap.add_argument("--disable-grad-bucket", action="store_true")
    ap.add_argument("--smooth-window", type=int, default=4)
    ap.add_argument("--profile-trace", action="store_true")
    ap.add_argument("--profile-model", default="resnet50", choices=MODELS)
    ap.add_argument("--profile-arms", nargs="+",
                    default=["lowbit_no_sr", "lowbit_sr", "no_compression"])
    ap.add_argument("--profile-steps", type=int, default=4)
    ap.add_argument("--out-dir", default="bench_outputs")
    ap.add_argument("--resnet-image-size", type=int, default=224)
    ap.add_argument("--resnet-num-classes", type=int, default=20)
    ap.add_argument("--resnet-depths", type=int, nargs=4, default=[3, 4, 6, 3])
    ap.add_argument("--resnet-width", type=int, default=64)
    ap.add_argument("--bert-seq-len", type=int, default=64)
    ap.add_argument("--bert-hidden", type=int, default=256)
    ap.add_argument("--bert-layers", type=int, default=4)
    ap.add_argument("--bert-heads", type=int, default=4)
    ap.add_argument("--bert-num-labels", type=int, default=2)
    ap.add_argument("--gpt2-seq-len", type=int, default=64)
    ap.add_argument("--gpt2-hidden", type=int, default=256)
    ap.add_argument("--gpt2-layers", type=int, default=4)
    ap.add_argument("--gpt2-heads", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--summary", action="store_true",
                    help="only combine the CSV files already in --out-dir")
    return ap


def main(argv=None):
    args = parser().parse_args(argv)
    if args.summary:
        table = summarize(args.out_dir, args.bitwidth)
        print(json.dumps({m: [{k: r[k] for k in ("arm", "final_loss", "throughput_samples_per_s",
                                                 "throughput_vs_no_compression")}
                              for r in rows] for m, rows in table.items()}))
        return
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if args.device == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    world = dist.get_world_size()
    arms = list(args.arms) + [f"ef_{m.replace('+', '_plus')}" for m in args.ef_modes]
    for name in args.models:
        runs = {}
        for arm in arms:
            runs[arm] = run_train(name, arm, args, rank, world, device)
            if rank == 0:
                r = runs[arm]
                print(json.dumps({"model": name, "arm": arm, "bitwidth": args.bitwidth,
                                  "world": world, "device": args.device,
                                  "steps": len(r["losses"]), "first_loss": r["losses"][0],
                                  "final_loss": r["losses"][-1],
                                  "avg_step_time_ms": r["avg_step_time_ms"],
                                  "throughput_samples_per_s": r["throughput_samples_per_s"]}))
        if rank == 0:
            save_outputs(args.out_dir, name, args.bitwidth, args.smooth_window, runs)
    if rank == 0:
        summarize(args.out_dir, args.bitwidth)
    dist.barrier()
    import bitscom_b200

    bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
