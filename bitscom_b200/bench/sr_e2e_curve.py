"""End-to-end loss curves of a small MLP trained data-parallel with low-bit gradient
all-reduce: nearest rounding vs stochastic rounding vs no compression (optionally with
error feedback, which the reference's Python path does not have).

Same experiment as the reference's ``benchmarks/stochastic_rounding_e2e_curve.py`` (TinyMLP
256-512-512-10, teacher-labelled synthetic data per rank, SGD momentum 0.9, lr 0.05, batch
128, gradient clipping 1.0, per-parameter ``LowBitGroup.all_reduce`` + ``div_``, 160 steps;
its "no compression" arm is an 8-bit group, i.e. a dense all-reduce).  The reference's
published endpoints at 4-bit, 2 ranks, step 160 are 0.2261 / 0.2393 / 0.2317
(``benchmarks/outputs/e2e_loss_curve_stochastic_vs_nocompress_bw4.csv:161``).

Runs on CPU ranks over gloo or on GPUs over NCCL:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m bitscom_b200.bench.sr_e2e_curve --bitwidth 4 --device cpu
"""

from __future__ import annotations

import argparse
import csv
import json
import os
from typing import List, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..api import LowBitGroup


class TinyMLP(nn.Module):
    def __init__(self, in_dim=256, hidden=512, classes=10):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(in_dim, hidden), nn.ReLU(), nn.Linear(hidden, hidden),
                                 nn.ReLU(), nn.Linear(hidden, classes))

    def forward(self, x):
        return self.net(x)


def local_dataset(rank: int, size: int, in_dim: int, classes: int, seed: int
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    g = torch.Generator().manual_seed(seed + rank * 100_000)
    tg = torch.Generator().manual_seed(seed + 9999)
    x = torch.randn(size, in_dim, generator=g)
    w = torch.randn(in_dim, classes, generator=tg)
    b = torch.randn(classes, generator=tg)
    return x, torch.argmax(x @ w + b, dim=1)


def train(args, rank, world, device, *, bitwidth, stochastic, error_feedback) -> List[float]:
    torch.manual_seed(args.seed)
    model = TinyMLP(args.in_dim, args.hidden, args.num_classes).to(device)
    opt = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=0.9)
    xs, ys = local_dataset(rank, args.dataset_size, args.in_dim, args.num_classes, args.data_seed)
    group = LowBitGroup(bitwidth=bitwidth, stochastic_rounding=stochastic,
                        error_feedback=error_feedback, sr_seed=args.seed if stochastic else None)
    losses = []
    for step in range(1, args.steps + 1):
        lo = ((step - 1) * args.batch_size) % args.dataset_size
        idx = (torch.arange(args.batch_size) + lo) % args.dataset_size
        x, y = xs[idx].to(device), ys[idx].to(device)
        opt.zero_grad(set_to_none=True)
        loss = nn.functional.cross_entropy(model(x), y)
        loss.backward()
        for i, p in enumerate(model.parameters()):
            if p.grad is not None:
                group.all_reduce(p.grad, ef_key=("param", i))
                p.grad.div_(world)
        if args.grad_clip_norm > 0:
            torch.nn.utils.clip_grad_norm_(model.parameters(), args.grad_clip_norm)
        opt.step()
        t = loss.detach().float().view(1)
        dist.all_reduce(t)
        losses.append(float(t.item()) / world)
    return losses


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--bitwidth", type=int, default=4)
    ap.add_argument("--steps", type=int, default=160)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--in-dim", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--num-classes", type=int, default=10)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=2026)
    ap.add_argument("--data-seed", type=int, default=7)
    ap.add_argument("--dataset-size", type=int, default=8192)
    ap.add_argument("--grad-clip-norm", type=float, default=1.0)
    ap.add_argument("--baseline-bitwidth", type=int, default=8)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out-dir", default=None)
    args = ap.parse_args(argv)

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
    arms = {
        "no_stochastic": dict(bitwidth=args.bitwidth, stochastic=False, error_feedback=False),
        "stochastic": dict(bitwidth=args.bitwidth, stochastic=True, error_feedback=False),
        "stochastic_ef": dict(bitwidth=args.bitwidth, stochastic=True, error_feedback=True),
        "no_compression": dict(bitwidth=args.baseline_bitwidth, stochastic=False,
                               error_feedback=False),
    }
    curves = {name: train(args, rank, world, device, **kw) for name, kw in arms.items()}
    if rank == 0:
        print(json.dumps({"bitwidth": args.bitwidth, "world": world, "steps": args.steps,
                          "device": args.device,
                          **{f"loss_{k}": v[-1] for k, v in curves.items()},
                          **{f"loss_{k}_mean_last10": sum(v[-10:]) / 10
                             for k, v in curves.items()}}))
        if args.out_dir:
            os.makedirs(args.out_dir, exist_ok=True)
            path = os.path.join(args.out_dir, f"e2e_loss_curve_bw{args.bitwidth}.csv")
            with open(path, "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(["step"] + [f"loss_{k}" for k in curves])
                for i in range(args.steps):
                    w.writerow([i + 1] + [curves[k][i] for k in curves])
            from ..utils.plot import save_line_plot

            steps = list(range(1, args.steps + 1))
            save_line_plot(path[:-4] + ".png", {k: (steps, v) for k, v in curves.items()},
                           title=f"TinyMLP loss, {args.bitwidth}-bit, world {world}",
                           xlabel="step", ylabel="loss")
    dist.barrier()
    import bitscom_b200

    bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
