"""Step-by-step comparison of a low-bit collective with its dense counterpart: relative
error of the result and time per call, for ``allreduce``, ``reduce_scatter`` and
``all_gather``, at one or several bitwidths.

Every step draws a fresh input on every rank (a ramp from -1 to 1 plus noise and a
per-rank offset, as in the reference's ``benchmarks/collective_compare.py:14-38``), runs
the dense collective and the low-bit one on clones of it and records
``||lowbit - dense|| / ||dense||`` together with both times, each the MAX over ranks.  On
CUDA the times come from CUDA events on the launching stream; on CPU ranks (gloo) from the
host clock.  One CSV per bitwidth and collective is written to ``--out-dir`` and a JSON
line per bitwidth is printed, which replaces the reference's per-bitwidth torchrun
driver (``benchmarks/collective_compare_multibw.py``): all bitwidths run in one job.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m bitscom_b200.bench.collective_compare --collective reduce_scatter \\
        --bitwidths 1 2 4 8 --device cpu
"""

from __future__ import annotations

import argparse
import csv
import json
import os
import time
from typing import Callable, List, Tuple

import torch
import torch.distributed as dist

from ..api import LowBitGroup

COLLECTIVES = ("allreduce", "reduce_scatter", "all_gather")


def make_input(rank: int, numel: int, seed: int, device, scale: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + rank * 31)
    base = torch.linspace(-1.0, 1.0, steps=numel)
    x = base + torch.randn(numel, generator=g) * 0.02 + rank * 0.05
    return (x * scale).to(device)


def timed(fn: Callable[[], None], device) -> float:
    """Milliseconds of one call (device time on CUDA, host time on CPU)."""
    if device.type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b)
    t0 = time.perf_counter()
    fn()
    return (time.perf_counter() - t0) * 1e3


def one_step(kind: str, group: LowBitGroup, rank: int, world: int, numel: int, seed: int,
             device) -> Tuple[float, float, float]:
    """Returns (relative error, low-bit ms, dense ms) of one step on this rank."""
    if kind == "allreduce":
        dense = make_input(rank, numel, seed, device)
        low = dense.clone()
        t_dense = timed(lambda: dist.all_reduce(dense), device)
        t_low = timed(lambda: group.all_reduce(low), device)
    elif kind == "reduce_scatter":
        full = make_input(rank, numel * world, seed, device)
        dense, low = torch.empty(numel, device=device), torch.empty(numel, device=device)
        t_dense = timed(lambda: dist.reduce_scatter_tensor(dense, full.clone())
                        if device.type == "cuda" else
                        dense.copy_(_gloo_reduce_scatter(full, rank, world)), device)
        t_low = timed(lambda: group.reduce_scatter_lowbit(low, full), device)
    else:
        mine = make_input(rank, numel, seed, device)
        dense, low = (torch.empty(numel * world, device=device) for _ in range(2))
        t_dense = timed(lambda: dist.all_gather_into_tensor(dense, mine)
                        if device.type == "cuda" else
                        dense.copy_(_gloo_all_gather(mine, world)), device)
        t_low = timed(lambda: group.all_gather_lowbit(low, mine), device)
    err = float((low.float() - dense.float()).norm() / dense.float().norm().clamp_min(1e-12))
    return err, t_low, t_dense


def _gloo_reduce_scatter(full: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    tmp = full.clone()  # gloo has no reduce_scatter: all-reduce and keep the own shard
    dist.all_reduce(tmp)
    n = tmp.numel() // world
    return tmp[rank * n:(rank + 1) * n]


def _gloo_all_gather(mine: torch.Tensor, world: int) -> torch.Tensor:
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    return torch.cat(parts)


def run(kind: str, bitwidth: int, args, rank: int, world: int, device) -> List[Tuple]:
    group = LowBitGroup(bitwidth=bitwidth, stochastic_rounding=args.stochastic_rounding,
                        error_feedback=args.error_feedback,
                        stage2_error_feedback=args.stage2_error_feedback,
                        block_size=args.block_size, sr_seed=args.seed)
    rows = []
    for step in range(1, args.steps + 1):
        err, t_low, t_dense = one_step(kind, group, rank, world, args.numel,
                                       args.seed + step * 13, device)
        t = torch.tensor([err, t_low, t_dense], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows.append((step, *[float(v) for v in t.tolist()]))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description="low-bit collective vs dense baseline")
    ap.add_argument("--collective", default="allreduce", choices=COLLECTIVES)
    ap.add_argument("--bitwidths", nargs="+", type=int, default=[4])
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup-steps", type=int, default=3,
                    help="leading steps left out of the mean times")
    ap.add_argument("--numel", type=int, default=1 << 18)
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--stochastic-rounding", action="store_true")
    ap.add_argument("--error-feedback", action="store_true")
    ap.add_argument("--stage2-error-feedback", action="store_true")
    ap.add_argument("--seed", type=int, default=2026)
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
    if world < 2:
        raise RuntimeError("collective_compare needs at least two ranks")
    results = []
    for bw in args.bitwidths:
        rows = run(args.collective, bw, args, rank, world, device)
        steady = rows[min(args.warmup_steps, len(rows) - 1):]
        mean = lambda i: sum(r[i] for r in steady) / len(steady)  # noqa: E731
        rec = {"collective": args.collective, "bitwidth": bw, "world": world,
               "numel": args.numel, "device": args.device, "steps": args.steps,
               "rel_error_mean": mean(1), "rel_error_max": max(r[1] for r in rows),
               "lowbit_ms": mean(2), "dense_ms": mean(3),
               "speedup_vs_dense": mean(3) / max(mean(2), 1e-12)}
        results.append(rec)
        if rank == 0:
            print(json.dumps(rec))
            if args.out_dir:
                os.makedirs(args.out_dir, exist_ok=True)
                path = os.path.join(args.out_dir, f"{args.collective}_compare_bw{bw}.csv")
                with open(path, "w", newline="") as f:
                    w = csv.writer(f)
                    w.writerow(["step", "rel_error", "lowbit_ms", "baseline_ms"])
                    w.writerows(rows)
                from ..utils.plot import save_line_plot

                steps = [r[0] for r in rows]
                save_line_plot(path[:-4] + ".png",
                               {"lowbit_ms": (steps, [r[2] for r in rows]),
                                "baseline_ms": (steps, [r[3] for r in rows])},
                               title=f"{args.collective} bw{bw} world {world}: time per call",
                               xlabel="step", ylabel="ms")
    dist.barrier()
    import bitscom_b200

    bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
    dist.destroy_process_group()
    return results


if __name__ == "__main__":
    main()
