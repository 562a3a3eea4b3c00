"""ResNet-18 CIFAR-shaped DDP training with low-bit gradient all-reduce.

Synthetic 32x32x3 images drawn N(0,1), uniform labels over 10 classes, batch 256 per
GPU, SGD momentum 0.9; gradients go through ``torch`` DDP's 25 MB buckets and the
``lowbit_ddp_comm_hook`` (2-bit, block 256, error feedback) which runs the fused kernel
on a side stream under backward.  ``--mode nccl`` is the dense baseline.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m bitscom_b200.trainer.resnet18_ddp --steps 50
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.nn.parallel import DistributedDataParallel as DDP

from ..api import LowBitGroup
from ..models.resnet import ResNet18
from ..parallel.hooks import lowbit_ddp_comm_hook, make_ddp_hook_state


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--bitwidth", type=int, default=2)
    ap.add_argument("--mode", default="lowbit", choices=["lowbit", "backend", "nccl"],
                    help="lowbit: NCCL group + the Python DDP comm hook; backend: the C++ "
                         "`lowbit` torch.distributed backend under DDP's own reducer (no Python "
                         "on the gradient path); nccl: plain DDP")
    ap.add_argument("--bucket-mb", type=int, default=25)
    ap.add_argument("--no-error-feedback", action="store_true")
    ap.add_argument("--out", default="bench_outputs/resnet18_ddp.jsonl")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu",
                    help="'cpu' runs the same program on CPU ranks over gloo (plumbing check)")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ.get("WORLD_SIZE", 1))
    cuda = args.device == "cuda"
    if cuda and args.mode == "backend":
        import bitscom_b200

        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        bitscom_b200.init(bitwidth=args.bitwidth, block_size=256,
                          error_feedback_mode="none" if args.no_error_feedback else "ef21_plus",
                          stage2_error_feedback=not args.no_error_feedback)
        dist.init_process_group("lowbit")
    elif cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    torch.manual_seed(0)
    model = ResNet18().to(dev).to(memory_format=torch.channels_last)
    ddp = DDP(model, device_ids=[local] if cuda else None, bucket_cap_mb=args.bucket_mb)
    if args.mode == "lowbit" and world > 1:
        group = LowBitGroup(bitwidth=args.bitwidth, block_size=256,
                            error_feedback=not args.no_error_feedback)
        ddp.register_comm_hook(make_ddp_hook_state(group), lowbit_ddp_comm_hook)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn(args.batch, 3, 32, 32, device=dev, generator=g).contiguous(
        memory_format=torch.channels_last)
    y = torch.randint(0, 10, (args.batch,), device=dev, generator=g)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16) if cuda else contextlib.nullcontext():
            loss = F.cross_entropy(ddp(x), y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(args.warmup):
        step()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    if cuda:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
    t0 = time.perf_counter()
    first = last = None
    for i in range(args.steps):
        loss = step()
        if i == 0:
            first = loss.detach()
        last = loss.detach()
    if cuda:
        e.record()
        torch.cuda.synchronize()
        elapsed_ms = s.elapsed_time(e)
    else:
        elapsed_ms = (time.perf_counter() - t0) * 1e3
    ms = torch.tensor([elapsed_ms / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        row = {"workload": "resnet18_cifar_ddp", "mode": args.mode, "world": world,
               "bitwidth": args.bitwidth if args.mode != "nccl" else 32,
               "device": args.device, "batch_per_gpu": args.batch,
               "ms_per_step": float(ms.item()),
               "samples_per_s": world * args.batch / float(ms.item()) * 1e3,
               "loss_first": float(first.item()), "loss_last": float(last.item())}
        print(json.dumps(row), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "a") as f:
                f.write(json.dumps(row) + "\n")
    dist.barrier()
    import bitscom_b200

    bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
