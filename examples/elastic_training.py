"""Data-parallel training that survives the loss of a rank (CPU ranks over gloo, or GPUs).

    python -m bitscom_b200.launch --nproc 3 --min-nproc 2 --shrink --max-restarts 2 -- \
        python examples/elastic_training.py --steps 12 --ckpt /tmp/elastic_ckpt \
            --fail-rank 2 --fail-step 5

Every rank heartbeats through the launcher's store.  When a rank disappears (here: rank 2
exits on purpose at step 5 of the first generation), the others notice on the host, stop
between steps with exit code 3, and the launcher starts a new generation with the survivors.
The program resumes from the per-rank checkpoints: weights and step from rank 0's file,
error-feedback residuals from each rank's own file when it belongs to the same step.
"""

import argparse
import json
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bitscom_b200 as bitscom  # noqa: E402
from bitscom_b200.launch import STOPPED_FOR_PEER, agent_store  # noqa: E402
from bitscom_b200.utils.checkpoint import checkpoint_path, load_checkpoint, save_checkpoint  # noqa: E402
from bitscom_b200.utils.health import HealthMonitor, PeerLostError  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--fail-rank", type=int, default=-1)
    ap.add_argument("--fail-step", type=int, default=-1)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--pg-timeout", type=float, default=10.0,
                    help="seconds after which a collective without its peer gives up")
    args = ap.parse_args(argv)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    generation = int(os.environ.get("BITSCOM_RESTART_COUNT", "0"))
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=args.pg_timeout))
    else:
        dev = torch.device("cpu")
        # a short timeout: a collective whose peer is gone must fail, not wait for half an hour
        dist.init_process_group("gloo", timeout=timedelta(seconds=args.pg_timeout))

    store = agent_store()
    monitor = None
    if store is not None and world > 1:
        # keys of an earlier generation must not be mistaken for this one's
        monitor = HealthMonitor(store, rank, world, interval_s=0.1, timeout_s=3.0,
                                prefix=f"bitscom/health/gen{generation}")

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(),
                                torch.nn.Linear(64, 1)).to(dev)
    params = list(model.parameters())
    group = bitscom.LowBitGroup(bitwidth=4, error_feedback=True)
    group.attach_health(monitor)  # checked again right before every collective
    teacher = torch.randn(32, 1, generator=torch.Generator().manual_seed(7)).to(dev)

    # -- resume ------------------------------------------------------------------------------
    start, mine = 0, None
    if os.path.exists(checkpoint_path(args.ckpt, rank)):
        mine = load_checkpoint(args.ckpt, rank)
    head = torch.tensor([mine["step"] if (rank == 0 and mine) else 0], dtype=torch.int64,
                        device=dev)
    dist.broadcast(head, src=0)
    start = int(head.item())
    if start > 0:
        if rank == 0:
            model.load_state_dict(mine["model"])
        for p in params:
            dist.broadcast(p.data, src=0)
        if mine is not None and mine["step"] == start:
            group.load_state_dict(mine["lowbit"])   # this rank's own residuals
            group.rebind()                           # ... re-laid out for the new world size

    loss = torch.zeros(())
    try:
        for step in range(start, args.steps):
            if monitor is not None:
                monitor.check()
            if generation == 0 and rank == args.fail_rank and step == args.fail_step:
                os._exit(17)  # the failure of this example: the process is simply gone
            g = torch.Generator().manual_seed(1000 * step + rank)
            x = torch.randn(64, 32, generator=g).to(dev)
            loss = torch.nn.functional.mse_loss(model(x), x @ teacher)
            model.zero_grad(set_to_none=True)
            loss.backward()
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            group.all_reduce(flat, ef_key="grads")
            flat.div_(world)
            off = 0
            with torch.no_grad():
                for p in params:
                    p.add_(flat[off:off + p.numel()].view_as(p), alpha=-0.05)
                    off += p.numel()
            save_checkpoint(args.ckpt, {"step": step + 1, "model": model.state_dict(),
                                        "lowbit": group.state_dict()}, rank)
    except Exception as exc:
        # a collective that lost its peer fails on its own; the monitor says who it was
        lost = {}
        deadline = time.monotonic() + 10.0
        while monitor is not None and not lost and time.monotonic() < deadline:
            lost = monitor.lost()
            time.sleep(0.05)
        if not lost and not isinstance(exc, PeerLostError):
            raise
        print(json.dumps({"rank": rank, "generation": generation,
                          "stopped": str(PeerLostError(lost) if lost else exc)}), flush=True)
        os._exit(STOPPED_FOR_PEER)  # no teardown collectives: the peer would never answer

    if rank == 0:
        print(json.dumps({"finished": True, "generation": generation, "world": world,
                          "resumed_at": start, "steps": args.steps,
                          "loss": float(loss.item())}), flush=True)
    dist.barrier()
    if monitor is not None:
        monitor.leave()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
