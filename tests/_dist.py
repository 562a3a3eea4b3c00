"""Spawn helper for multi-process tests (gloo on CPU, nccl on GPUs)."""

import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, backend, init_file, fn, args, errq, lowbit_options=None):
    try:
        os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"
        if backend in ("nccl", "lowbit"):
            torch.cuda.set_device(rank)
        if backend == "lowbit":
            import bitscom_b200

            bitscom_b200.init(**(lowbit_options or {}))
        dist.init_process_group(backend, init_method=f"file://{init_file}", rank=rank,
                                world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world, *args, backend="gloo", timeout=300, lowbit_options=None):
    """Run ``fn(rank, world, *args)`` in ``world`` processes; raise on any failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as tmp:
        init_file = os.path.join(tmp, "rendezvous")
        procs = [ctx.Process(target=_entry,
                             args=(r, world, backend, init_file, fn, args, errq, lowbit_options))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        failed = []
        for r, p in enumerate(procs):
            if p.is_alive():
                p.kill()
                failed.append(f"rank {r} timed out")
            elif p.exitcode != 0:
                failed.append(f"rank {r} exit code {p.exitcode}")
        msgs = []
        while not errq.empty():
            msgs.append("rank %d:\n%s" % errq.get())
        if failed or msgs:
            raise AssertionError("; ".join(failed) + "\n" + "\n".join(msgs))
