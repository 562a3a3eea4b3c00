"""Spawn helper for multi-process tests (gloo on CPU, nccl on GPUs).

Every rank runs ``fn(rank, world, *args)`` and then tears down in order: the library's own
collective ``shutdown()`` (symmetric blocks released with a handshake), a barrier, and
``destroy_process_group``.  The parent gives the whole group ONE deadline (not one per
process), and a rank is only called "timed out" if it is still alive a grace period after the
deadline or after its peers have gone.  With ``BITSCOM_TEST_TRACE_DIR`` set, every rank appends
time stamps of its phases (import, rendezvous, body, shutdown, destroy) to a file there, so a
slow or stuck run can be attributed to a phase afterwards.
"""

import json
import os
import tempfile
import time
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class _Trace:
    def __init__(self, rank, label):
        self.dir = os.environ.get("BITSCOM_TEST_TRACE_DIR")
        self.rank, self.label, self.t0 = rank, label, time.time()

    def mark(self, phase):
        if not self.dir:
            return
        try:
            os.makedirs(self.dir, exist_ok=True)
            with open(os.path.join(self.dir, "ranks.jsonl"), "a") as f:
                f.write(json.dumps({"test": self.label, "rank": self.rank, "phase": phase,
                                    "t": round(time.time() - self.t0, 3),
                                    "wall": time.time()}) + "\n")
        except OSError:
            pass


def _entry(rank, world, backend, init_file, fn, args, errq, lowbit_options=None):
    trace = _Trace(rank, getattr(fn, "__module__", "") + "." + getattr(fn, "__name__", "fn"))
    try:
        os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"
        # the ranks share the machine's cores: one intra-op thread each, or W processes times
        # one OpenMP team per hardware thread oversubscribe the CPUs the job may use
        torch.set_num_threads(1)
        trace.mark("start")
        if backend in ("nccl", "lowbit"):
            torch.cuda.set_device(rank)
        import bitscom_b200

        if backend == "lowbit":
            bitscom_b200.init(**(lowbit_options or {}))
        dist.init_process_group(backend, init_method=f"file://{init_file}", rank=rank,
                                world_size=world)
        trace.mark("rendezvous")
        fn(rank, world, *args)
        trace.mark("body")
        dist.barrier()
        bitscom_b200.shutdown()
        trace.mark("shutdown")
        if dist.is_initialized():
            dist.destroy_process_group()
        trace.mark("destroyed")
    except Exception:
        trace.mark("failed")
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world, *args, backend="gloo", timeout=300, lowbit_options=None, grace=20):
    """Run ``fn(rank, world, *args)`` in ``world`` processes; raise on any failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    env_before = os.environ.get("OMP_NUM_THREADS")
    os.environ["OMP_NUM_THREADS"] = "1"  # inherited by the children
    try:
        with tempfile.TemporaryDirectory() as tmp:
            init_file = os.path.join(tmp, "rendezvous")
            procs = [ctx.Process(target=_entry,
                                 args=(r, world, backend, init_file, fn, args, errq,
                                       lowbit_options))
                     for r in range(world)]
            t0 = time.monotonic()
            for p in procs:
                p.start()
            deadline = t0 + timeout
            while time.monotonic() < deadline and any(p.is_alive() for p in procs):
                time.sleep(0.05)
                if any(p.exitcode not in (None, 0) for p in procs):
                    # a rank failed: its peers will never finish a collective with it
                    deadline = min(deadline, time.monotonic() + grace)
            # ranks still alive get a grace period (teardown is not instantaneous) before they
            # are called stuck
            end = time.monotonic() + grace
            while time.monotonic() < end and any(p.is_alive() for p in procs):
                time.sleep(0.05)
            failed = []
            for r, p in enumerate(procs):
                if p.is_alive():
                    p.kill()
                    p.join(10)
                    failed.append(f"rank {r} still running after {time.monotonic() - t0:.0f} s")
                elif p.exitcode != 0:
                    failed.append(f"rank {r} exit code {p.exitcode}")
            msgs = []
            while not errq.empty():
                msgs.append("rank %d:\n%s" % errq.get())
            if failed or msgs:
                raise AssertionError("; ".join(failed) + "\n" + "\n".join(msgs))
    finally:
        if env_before is None:
            os.environ.pop("OMP_NUM_THREADS", None)
        else:
            os.environ["OMP_NUM_THREADS"] = env_before
