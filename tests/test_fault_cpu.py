"""Failure detection with failures made on the HOST, among CPU ranks (gloo): mismatched
options, a rank that raises before the collective, a rank that leaves between steps.  The
survivors must get an exception within the process-group timeout, never a hang."""

import os
import tempfile
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _spawn(fn, world, timeout_s=5, join_s=60):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as tmp:
        init = os.path.join(tmp, "rdzv")
        procs = [ctx.Process(target=_entry, args=(r, world, init, timeout_s, fn, q))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(join_s)
        alive = [p.is_alive() for p in procs]
        for p in procs:
            if p.is_alive():
                p.kill()
        out = {}
        while not q.empty():
            r, v = q.get()
            out[r] = v
        assert not any(alive), f"ranks hung: {alive}"
        return out


def _entry(rank, world, init, timeout_s, fn, q):
    os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"
    dist.init_process_group("gloo", init_method=f"file://{init}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=timeout_s))
    try:
        q.put((rank, fn(rank, world)))
    except BaseException as exc:  # report, then leave without cleanup
        q.put((rank, f"unhandled {type(exc).__name__}: {exc}"))
    os._exit(0)


def _mismatch(rank, world):
    from bitscom_b200 import LowBitGroup

    group = LowBitGroup(bitwidth=4 if rank == 0 else 2)
    try:
        group.check_consistency()
    except RuntimeError as exc:
        return "raised: " + str(exc)[:60]
    return "no error"


def test_mismatched_options_are_detected_on_every_rank():
    out = _spawn(_mismatch, 2)
    assert all(v.startswith("raised: LowBitGroup options differ") for v in out.values()), out


def _one_rank_raises(rank, world):
    from bitscom_b200 import LowBitGroup

    group = LowBitGroup(bitwidth=4)
    x = torch.randn(4096)
    group.all_reduce(x.clone())            # a healthy step first
    if rank == 1:
        return "left before step 2"        # never joins the second collective
    t0 = time.time()
    try:
        group.all_reduce(x.clone())
    except Exception as exc:
        return f"error after {time.time() - t0:.1f}s: {type(exc).__name__}"
    return "no error"


def test_survivor_gets_an_error_when_a_rank_leaves_between_steps():
    out = _spawn(_one_rank_raises, 2, timeout_s=4)
    assert out[1] == "left before step 2"
    assert out[0].startswith("error after"), out
    assert float(out[0].split()[2][:-2]) < 30.0


def _async_error_surfaces_at_wait(rank, world):
    from bitscom_b200 import LowBitGroup

    group = LowBitGroup(bitwidth=4)
    x = torch.randn(4096)
    if rank == 1:
        return "absent"
    try:
        work = group.all_reduce(x, async_op=True)
        work.wait()
    except Exception as exc:
        return "error: " + type(exc).__name__
    return "no error"


def test_async_work_reports_peer_failure_at_wait():
    out = _spawn(_async_error_surfaces_at_wait, 2, timeout_s=4)
    assert out[0].startswith("error: "), out
