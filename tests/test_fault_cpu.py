"""Failure detection with failures made on the HOST, among CPU ranks (gloo): mismatched
options, a rank that raises before the collective, a rank that leaves between steps.  The
survivors must get an exception within the process-group timeout, never a hang."""

import os
import tempfile
import time
from datetime import timedelta

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


# ---------------------------------------------------------------------------------------
# a fake transport: the collectives the host engine uses are wrapped on ONE rank so that a
# shard arrives late or damaged
# ---------------------------------------------------------------------------------------
def _with_fake_transport(rank, world, mode):
    from bitscom_b200 import LowBitGroup

    real_a2a, real_gather = dist.all_to_all_single, dist.all_gather
    calls = {"n": 0}

    def fake_a2a(output, input, *args, **kwargs):
        if mode == "delay":
            time.sleep(0.5)                       # a slow link: later, but intact
        return real_a2a(output, input, *args, **kwargs)

    def fake_gather(tensor_list, tensor, *args, **kwargs):
        # the gather half carries the reduced, re-quantized shards: damage on this path makes
        # one rank dequantize different bits than the others
        work = real_gather(tensor_list, tensor, *args, **kwargs)
        calls["n"] += 1
        if mode == "corrupt" and calls["n"] == 1 and tensor.dtype == torch.uint8:
            if work is not None:
                work.wait()
            tensor_list[1].view(-1)[5] ^= 0x7F    # one damaged byte of packed codes
        return work

    if rank == 0:
        dist.all_to_all_single, dist.all_gather = fake_a2a, fake_gather
    group = LowBitGroup(bitwidth=4)
    x = torch.randn(8192, generator=torch.Generator().manual_seed(3 + rank))
    group.all_reduce(x)
    try:
        group.check_agreement(x)
    except RuntimeError as exc:
        return "disagree: " + str(exc)[:40]
    return "agree"


def _delay(rank, world):
    return _with_fake_transport(rank, world, "delay")


def _corrupt(rank, world):
    return _with_fake_transport(rank, world, "corrupt")


def test_delayed_shard_is_only_late():
    out = _spawn(_delay, 2, timeout_s=20)
    assert out == {0: "agree", 1: "agree"}, out


def test_damaged_shard_is_caught_by_the_agreement_check():
    out = _spawn(_corrupt, 2, timeout_s=20)
    assert all(v.startswith("disagree: ranks disagree") for v in out.values()), out
