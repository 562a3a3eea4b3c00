"""A rank leaves a multi-GPU job between steps; the others learn of it on the host, shrink the
process group to the survivors and carry on with the fused collectives (GPU form of
tests/test_health_cpu.py).  The rank leaves with none of its kernels or collectives in
flight and frees its symmetric block only after its peers have unmapped it; NVLS is off in
NCCL and the fused kernels use plain peer stores, as failure tests must."""

import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu,
              pytest.mark.skipif(os.environ.get("BITSCOM_EXPERIMENTAL", "0") != "1",
                                 reason="not yet run on GPUs; set BITSCOM_EXPERIMENTAL=1")]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        os.environ.pop("BITSCOM_NVLS", None)
        import bitscom_b200 as bitscom
        from bitscom_b200.parallel.fused import FusedLowBitComm
        from bitscom_b200.utils.health import (HealthMonitor, PeerLostError, agree_on_survivors,
                                               shrink_process_group)

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=120), wait_for_workers=False)
        dist.init_process_group("nccl", store=dist.PrefixStore("epoch0", store), rank=rank,
                                world_size=world, timeout=datetime.timedelta(seconds=120),
                                device_id=dev)
        mon = HealthMonitor(store, rank, world, interval_s=0.1, timeout_s=20.0)
        group = bitscom.LowBitGroup(bitwidth=4, error_feedback=True, stage2_error_feedback=True,
                                    fused=True)
        n = 1 << 20
        gen = torch.Generator().manual_seed(100 + rank)
        grads = [torch.randn(n, generator=gen).cuda() for _ in range(3)]

        def step(i):
            t = grads[i].clone()
            dense = t.clone()
            group.all_reduce(t, ef_key="bucket")
            dist.all_reduce(dense)
            torch.cuda.synchronize()
            group.check_agreement(t)
            return (t - dense).abs().max().item()

        assert step(0) < 2.0
        dist.barrier()
        torch.cuda.synchronize()
        leaver = world - 1
        if rank == leaver:
            released = mon.leave(wait_release_s=120.0)  # peers unmap this rank's block first
            FusedLowBitComm.drop_cache()
            dist.destroy_process_group()
            q.put((rank, "left" if released else "left without release"))
            return
        deadline = time.monotonic() + 60
        lost = {}
        while time.monotonic() < deadline:
            try:
                mon.check()
            except PeerLostError as exc:
                lost = exc.ranks
                break
            time.sleep(0.02)
        assert lost == {leaver: "left"}, lost
        members = agree_on_survivors(store, rank, mon.alive(), epoch=1)
        new_rank, new_world = shrink_process_group(store, rank, members, epoch=1, device_id=dev)
        assert new_world == world - 1 and new_rank == rank
        group.rebind()            # drops the communicators (and peer mappings) of the old group
        mon.release([leaver])
        for i in (1, 2):
            assert step(i) < 2.0
        if new_world > 1:
            comm = group._fused_comms[id(group.pg)]
            assert comm.world == new_world
            comm.check_status()
            comm.check_canaries()
        mon.close()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as exc:  # surfaced in the parent
        import traceback

        q.put((rank, f"error: {exc}\n{traceback.format_exc()}"))


def test_a_rank_leaves_and_the_others_shrink_and_continue():
    n_gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n_gpus < 2:
        pytest.skip("needs 2 or more GPUs")
    world = min(n_gpus, 4)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    results = {}
    try:
        for _ in range(world):
            rank, msg = q.get(timeout=600)
            results[rank] = msg
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.terminate()
    want = {r: "ok" for r in range(world - 1)}
    want[world - 1] = "left"
    assert results == want, results
