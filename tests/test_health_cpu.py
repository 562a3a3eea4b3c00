"""Host-side failure detection (utils/health.py) and shrink-to-survivors recovery, on CPU
ranks: every failure is made on the host (a rank that leaves, raises, or just stops)."""

import multiprocessing as mp
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist

from bitscom_b200.utils.health import (HealthMonitor, PeerLostError, agree_on_survivors,
                                       shrink_process_group)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# -- single process, store shared by hand-driven monitors ------------------------------------
def _monitors(world, **kw):
    store = dist.HashStore()
    return [HealthMonitor(store, r, world, start=False, **kw) for r in range(world)]


def test_all_beating_means_all_alive():
    mons = _monitors(3, interval_s=0.1, timeout_s=1.0)
    for step in range(5):
        for m in mons:
            m.beat()
        for m in mons:
            m.poll(now=time.monotonic() + 0.5 * step)
    for m in mons:
        m.check()
        assert m.alive() == [0, 1, 2]


def test_silent_peer_is_reported_after_the_timeout_and_forgiven_if_it_returns():
    a, b = _monitors(2, interval_s=0.1, timeout_s=1.0)
    a.beat(), b.beat()
    t0 = time.monotonic()
    a.poll(now=t0)
    a.poll(now=t0 + 0.9)
    a.check()  # not yet
    a.poll(now=t0 + 1.2)
    with pytest.raises(PeerLostError) as err:
        a.check()
    assert list(err.value.ranks) == [1] and "silent" in err.value.ranks[1]
    b.beat()  # it was only slow
    a.poll(now=t0 + 1.3)
    a.check()


def test_a_peer_that_never_started_counts_as_silent():
    a, _ = _monitors(2, interval_s=0.1, timeout_s=0.5)
    a.beat()
    a.poll(now=time.monotonic() + 1.0)
    with pytest.raises(PeerLostError):
        a.check()


def test_leave_and_reported_failure_are_seen_at_the_next_poll_and_are_final():
    a, b, c = _monitors(3, interval_s=0.1, timeout_s=60.0)
    for m in (a, b, c):
        m.beat()
    b.leave()
    with pytest.raises(ValueError):
        with c.guard():
            raise ValueError("loss is NaN")
    a.poll()
    with pytest.raises(PeerLostError) as err:
        a.check()
    assert err.value.ranks[1] == "left"
    assert err.value.ranks[2].startswith("failed: ValueError: loss is NaN")
    assert a.alive() == [0]
    c.beat()  # a failed rank that keeps beating stays failed
    a.poll()
    assert 2 in a.lost()


def test_leaver_waits_until_its_peers_have_released_its_memory():
    import threading

    a, b, c = _monitors(3, interval_s=0.05, timeout_s=60.0)
    for m in (a, b, c):
        m.beat()
    assert c.leave(wait_release_s=0.3) is False  # nobody released yet: gives up after 0.3 s
    done = {}
    t = threading.Thread(target=lambda: done.setdefault("ok", c.leave(wait_release_s=10.0)))
    t.start()
    time.sleep(0.1)
    a.poll()
    assert a.lost() == {2: "left"}
    a.release([2])
    time.sleep(0.2)
    assert "ok" not in done  # rank 1 still holds a mapping
    b.release([2])
    t.join(timeout=10)
    assert done.get("ok") is True


def test_attached_monitor_stops_a_collective_before_it_is_launched(monkeypatch):
    """``LowBitGroup.attach_health``: with a lost peer every collective entry point raises on
    the host and nothing reaches the process group."""
    import bitscom_b200.api as api

    calls = []
    monkeypatch.setattr(api.dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(api.dist, "get_rank", lambda group=None: 0)
    class Done:
        def wait(self):
            return True

    monkeypatch.setattr(api.dist, "all_reduce",
                        lambda *a, **k: (calls.append("all_reduce"), Done())[1])
    group = api.LowBitGroup(bitwidth=8, process_group=object())
    a, b = _monitors(2, interval_s=0.1, timeout_s=60.0)
    a.beat(), b.beat()
    a.poll()
    group.attach_health(a)
    group.all_reduce(torch.ones(8))          # healthy: goes through (8 bit = dense path)
    assert calls == ["all_reduce"]
    b.leave()
    a.poll()
    for call in (lambda: group.all_reduce(torch.ones(8)),
                 lambda: group.all_reduce_stream(torch.ones(8), stream=None),
                 lambda: group.reduce_scatter_lowbit(torch.ones(4), torch.ones(8)),
                 lambda: group.all_gather_lowbit(torch.ones(8), torch.ones(4))):
        with pytest.raises(PeerLostError):
            call()
    assert calls == ["all_reduce"]
    group.attach_health(None)
    group.all_reduce(torch.ones(8))
    assert calls == ["all_reduce", "all_reduce"]


def test_guard_does_not_publish_news_about_other_ranks():
    a, b = _monitors(2, interval_s=0.1, timeout_s=60.0)
    with pytest.raises(PeerLostError):
        with a.guard():
            raise PeerLostError({1: "left"})
    b.beat()
    b.poll()
    b.check()  # rank 0 did not mark itself failed


def test_background_thread_detects_a_stopped_peer():
    store = dist.HashStore()
    a = HealthMonitor(store, 0, 2, interval_s=0.05, timeout_s=0.4)
    b = HealthMonitor(store, 1, 2, interval_s=0.05, timeout_s=0.4)
    try:
        time.sleep(0.3)
        a.check(), b.check()
        b.close()  # stops beating without a word
        deadline = time.monotonic() + 5.0
        while not a.lost() and time.monotonic() < deadline:
            time.sleep(0.05)
        assert "silent" in a.lost().get(1, "")
    finally:
        a.close(), b.close()


def test_survivor_views_must_match():
    store = dist.HashStore()
    import threading

    out = {}

    def vote(rank, view):
        try:
            out[rank] = agree_on_survivors(store, rank, view, epoch=1, timeout_s=5.0)
        except PeerLostError as exc:
            out[rank] = exc

    ts = [threading.Thread(target=vote, args=(0, [0, 1])),
          threading.Thread(target=vote, args=(1, [0, 1]))]
    [t.start() for t in ts], [t.join() for t in ts]
    assert out == {0: [0, 1], 1: [0, 1]}
    out.clear()

    def vote2(rank, view):
        try:
            out[rank] = agree_on_survivors(store, rank, view, epoch=2, timeout_s=1.0)
        except PeerLostError as exc:
            out[rank] = exc

    ts = [threading.Thread(target=vote2, args=(0, [0, 1, 2])),
          threading.Thread(target=vote2, args=(1, [0, 1]))]
    [t.start() for t in ts], [t.join() for t in ts]
    assert isinstance(out[0], PeerLostError)  # disagreement (or rank 2 never voted)
    assert isinstance(out[1], PeerLostError)


# -- three CPU ranks: one leaves between steps, two shrink and carry on -----------------------
def _elastic_worker(rank, world, port, q):
    try:
        os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"
        import datetime

        import bitscom_b200 as bitscom

        # the store is hosted by rank 0, which survives
        store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=60), wait_for_workers=False)
        dist.init_process_group("gloo", store=dist.PrefixStore("epoch0", store), rank=rank,
                                world_size=world, timeout=datetime.timedelta(seconds=60))
        mon = HealthMonitor(store, rank, world, interval_s=0.05, timeout_s=2.0)
        group = bitscom.LowBitGroup(bitwidth=4, error_feedback=True, stage2_error_feedback=True,
                                    sr_seed=3)
        n = 1000  # not a multiple of 3 * 256, nor of 2 * 256
        gen = torch.Generator().manual_seed(100 + rank)
        grads = [torch.randn(n, generator=gen) for _ in range(4)]

        def step(i):
            t = grads[i].clone()
            group.all_reduce(t, ef_key="bucket")
            return t

        out0 = step(0)
        want0 = sum(torch.randn(n, generator=torch.Generator().manual_seed(100 + r))
                    for r in range(world))
        assert (out0 - want0).abs().max() < 1.5, "3-rank low-bit sum is off"
        res_before = group._ef_states["bucket"].stage1[:n].clone()
        dist.barrier()
        if rank == 2:
            mon.leave()            # between steps, nothing in flight
            dist.destroy_process_group()
            q.put((rank, "left"))
            return
        # survivors: learn of it on the host, before the next collective
        deadline = time.monotonic() + 20
        lost = {}
        while time.monotonic() < deadline:
            try:
                mon.check()
            except PeerLostError as exc:
                lost = exc.ranks
                break
            time.sleep(0.02)
        assert lost == {2: "left"}, lost
        members = agree_on_survivors(store, rank, mon.alive(), epoch=1)
        assert members == [0, 1]
        new_rank, new_world = shrink_process_group(store, rank, members, epoch=1)
        assert (new_rank, new_world) == (rank, 2)
        group.rebind()
        out1 = step(1)
        st = group._ef_states["bucket"]
        assert st.stage1.numel() == 2 * 500 and st.stage2.numel() == 500
        # the residual was carried into the new shard plan, not reset: the result equals,
        # bit for bit, the golden model started from the residuals held before the shrink
        from bitscom_b200.parallel.simulate import SimState, simulate_all_reduce

        g_all = [torch.empty(n) for _ in range(2)]
        r_all = [torch.empty(n) for _ in range(2)]
        dist.all_gather(g_all, grads[1])
        dist.all_gather(r_all, res_before)
        state = SimState(stage1=[torch.nn.functional.pad(r, (0, 1000 - n)) for r in r_all],
                         stage2=[torch.zeros(500) for _ in range(2)])
        want1 = simulate_all_reduce(g_all, 4, 256, state=state, stage2=True)[rank]
        assert torch.equal(out1, want1), "result after the shrink differs from the golden model"
        assert res_before.abs().max() > 0  # there was something to carry
        group.check_agreement(out1)
        out2 = step(2)
        group.check_agreement(out2)
        mon.close()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as exc:  # surfaced in the parent
        import traceback

        q.put((rank, f"error: {exc}\n{traceback.format_exc()}"))


def test_three_ranks_shrink_to_two_after_one_leaves():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_elastic_worker, args=(r, 3, port, q)) for r in range(3)]
    [p.start() for p in procs]
    results = {}
    try:
        for _ in range(3):
            rank, msg = q.get(timeout=180)
            results[rank] = msg
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    assert results == {0: "ok", 1: "ok", 2: "left"}, results
