"""1F1B schedule: action order, activation memory bound, and a deadlock-freedom check of
the point-to-point plan (every posted batch must find its matching batch on the peer)."""

import pytest

from bitscom_b200.parallel.pp_schedule import (build_1f1b, communication_plan,
                                               max_live_microbatches)


@pytest.mark.parametrize("stages,mbs", [(1, 4), (2, 4), (4, 8), (4, 2), (8, 16), (3, 5)])
def test_1f1b_order_and_memory(stages, mbs):
    for s in range(stages):
        acts = build_1f1b(s, stages, mbs)
        assert sorted(i for k, i in acts if k == "F") == list(range(mbs))
        assert [i for k, i in acts if k == "B"] == list(range(mbs))
        seen = set()
        for k, i in acts:
            if k == "F":
                seen.add(i)
            else:
                assert i in seen  # backward only after its forward
        assert max_live_microbatches(acts) <= min(stages - s, mbs)


def _simulate(stages, mbs):
    """Play all stages' plans with NCCL's grouping rule: the operations of one batch run
    concurrently and complete one by one as the peer's CURRENT batch offers the matching
    operation; a stage moves on when its batch is empty.  Returns, per stage, the
    micro-batches whose activations / gradients it received, in arrival order."""
    plans = [[(k, mb, c) for k, mb, c in communication_plan(s, stages, mbs) if c.any()]
             for s in range(stages)]
    pos = [0] * stages
    got_fwd = [[] for _ in range(stages)]
    got_bwd = [[] for _ in range(stages)]

    def pending_ops(s):
        if pos[s] >= len(plans[s]):
            return None
        _, mb, c = plans[s][pos[s]]
        ops = set()
        if c.send_next:
            ops.add(("send", s + 1, mb))
        if c.send_prev:
            ops.add(("send", s - 1, mb))
        if c.recv_prev:
            ops.add(("recv", s - 1, None))
        if c.recv_next:
            ops.add(("recv", s + 1, None))
        return ops

    pending = [pending_ops(s) for s in range(stages)]
    for _ in range(20 * stages * mbs + 20):
        if all(p is None for p in pending):
            return got_fwd, got_bwd
        progressed = False
        for s in range(stages):
            if not pending[s]:
                continue
            for op in list(pending[s]):
                kind, peer, mb = op
                if kind != "send" or pending[peer] is None:
                    continue
                match = ("recv", s, None)
                if match in pending[peer]:
                    pending[peer].discard(match)
                    pending[s].discard(op)
                    (got_fwd if peer == s + 1 else got_bwd)[peer].append(mb)
                    progressed = True
        for s in range(stages):
            if pending[s] is not None and not pending[s]:
                pos[s] += 1
                pending[s] = pending_ops(s)
                progressed = True
        if not progressed:
            raise AssertionError(f"deadlock: {pending}")
    raise AssertionError("simulation did not terminate")


@pytest.mark.parametrize("stages,mbs", [(2, 4), (2, 1), (4, 8), (4, 4), (4, 2), (3, 7), (8, 16)])
def test_p2p_plan_is_deadlock_free_and_ordered(stages, mbs):
    got_fwd, got_bwd = _simulate(stages, mbs)
    for s in range(1, stages):
        assert got_fwd[s] == list(range(mbs))       # activations arrive in order
    for s in range(stages - 1):
        assert got_bwd[s] == list(range(mbs))       # gradients arrive in order


def test_timeline_simulation_matches_the_bubble_formula_and_shows_what_deferral_buys():
    """Plain 1F1B idles (P - 1) forward + backward slots; deferring weight gradients shortens
    the step only when the step's last backward is deferred too (the drain runs through it)."""
    from bitscom_b200.parallel.pp_schedule import simulate_timeline

    for stages, mbs in [(1, 4), (2, 8), (4, 8), (4, 16), (8, 32)]:
        plain = simulate_timeline(stages, mbs)
        assert abs(plain["efficiency"] - mbs / (mbs + stages - 1)) < 1e-12
        partly = simulate_timeline(stages, mbs, defer_wgrad=True)
        fully = simulate_timeline(stages, mbs, defer_wgrad=True, defer_last=True)
        assert partly["step_time"] == plain["step_time"]
        if stages > 1:
            assert fully["step_time"] == plain["step_time"] - (stages - 1) * 1.0
        assert fully["ideal_time"] == plain["ideal_time"]
    uneven = simulate_timeline(2, 8, t_forward=1.0, t_input_grad=1.4, t_weight_grad=0.6,
                               defer_wgrad=True, defer_last=True, t_send=0.05)
    assert 0.9 < uneven["efficiency"] < 1.0


# ---- interleaved (virtual-stage) schedule ------------------------------------------------

from bitscom_b200.parallel.pp_schedule import (build_interleaved, check_virtual_plan,  # noqa: E402
                                               interleaved_warmup, schedule_units,
                                               simulate_interleaved_timeline, virtual_plan)


@pytest.mark.parametrize("stages,mbs,chunks", [(2, 8, 2), (2, 4, 2), (4, 8, 2), (2, 8, 4),
                                               (4, 16, 2), (8, 16, 2), (3, 6, 2), (4, 4, 2),
                                               (2, 2, 3), (2, 8, 1), (4, 8, 1)])
def test_interleaved_order(stages, mbs, chunks):
    for rank in range(stages):
        acts = build_interleaved(rank, stages, mbs, chunks)
        want = sorted((mb, c) for mb in range(mbs) for c in range(chunks))
        assert sorted(a[1:] for a in acts if a[0] == "F") == want
        assert sorted(a[1:] for a in acts if a[0] == "B") == want
        seen = set()
        for kind, mb, c in acts:
            if kind == "F":
                # a micro-batch climbs the chunks in order
                assert c == 0 or (mb, c - 1) in seen
                seen.add((mb, c))
            else:
                assert (mb, c) in seen
        units = schedule_units(acts, interleaved_warmup(rank, stages, mbs, chunks))
        assert [a for u in units for a in u] == acts
        assert all(len(u) == 1 or (u[0][0], u[1][0]) == ("F", "B") for u in units)


@pytest.mark.parametrize("stages", [2, 3, 4, 8])
@pytest.mark.parametrize("mult", [1, 2, 4])
@pytest.mark.parametrize("chunks", [1, 2, 3])
def test_interleaved_plan_has_no_deadlock(stages, mult, chunks):
    mbs = stages * mult
    delivered = check_virtual_plan(stages, mbs, chunks)
    # every virtual-stage boundary carries one activation and one gradient per micro-batch
    assert delivered == 2 * mbs * (stages * chunks - 1)
    # each message is sent once and received once
    sent, got = [], []
    for rank in range(stages):
        for _, s, r in virtual_plan(rank, stages, mbs, chunks):
            sent += [m.tag() for m in s]
            got += [m.tag() for m in r]
    assert sorted(sent) == sorted(got) and len(set(sent)) == len(sent)


@pytest.mark.parametrize("stages,mbs,chunks", [(2, 8, 1), (2, 8, 2), (2, 8, 4), (4, 8, 2),
                                               (4, 16, 2), (8, 16, 2)])
def test_interleaved_bubble_matches_formula(stages, mbs, chunks):
    t = simulate_interleaved_timeline(stages, mbs, chunks)
    want = chunks * mbs / (chunks * mbs + stages - 1)
    assert abs(t["efficiency"] - want) < 1e-9


@pytest.mark.parametrize("stages,mbs,chunks", [(2, 8, 2), (2, 8, 4), (4, 8, 2), (4, 16, 2),
                                               (8, 16, 2)])
def test_interleaved_activation_memory(stages, mbs, chunks):
    """Peak number of chunk activations alive on a rank: the warm-up depth plus one."""
    for rank in range(stages):
        acts = build_interleaved(rank, stages, mbs, chunks)
        want = min((stages - rank - 1) * 2 + (chunks - 1) * stages + 1, mbs * chunks)
        assert max_live_microbatches(acts) == want


def test_interleaved_rejects_ragged_microbatches():
    with pytest.raises(ValueError):
        build_interleaved(0, 4, 6, 2)
