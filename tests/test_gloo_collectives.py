"""Multi-process CPU tests over gloo: the host engines against the golden model.

test_config1_* is the plumbing configuration: world 2, 1 Mi fp32 elements drawn N(0,1)
from seed 1234+rank, 4-bit, block 256, nearest rounding, error feedback on, 5 iterations;
every iteration must equal the single-process simulation bit for bit.
"""

import pytest
import torch
import torch.distributed as dist

from _dist import run_ranks
from bitscom_b200 import LowBitGroup
from bitscom_b200.parallel.simulate import (SimState, simulate_all_gather,
                                            simulate_all_reduce, simulate_reduce_scatter)


def _rank_input(rank, numel, it=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(1234 + rank + 1000 * it)
    return torch.randn(numel, generator=g).to(dtype)


def _ar_worker(rank, world, numel, bits, block, iters, ef, stage2, sr, dtype):
    group = LowBitGroup(bitwidth=bits, block_size=block, error_feedback=ef,
                        stage2_error_feedback=stage2, stochastic_rounding=sr,
                        sr_seed=99 if sr else None)
    state = SimState() if ef else None
    sim_calls = 0
    for it in range(iters):
        mine = _rank_input(rank, numel, it, dtype)
        everyone = [_rank_input(r, numel, it, dtype) for r in range(world)]
        sim_calls += 1
        seed = (99 * 0x9E3779B97F4A7C15 + sim_calls) & 0xFFFFFFFFFFFFFFFF if sr else None
        want = simulate_all_reduce(everyone, bits, block, stochastic=sr, seed=seed,
                                   state=state, stage2=stage2)[rank]
        group.all_reduce(mine, ef_key="bucket")
        assert mine.dtype == dtype and mine.shape == want.shape
        assert torch.equal(mine, want), f"iter {it}: max diff {(mine - want).abs().max()}"
        dense = torch.stack([e.float() for e in everyone]).sum(0)
        rel = (mine.float() - dense).norm() / dense.norm()
        assert rel < {1: 2.0, 2: 1.2, 4: 0.35}[bits]


def test_config1_world2_1mi_4bit_ef_5iters():
    run_ranks(_ar_worker, 2, 1 << 20, 4, 256, 5, True, False, False, torch.float32)


@pytest.mark.parametrize("bits,numel,world", [(4, 1031, 2), (2, 4099, 3), (1, 2048, 2),
                                              (4, 777, 4)])
def test_allreduce_matches_model_odd_sizes(bits, numel, world):
    run_ranks(_ar_worker, world, numel, bits, 256, 2, False, False, False, torch.float32)


def test_allreduce_stage2_ef_and_seeded_sr_bf16():
    run_ranks(_ar_worker, 2, 5000, 4, 64, 3, True, True, True, torch.bfloat16)


def _async_worker(rank, world):
    group = LowBitGroup(bitwidth=4)
    x = _rank_input(rank, 3000)
    y = x.clone()
    work = group.all_reduce(x, async_op=True)
    assert work.wait() is True and work.is_completed()
    group.all_reduce(y)
    assert torch.equal(x, y)
    others = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(others, x)
    assert all(torch.equal(o, x) for o in others)  # every rank holds the same bits


def test_async_equals_sync_and_ranks_agree():
    run_ranks(_async_worker, 2)


def _sharded_worker(rank, world, bits, n, ef):
    group = LowBitGroup(bitwidth=bits, block_size=128, error_feedback=ef)
    rs_state, ag_state = (SimState(), SimState()) if ef else (None, None)
    for it in range(2):
        ins = [_rank_input(r, world * n, it) for r in range(world)]
        want = simulate_reduce_scatter(ins, bits, 128, state=rs_state)[rank]
        out = torch.empty(n)
        group.reduce_scatter_lowbit(out, ins[rank], ef_key="g")
        assert torch.equal(out, want)
        shards = [_rank_input(r, n, it + 7) for r in range(world)]
        want_full = simulate_all_gather(shards, bits, 128, state=ag_state)
        full = torch.empty(world * n)
        group.all_gather_lowbit(full, shards[rank], ef_key="p")
        assert torch.equal(full, want_full)


@pytest.mark.parametrize("bits,ef", [(4, False), (8, True), (2, True)])
def test_lowbit_reduce_scatter_and_all_gather(bits, ef):
    run_ranks(_sharded_worker, 2, bits, 1000, ef)


def _pipeline_worker(rank, world, local_quantize):
    # two "nodes" of two ranks; leaders are global ranks 0 and 2
    pairs = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    inter = dist.new_group([0, 2])
    local = pairs[rank // 2]
    group = LowBitGroup(bitwidth=4)
    x = _rank_input(rank, 257)
    dense = torch.stack([_rank_input(r, 257) for r in range(world)]).sum(0)
    group.all_reduce(x, local_group=local, inter_group=inter, chunk_size=63,
                     local_quantize=local_quantize)
    others = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(others, x)
    assert all((o - x).abs().max() < 1e-6 for o in others)
    err = (x - dense).abs()
    assert err.max() < 1.5 and (err.norm() / dense.norm()) < 0.2


@pytest.mark.parametrize("local_quantize", [False, True])
def test_pipeline_a_two_nodes_of_two(local_quantize):
    run_ranks(_pipeline_worker, 4, local_quantize)


def _pipeline_singleton_worker(rank, world):
    # the reference's own topology trick: local = {self}, inter = everyone
    locals_ = [dist.new_group([r]) for r in range(world)]
    group = LowBitGroup(bitwidth=4)
    x = _rank_input(rank, 257)
    flat = x.clone()
    group.all_reduce(x, local_group=locals_[rank], inter_group=dist.group.WORLD, chunk_size=63)
    # chunked flat low-bit all-reduce must equal the per-chunk model
    want = torch.cat([
        simulate_all_reduce([_rank_input(r, 257)[s:s + 63] for r in range(world)], 4, 256)[rank]
        for s in range(0, 257, 63)])
    assert torch.equal(x, want)
    assert flat.shape == x.shape


def test_pipeline_a_singleton_local_groups():
    run_ranks(_pipeline_singleton_worker, 2)


def _bucket_sync_worker(rank, world):
    from bitscom_b200.parallel.hooks import GradBucketSync

    group = LowBitGroup(bitwidth=4, error_feedback=True)
    n = 5000
    ranges = [(3000, 2000), (0, 3000)]          # backward order: last slice first
    flat = torch.zeros(n)
    sync = GradBucketSync(group, flat, ranges, mode="flat")
    states = [SimState(), SimState()]
    for it in range(3):
        everyone = [_rank_input(r, n, it) for r in range(world)]
        flat.copy_(everyone[rank])
        sync.on_ready(0)                          # slice 0 is final early ...
        sync.finish()                             # ... the rest at the end
        for idx, (start, length) in enumerate(ranges):
            want = simulate_all_reduce([e[start:start + length] for e in everyone], 4, 256,
                                       state=states[idx])[rank] * (1.0 / world)
            assert torch.equal(flat[start:start + length], want), (it, idx)


def test_grad_bucket_sync_matches_model_with_per_bucket_residuals():
    run_ranks(_bucket_sync_worker, 2)


def _counters_worker(rank, world):
    from bitscom_b200.utils import timing

    timing.reset_counters()
    group = LowBitGroup(bitwidth=4, error_feedback=True, stage2_error_feedback=True)
    n = 10_000
    for it in range(3):
        t = torch.randn(n, generator=torch.Generator().manual_seed(100 * it + rank))
        group.all_reduce(t, ef_key="bucket0")
    c = timing.counters()
    shard = -(-n // world)
    wire = (shard * 4 + 7) // 8 + 2 * -(-shard // 256)
    assert c["host_engine_calls"] == 3
    assert c["host_engine_payload_bytes"] == 3 * n * 4
    assert c["host_engine_wire_bytes"] == 3 * 2 * (world - 1) * wire
    norms = group.residual_norms()
    assert set(norms) == {"bucket0"}
    n1, n2 = norms["bucket0"]
    # 4-bit residuals of unit-variance data: non-zero, and well below the data norm
    assert 0 < n1 < 0.3 * (n ** 0.5) and 0 < n2 < 0.3 * (shard ** 0.5) * world
    plain = LowBitGroup(bitwidth=4)
    plain.all_reduce(torch.randn(64))
    assert plain.residual_norms() == {}


def test_traffic_counters_and_residual_norms():
    run_ranks(_counters_worker, 2)


# The reference's distributed all-reduce test walks five deterministic input patterns
# (tests/test_lowbit_allreduce_reference.py:24-60,167-194: linspace / random / alternating /
# small_range / sparse_spikes at 4, 2 and 1 bit, sizes 1031 / 4099 / 2048 / 512 / 777) and
# compares with a CPU simulation to 1e-4.  Here the result must equal the model bit for bit.
_PATTERNS = [("linspace", 4, 1031), ("random", 2, 4099), ("alternating", 1, 2048),
             ("small_range", 4, 512), ("sparse_spikes", 2, 777)]


def _pattern(name, rank, numel):
    if name == "linspace":
        return torch.linspace(-1.0, 1.0, numel) * (rank + 1)
    if name == "random":
        return torch.randn(numel, generator=torch.Generator().manual_seed(17 + rank))
    if name == "alternating":
        sign = torch.where(torch.arange(numel) % 2 == 0, 1.0, -1.0)
        return sign * (0.5 + 0.25 * rank)
    if name == "small_range":
        return torch.linspace(-1e-4, 1e-4, numel) + 1e-5 * rank
    x = torch.zeros(numel)
    x[:: 97 + rank] = 10.0 * (rank + 1)
    x[1::211] = -3.0
    return x


def _pattern_worker(rank, world):
    for name, bits, numel in _PATTERNS:
        everyone = [_pattern(name, r, numel) for r in range(world)]
        want = simulate_all_reduce(everyone, bits, 256)[rank]
        mine = everyone[rank].clone()
        LowBitGroup(bitwidth=bits).all_reduce(mine)
        assert torch.equal(mine, want), name
        assert torch.isfinite(mine).all()
    # stochastic rounding: two unseeded runs differ, stay finite, and all ranks agree
    base = _pattern("random", rank, 4099)
    runs = []
    for _ in range(2):
        t = base.clone()
        g = LowBitGroup(bitwidth=4, stochastic_rounding=True)
        g.all_reduce(t)
        g.check_agreement(t)
        runs.append(t)
    assert torch.isfinite(runs[0]).all() and not torch.equal(runs[0], runs[1])
    dense = torch.stack([_pattern("random", r, 4099) for r in range(world)]).sum(0)
    assert (runs[0] - dense).abs().max() < 3.0


def test_reference_input_patterns_match_the_model():
    run_ranks(_pattern_worker, 2)
