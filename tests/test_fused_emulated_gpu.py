"""The fused collective kernel with all ranks emulated on ONE GPU (CTA groups of one
cooperative launch play the ranks), compared bit for bit with the golden model."""

import pytest
import torch

from bitscom_b200.parallel.simulate import (SimState, simulate_all_gather,
                                            simulate_all_reduce, simulate_reduce_scatter)

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.parallel import fused


def _inputs(world, n, dtype, scale=1e-2, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, generator=g) * scale).to(dtype) for _ in range(world)]


@pytest.fixture(params=["three-phase", "flag-in-data"])
def make_world(request):
    """Every test runs twice: with the small-bucket form (packed words that carry their own
    arrival flags, taken by 4- and 8-bit all-reduces that fit its slots) switched off, and with
    the library's default threshold."""
    worlds = []
    ll_max_bytes = 0 if request.param == "three-phase" else None

    def make(world, region_bytes=8 << 20, timeout_ms=5000.0):
        w = fused.EmulatedWorld(world, "cuda:0", region_bytes, timeout_ms,
                                ll_max_bytes=ll_max_bytes)
        worlds.append(w)
        return w

    yield make
    torch.cuda.synchronize()
    try:
        for w in worlds:
            w.check_canaries()  # no store landed outside the regions of any rank's block
    finally:
        for w in worlds:
            w.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype,n", [(torch.float32, 8192), (torch.float32, 4099),
                                     (torch.bfloat16, 65536), (torch.float16, 1031)])
def test_all_reduce_bit_exact(make_world, world, bits, dtype, n):
    w = make_world(world)
    ins = _inputs(world, n, dtype, seed=n + bits)
    want = simulate_all_reduce(ins, bits, 256)
    dev = [t.cuda() for t in ins]
    w.all_reduce(dev, bitwidth=bits, block_size=256)
    torch.cuda.synchronize()
    assert all(s[0] == 0 for s in w.status())
    for r in range(world):
        assert torch.equal(dev[r].cpu(), want[r]), f"rank {r}"


@pytest.mark.parametrize("block", [8, 32, 64, 128])
def test_all_reduce_other_block_sizes(make_world, block):
    w = make_world(4)
    ins = _inputs(4, 10000, torch.float32, seed=block)
    want = simulate_all_reduce(ins, 4, block)
    dev = [t.cuda() for t in ins]
    w.all_reduce(dev, bitwidth=4, block_size=block)
    assert torch.equal(dev[2].cpu(), want[2])


@pytest.mark.parametrize("stochastic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_error_feedback_two_stages_over_iterations(make_world, stochastic, dtype):
    world, n, bits = 4, 20000, 2
    w = make_world(world)
    S = -(-n // world)
    res1 = [torch.zeros(S * world, device="cuda") for _ in range(world)]
    res2 = [torch.zeros(S, device="cuda") for _ in range(world)]
    state = SimState()
    for it in range(4):
        ins = _inputs(world, n, dtype, seed=100 + it)
        seed = 7000 + it if stochastic else None
        want = simulate_all_reduce(ins, bits, 256, stochastic=stochastic, seed=seed,
                                   state=state, stage2=True, post_scale=0.25)
        dev = [t.cuda() for t in ins]
        w.all_reduce(dev, bitwidth=bits, block_size=256, stochastic=stochastic, seed=seed,
                     res1=res1, res2=res2, post_scale=0.25)
        for r in range(world):
            assert torch.equal(dev[r].cpu(), want[r]), f"iter {it} rank {r}"
            assert torch.equal(res1[r].cpu(), state.stage1[r])
            assert torch.equal(res2[r].cpu(), state.stage2[r])


def test_chunked_launches_match_single_pass(make_world):
    # a region so small that the bucket needs several launches per call
    world, n = 2, 300000
    w = make_world(world, region_bytes=64 << 10)
    assert w.max_chunk(4, 256) * world < n
    ins = _inputs(world, n, torch.float32, seed=5)
    want = simulate_all_reduce(ins, 4, 256)
    dev = [t.cuda() for t in ins]
    w.all_reduce(dev, bitwidth=4, block_size=256)
    assert torch.equal(dev[0].cpu(), want[0]) and torch.equal(dev[1].cpu(), want[1])


@pytest.mark.parametrize("bits", [4, 8])
def test_reduce_scatter_and_all_gather(make_world, bits):
    world, S = 4, 5000
    w = make_world(world)
    ins = _inputs(world, world * S, torch.bfloat16, seed=bits)
    want = simulate_reduce_scatter(ins, bits, 128)
    outs = [torch.empty(S, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    w.reduce_scatter(outs, [t.cuda() for t in ins], bitwidth=bits, block_size=128)
    for r in range(world):
        assert torch.equal(outs[r].cpu(), want[r])
    shards = _inputs(world, S, torch.float32, seed=bits + 1)
    res2 = [torch.zeros(S, device="cuda") for _ in range(world)]
    state = SimState()
    for it in range(2):
        want_full = simulate_all_gather(shards, bits, 128, state=state)
        fulls = [torch.empty(world * S, device="cuda") for _ in range(world)]
        w.all_gather(fulls, [t.cuda() for t in shards], bitwidth=bits, block_size=128,
                     res2=res2)
        for r in range(world):
            assert torch.equal(fulls[r].cpu(), want_full)


def test_phase_time_stamps_are_ordered_and_add_up(make_world):
    """Every rank's first CTA stamps the device timer at its phase boundaries; after a launch
    the five intervals are non-negative, sum to the total, and a reduce-scatter leaves the
    third phase empty."""
    world, n = 4, 1 << 20
    w = make_world(world, region_bytes=16 << 20)
    bufs = [t.cuda() for t in _inputs(world, n, torch.float32)]
    w.all_reduce(bufs, bitwidth=4, block_size=256)
    torch.cuda.synchronize()
    for phases in w.phase_times_us():
        parts = [phases[k] for k in ("phase1", "wait1", "phase2", "wait2", "phase3")]
        assert all(v >= 0 for v in parts) and phases["phase1"] > 0 and phases["phase3"] > 0
        assert abs(sum(parts) - phases["total"]) < 1e-3
        assert phases["total"] < 50_000     # microseconds: a 4 MB bucket, not a timeout
    outs = [torch.empty(n // world, device="cuda") for _ in range(world)]
    w.reduce_scatter(outs, bufs, bitwidth=4, block_size=256)
    torch.cuda.synchronize()
    # the last two stamps of a reduce-scatter are taken back to back: a timer tick at most
    assert all(p["phase3"] < 1.0 and p["phase1"] > 0 for p in w.phase_times_us())


def test_back_to_back_calls_need_no_barrier(make_world):
    w = make_world(4)
    ins = _inputs(4, 50000, torch.float32, seed=9)
    dev = [t.cuda() for t in ins]
    cur = [t.clone() for t in ins]
    for _ in range(5):
        w.all_reduce(dev, bitwidth=4, block_size=256, post_scale=0.25)
        cur = simulate_all_reduce(cur, 4, 256, post_scale=0.25)
    assert torch.equal(dev[1].cpu(), cur[1])


def test_peer_that_never_arrives_times_out_with_status(make_world):
    """Only rank 0 launches: its wait on rank 1's flag runs out, the kernel records who it
    waited for and returns; the context stays usable and the communicator re-arms."""
    import ctypes

    w = make_world(2, timeout_ms=200.0)
    x = torch.ones(4096, device="cuda")
    args = fused._args(x, x, None, None, 4096, 2048, x.dtype, 4, 256,
                       fused.MODE_ALL_REDUCE, False, None, 1.0, 0, 0)
    rc = w.lib.bcom_collective(w.comms[0].handle, ctypes.byref(args),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    st = w.comms[0].status()
    assert st[0] == 1 and st[2] == 1 and st[3] == 0  # phase-1 flags, waited on peer 1
    assert "peer 1" in fused._describe(st)
    assert float((x + 1).sum()) == 2 * 4096  # device still answers
    # the two ranks now disagree on the epoch: re-arm, drop this world, build a new one
    w.reset()
    w2 = make_world(2)
    ins = _inputs(2, 4096, torch.float32, seed=1)
    dev = [t.cuda() for t in ins]
    w2.all_reduce(dev, bitwidth=4, block_size=256)
    assert torch.equal(dev[0].cpu(), simulate_all_reduce(ins, 4, 256)[0])
