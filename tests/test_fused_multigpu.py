"""Fused collectives across real GPUs (one process per GPU, NCCL for the plumbing)."""

import os

import pytest
import torch
import torch.distributed as dist

from _dist import run_ranks
from bitscom_b200.parallel.simulate import SimState, simulate_all_reduce

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _input(rank, n, it, dtype):
    g = torch.Generator().manual_seed(1234 + rank + 1000 * it)
    return (torch.randn(n, generator=g) * 1e-3).to(dtype)


def _worker(rank, world, n, bits, dtype, iters):
    from bitscom_b200 import LowBitGroup

    torch.set_num_threads(1)  # every rank replays the golden model on the CPU

    group = LowBitGroup(bitwidth=bits, error_feedback=True, stage2_error_feedback=True,
                        stochastic_rounding=True, sr_seed=5, fused=True)
    state = SimState()
    for it in range(iters):
        everyone = [_input(r, n, it, dtype) for r in range(world)]
        seed = (5 * 0x9E3779B97F4A7C15 + it + 1) & 0xFFFFFFFFFFFFFFFF
        want = simulate_all_reduce(everyone, bits, 256, stochastic=True, seed=seed,
                                   state=state, stage2=True)[rank]
        x = everyone[rank].cuda()
        if it % 2:
            group.all_reduce(x, async_op=True, ef_key="b").wait()
        else:
            group.all_reduce(x, ef_key="b")
        torch.cuda.synchronize()
        assert torch.equal(x.cpu(), want), f"rank {rank} iter {it}"
    comm = group._fused_comms[id(group.pg)]
    assert comm.launches == iters
    comm.check_status()
    torch.distributed.barrier()  # every peer's pushes have landed
    comm.check_canaries()
    if os.environ.get("BITSCOM_NVLS", "0") == "1" and os.environ.get("BITSCOM_REQUIRE_NVLS"):
        assert comm.multicast, "the NVLS path was asked for but not set up"
    # stream-ordered variant with fused post-scale
    y = _input(rank, n, 99, dtype).cuda()
    side = torch.cuda.Stream()
    work = group.all_reduce_stream(y, stream=side, post_scale=1.0 / world, ef_key="c")
    work.block_current_stream()
    assert work.wait() and torch.isfinite(y.float()).all()
    # low-bit reduce-scatter + all-gather round trip
    S = 4096
    full = _input(rank, world * S, 7, dtype).cuda()
    shard = torch.empty(S, dtype=dtype, device="cuda")
    group.reduce_scatter_lowbit(shard, full)
    back = torch.empty_like(full)
    group.all_gather_lowbit(back, shard)
    torch.cuda.synchronize()
    dense = full.float().clone()
    dist.all_reduce(dense)
    rel = (back.float() - dense).norm() / dense.norm()
    assert rel < {2: 2.5, 4: 0.5}[bits], rel


@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (2, torch.bfloat16, 300001)])
def test_two_gpu_all_reduce_bit_exact(bits, dtype, n):
    _need(2)
    run_ranks(_worker, 2, n, bits, dtype, 3, backend="nccl")


def test_all_gpus_all_reduce_bit_exact():
    n_gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n_gpus < 4:
        pytest.skip("needs 4 or more GPUs")
    run_ranks(_worker, n_gpus, 1 << 17, 4, torch.float32, 2, backend="nccl", timeout=600)


@pytest.mark.skipif(os.environ.get("BITSCOM_EXPERIMENTAL", "0") != "1",
                    reason="the NVLS (multimem) path has not been run on GPUs yet; "
                           "set BITSCOM_EXPERIMENTAL=1 to try it")
@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (8, torch.bfloat16, 300032)])
def test_two_gpu_all_reduce_bit_exact_over_nvls(bits, dtype, n, monkeypatch):
    """The same bit-exact check with the all-gather half on multimem stores (the children
    inherit the environment).  Not for failure tests: a rank that dies while its memory is
    bound to a multicast object can fault its peers."""
    _need(2)
    monkeypatch.setenv("BITSCOM_NVLS", "1")
    monkeypatch.setenv("BITSCOM_REQUIRE_NVLS", "1")
    run_ranks(_worker8 if bits == 8 else _worker, 2, n, bits, dtype, 3, backend="nccl")


def _worker8(rank, world, n, bits, dtype, iters):
    """8-bit goes through the communicator directly (LowBitGroup all-reduces 8-bit densely)."""
    from bitscom_b200.api import ErrorFeedbackState
    from bitscom_b200.parallel.fused import FusedLowBitComm

    torch.set_num_threads(1)
    comm = FusedLowBitComm.for_group(dist.group.WORLD, torch.device("cuda", rank))
    assert comm.multicast or not os.environ.get("BITSCOM_REQUIRE_NVLS")
    state, ef = SimState(), ErrorFeedbackState()
    for it in range(iters):
        everyone = [_input(r, n, it, dtype) for r in range(world)]
        want = simulate_all_reduce(everyone, bits, 256, state=state, stage2=True)[rank]
        x = everyone[rank].cuda()
        comm.all_reduce(x, bitwidth=bits, block_size=256, ef=ef, stage2=True)
        torch.cuda.synchronize()
        assert torch.equal(x.cpu(), want), f"rank {rank} iter {it}"
    comm.check_status()
    torch.distributed.barrier()  # every peer's pushes have landed
    comm.check_canaries()
