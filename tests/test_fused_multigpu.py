"""Fused collectives across real GPUs (one process per GPU, NCCL for the plumbing).

The golden model (``parallel/simulate.py``: the wire protocol replayed with the host quantizer)
runs ONCE, in the parent, and every rank loads its inputs and its expected bits from a file:
W ranks that each replay W quantizers compete for the same cores and tell nothing new."""

import os
import tempfile

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


def _golden(folder, world, n, bits, dtype, iters, stochastic=True):
    """Per rank: ``{"inputs": [iters tensors], "wants": [iters tensors]}`` in
    ``folder/rank<r>.pt``.  Seeds follow ``LowBitGroup._next_sr_seed`` for ``sr_seed=5``."""
    state = SimState()
    per_rank = [{"inputs": [], "wants": []} for _ in range(world)]
    for it in range(iters):
        everyone = [_input(r, n, it, dtype) for r in range(world)]
        seed = (5 * 0x9E3779B97F4A7C15 + it + 1) & 0xFFFFFFFFFFFFFFFF
        outs = simulate_all_reduce(everyone, bits, 256, stochastic=stochastic,
                                   seed=seed if stochastic else None, state=state, stage2=True)
        for r in range(world):
            per_rank[r]["inputs"].append(everyone[r])
            per_rank[r]["wants"].append(outs[r].clone())
    for r in range(world):
        torch.save(per_rank[r], os.path.join(folder, f"rank{r}.pt"))


def _run_with_golden(worker, world, n, bits, dtype, iters, stochastic=True, **kw):
    with tempfile.TemporaryDirectory() as folder:
        _golden(folder, world, n, bits, dtype, iters, stochastic)
        run_ranks(worker, world, folder, n, bits, dtype, iters, backend="nccl", **kw)


def _worker(rank, world, folder, n, bits, dtype, iters):
    from bitscom_b200 import LowBitGroup

    gold = torch.load(os.path.join(folder, f"rank{rank}.pt"))
    group = LowBitGroup(bitwidth=bits, error_feedback=True, stage2_error_feedback=True,
                        stochastic_rounding=True, sr_seed=5, fused=True)
    for it in range(iters):
        want = gold["wants"][it]
        x = gold["inputs"][it].cuda()
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
    assert torch.isfinite(rel)
    if bits > 1:  # the 1-bit code keeps magnitudes only: no meaningful distance to the dense sum
        assert rel < {2: 2.5, 4: 0.5}[bits], rel


# "three-phase": the small-bucket form (packed words that carry their own arrival flags) is
# switched off, so the 4 MB fp32 case runs through the three phases and their two flag
# handshakes; "default": it takes the small-bucket form.  The other case of each test (odd
# length, or 1- / 2-bit codes) runs through the three phases either way.
FORMS = [("three-phase", "0"), ("default", "")]


def _form(monkeypatch, form):
    if form[1]:
        monkeypatch.setenv("BITSCOM_LL_MAX_MB", form[1])
    else:
        monkeypatch.delenv("BITSCOM_LL_MAX_MB", raising=False)


@pytest.mark.parametrize("form", FORMS, ids=[f[0] for f in FORMS])
@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (2, torch.bfloat16, 300001)])
def test_two_gpu_all_reduce_bit_exact(bits, dtype, n, form, monkeypatch):
    _need(2)
    if bits != 4 and form[0] == "default":
        pytest.skip("same path as three-phase for this case")
    _form(monkeypatch, form)
    _run_with_golden(_worker, 2, n, bits, dtype, 3)


@pytest.mark.parametrize("form", FORMS, ids=[f[0] for f in FORMS])
@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (1, torch.bfloat16, 300001)])
def test_four_gpu_all_reduce_bit_exact(bits, dtype, n, form, monkeypatch):
    _need(4)
    if bits != 4 and form[0] == "default":
        pytest.skip("same path as three-phase for this case")
    _form(monkeypatch, form)
    _run_with_golden(_worker, 4, n, bits, dtype, 3)


@pytest.mark.parametrize("form", FORMS, ids=[f[0] for f in FORMS])
@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (4, torch.bfloat16, 3000001)])
def test_eight_gpu_all_reduce_bit_exact(bits, dtype, n, form, monkeypatch):
    _need(8)
    if n % 8 and form[0] == "default":
        pytest.skip("same path as three-phase for this case")
    _form(monkeypatch, form)
    _run_with_golden(_worker, 8, n, bits, dtype, 3)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("bits,dtype,n", [(4, torch.float32, 1 << 20),
                                          (8, torch.bfloat16, 300032)])
def test_all_reduce_bit_exact_over_nvls(world, bits, dtype, n, monkeypatch):
    """The same bit-exact check with the all-gather half on multimem stores (the children
    inherit the environment).  Not for failure tests: a rank that dies while its memory is
    bound to a multicast object can fault its peers."""
    _need(world)
    monkeypatch.setenv("BITSCOM_NVLS", "1")
    monkeypatch.setenv("BITSCOM_REQUIRE_NVLS", "1")
    monkeypatch.setenv("BITSCOM_LL_MAX_MB", "0")   # small buckets would bypass the multimem stores
    _run_with_golden(_worker8 if bits == 8 else _worker, world, n, bits, dtype, 3,
                     stochastic=bits != 8)


def _worker8(rank, world, folder, n, bits, dtype, iters):
    """8-bit goes through the communicator directly (LowBitGroup all-reduces 8-bit densely)."""
    from bitscom_b200.api import ErrorFeedbackState
    from bitscom_b200.parallel.fused import FusedLowBitComm

    gold = torch.load(os.path.join(folder, f"rank{rank}.pt"))
    comm = FusedLowBitComm.for_group(dist.group.WORLD, torch.device("cuda", rank))
    assert comm.multicast or not os.environ.get("BITSCOM_REQUIRE_NVLS")
    ef = ErrorFeedbackState()
    for it in range(iters):
        want = gold["wants"][it]
        x = gold["inputs"][it].cuda()
        comm.all_reduce(x, bitwidth=bits, block_size=256, ef=ef, stage2=True)
        torch.cuda.synchronize()
        assert torch.equal(x.cpu(), want), f"rank {rank} iter {it}"
    comm.check_status()
    torch.distributed.barrier()  # every peer's pushes have landed
    comm.check_canaries()
