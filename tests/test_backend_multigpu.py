"""The C++ ``lowbit`` torch.distributed backend on real GPUs: ``dist.all_reduce`` on the
backend's group runs the fused kernel (with error feedback) and must equal the golden
model; the other collectives pass through to NCCL."""

import pytest
import torch
import torch.distributed as dist

from _dist import run_ranks
from bitscom_b200.parallel.simulate import (SimState, simulate_all_reduce,
                                            simulate_reduce_scatter)

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _input(rank, n, it, dtype=torch.float32):
    g = torch.Generator().manual_seed(77 + rank + 100 * it)
    return (torch.randn(n, generator=g) * 1e-2).to(dtype)


def _worker(rank, world, n):
    import bitscom_b200
    from bitscom_b200 import LowBitGroup

    assert dist.get_backend() == "lowbit"
    pg = dist.distributed_c10d._get_default_group()
    backend = pg._get_backend(torch.device("cuda"))
    state = SimState()
    grad = torch.empty(n, device="cuda")          # persistent bucket: residuals carry over
    for it in range(3):
        everyone = [_input(r, n, it) for r in range(world)]
        want = simulate_all_reduce(everyone, 4, 256, state=state, stage2=True)[rank]
        grad.copy_(everyone[rank])
        if it == 1:
            dist.all_reduce(grad, async_op=True).wait()
        else:
            dist.all_reduce(grad)
        torch.cuda.synchronize()
        assert torch.equal(grad.cpu(), want), f"iter {it}"
    assert backend.fused_launches() == 3
    assert len(backend.residual_state()) == 1

    # non-SUM goes dense through NCCL
    t = torch.full((8,), float(rank + 1), device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t[0].item() == world

    # broadcast / all_gather pass through
    b = torch.full((4,), float(rank), device="cuda")
    dist.broadcast(b, src=world - 1)
    assert b[0].item() == world - 1
    outs = [torch.empty(4, device="cuda") for _ in range(world)]
    dist.all_gather(outs, torch.full((4,), float(rank), device="cuda"))
    assert [o[0].item() for o in outs] == list(range(world))

    # low-bit reduce_scatter (tensor form)
    S = 4096
    ins = [_input(r, world * S, 9) for r in range(world)]
    want = simulate_reduce_scatter(ins, 4, 256)[rank]
    out = torch.empty(S, device="cuda")
    dist.reduce_scatter_tensor(out, ins[rank].cuda())
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), want)

    # scheduled-handle API and the LowBitGroup wrapper that delegates to the backend
    group = LowBitGroup(bitwidth=4, backend_allreduce=True)
    x = _input(rank, 2048, 5).cuda()
    handle = backend.schedule_lowbit_allreduce(x)
    assert group.launch_lowbit_phase2(handle) and group.launch_lowbit_restore(handle)
    handle.block_current_stream()
    assert handle.wait() and handle.is_completed()
    assert group.progress_lowbit(True) is True
    y = _input(rank, 2048, 5).cuda()
    group.all_reduce(y)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    assert bitscom_b200.is_extension_available()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_lowbit_backend_on_gpus(world):
    _need(world)
    run_ranks(_worker, world, 100003, backend="lowbit",
              lowbit_options=dict(bitwidth=4, error_feedback_mode="ef21_plus",
                                  stage2_error_feedback=True))
