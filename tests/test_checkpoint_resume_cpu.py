"""Exact resume on CPU ranks: a run that is checkpointed (weights, optimizer, error-feedback
residuals, stochastic-rounding counter), torn down and resumed follows the uninterrupted run
bit for bit; dropping the low-bit state from the checkpoint does not."""

import torch
import torch.distributed as dist

from bitscom_b200 import LowBitGroup
from bitscom_b200.utils.checkpoint import load_checkpoint, save_checkpoint

from _dist import run_ranks


def _make():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 8))
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    group = LowBitGroup(bitwidth=4, stochastic_rounding=True, sr_seed=11, error_feedback=True,
                        stage2_error_feedback=True)
    return model, opt, group


def _step(model, opt, group, step, rank, world):
    g = torch.Generator().manual_seed(1000 * step + rank)
    x, y = torch.randn(16, 32, generator=g), torch.randn(16, 8, generator=g)
    opt.zero_grad(set_to_none=True)
    torch.nn.functional.mse_loss(model(x), y).backward()
    for i, p in enumerate(model.parameters()):
        group.all_reduce(p.grad, ef_key=("p", i))
        p.grad.div_(world)
    opt.step()


def _flat(model):
    return torch.cat([p.detach().reshape(-1) for p in model.parameters()])


def _worker(rank, world, tmp):
    # uninterrupted run
    model, opt, group = _make()
    for step in range(8):
        _step(model, opt, group, step, rank, world)
    want = _flat(model).clone()

    # run, checkpoint after 4 steps, throw everything away, resume
    model, opt, group = _make()
    for step in range(4):
        _step(model, opt, group, step, rank, world)
    save_checkpoint(tmp, {"model": model.state_dict(), "opt": opt.state_dict(),
                          "lowbit": group.state_dict(), "step": 4}, rank)
    del model, opt, group
    dist.barrier()
    ckpt = load_checkpoint(tmp, rank)
    model, opt, group = _make()
    model.load_state_dict(ckpt["model"])
    opt.load_state_dict(ckpt["opt"])
    group.load_state_dict(ckpt["lowbit"])
    for step in range(ckpt["step"], 8):
        _step(model, opt, group, step, rank, world)
    assert torch.equal(_flat(model), want), "resumed run left the trajectory"

    # without the residuals and the rounding counter the run diverges (slightly)
    model, opt, group = _make()
    model.load_state_dict(ckpt["model"])
    opt.load_state_dict(ckpt["opt"])
    for step in range(ckpt["step"], 8):
        _step(model, opt, group, step, rank, world)
    assert not torch.equal(_flat(model), want)
    assert torch.allclose(_flat(model), want, atol=0.05)


def test_checkpointed_run_resumes_bit_exactly(tmp_path):
    run_ranks(_worker, 2, str(tmp_path))
