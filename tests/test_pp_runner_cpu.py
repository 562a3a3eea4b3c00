"""The 1F1B runner executed for real on CPU ranks (gloo point-to-point): a stack of small
layers split over pipeline stages gives the same losses and the same parameter gradients as
the unsplit model run micro-batch by micro-batch in one process."""

import pytest
import torch
import torch.distributed as dist

from bitscom_b200.parallel.pp_schedule import PipelineRunner

from _dist import run_ranks

WIDTH, LAYERS_PER_STAGE, MB_ROWS = 16, 2, 4


def _stage_layers(stage):
    g = torch.Generator().manual_seed(100 + stage)
    layers = []
    for _ in range(LAYERS_PER_STAGE):
        lin = torch.nn.Linear(WIDTH, WIDTH)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(WIDTH, WIDTH, generator=g) * 0.3)
            lin.bias.copy_(torch.randn(WIDTH, generator=g) * 0.1)
        layers += [lin, torch.nn.Tanh()]
    return torch.nn.Sequential(*layers)


def _micro_batch(mb):
    g = torch.Generator().manual_seed(7 + mb)
    return torch.randn(MB_ROWS, WIDTH, generator=g), torch.randn(MB_ROWS, WIDTH, generator=g)


def _reference(stages, microbatches):
    model = torch.nn.Sequential(*[_stage_layers(s) for s in range(stages)])
    losses = []
    for mb in range(microbatches):
        x, y = _micro_batch(mb)
        loss = torch.nn.functional.mse_loss(model(x), y) / microbatches
        loss.backward()
        losses.append(loss.detach())
    return losses, [[p.grad.clone() for p in model[s].parameters()] for s in range(stages)]


def _worker(rank, world, microbatches):
    torch.manual_seed(0)
    torch.set_num_threads(1)
    net = _stage_layers(rank)
    runner = PipelineRunner(rank, world, dist.group.WORLD, rank - 1 if rank > 0 else None,
                            rank + 1 if rank < world - 1 else None, (MB_ROWS, WIDTH),
                            dtype=torch.float32, device="cpu")
    fired = []

    def forward_fn(mb, x):
        inp, tgt = _micro_batch(mb)
        h = net(inp if rank == 0 else x)
        if rank == world - 1:
            return torch.nn.functional.mse_loss(h, tgt) / microbatches
        return h

    losses = runner.run(microbatches, forward_fn, on_last_backward=lambda: fired.append(1))
    want_losses, want_grads = _reference(world, microbatches)
    assert fired == [1]
    if rank == world - 1:
        assert len(losses) == microbatches
        for a, b in zip(losses, want_losses):
            assert torch.allclose(a, b, atol=1e-6)
    else:
        assert losses == []
    for p, g in zip(net.parameters(), want_grads[rank]):
        assert torch.allclose(p.grad, g, atol=1e-5), (rank, (p.grad - g).abs().max())


@pytest.mark.parametrize("stages,microbatches", [(2, 4), (3, 5), (4, 4), (2, 1)])
def test_1f1b_runner_matches_unsplit_model(stages, microbatches):
    run_ranks(_worker, stages, microbatches)
