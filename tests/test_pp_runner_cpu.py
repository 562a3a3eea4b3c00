"""The 1F1B runner executed for real on CPU ranks (gloo point-to-point): a stack of small
layers split over pipeline stages gives the same losses and the same parameter gradients as
the unsplit model run micro-batch by micro-batch in one process."""

import pytest
import torch
import torch.distributed as dist

from bitscom_b200.parallel.deferred import DeferredWork
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


class _DeferringLinear(torch.autograd.Function):
    """A linear layer whose weight gradient goes to ``weight.main_grad`` and is queued when a
    ``DeferredWork`` context is active: the CPU twin of ``ops.gemm.LinearFunction``."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return x @ weight.t()

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        queue = DeferredWork.active()
        work = lambda: weight.main_grad.add_(dy.t() @ x)  # noqa: E731
        if queue is not None:
            queue.add(work)
            _LOG.append("queued")
        else:
            work()
            _LOG.append("now")
        return dy @ weight, None


_LOG = []


def _deferral_worker(rank, world, microbatches, defer):
    defer, defer_last = bool(defer), defer == "all"
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(50 + rank)
    weights = [torch.nn.Parameter(torch.randn(WIDTH, WIDTH, generator=g) * 0.3) for _ in range(2)]
    for w in weights:
        w.main_grad = torch.zeros_like(w)
    runner = PipelineRunner(rank, world, dist.group.WORLD, rank - 1 if rank > 0 else None,
                            rank + 1 if rank < world - 1 else None, (MB_ROWS, WIDTH),
                            dtype=torch.float32, device="cpu", defer_wgrad=defer,
                            defer_last=defer_last)
    sent_before_flush = []
    real_exchange = runner._exchange

    def spy(comm, to_next=None, to_prev=None, between=None):
        def wrapped():
            sent_before_flush.append(to_prev is not None)
            between()
        return real_exchange(comm, to_next, to_prev, between=wrapped if between else None)

    runner._exchange = spy

    def forward_fn(mb, x):
        inp, tgt = _micro_batch(mb)
        h = inp if rank == 0 else x
        for w in weights:
            h = torch.tanh(_DeferringLinear.apply(h, w))
        return torch.nn.functional.mse_loss(h, tgt) / microbatches if rank == world - 1 else h

    runner.run(microbatches, forward_fn)
    grads = torch.stack([w.main_grad for w in weights])
    everyone = [torch.empty_like(grads) for _ in range(world)]
    dist.all_gather(everyone, grads)
    # reference: the same stack of layers, unsplit, plain autograd
    ws = []
    for r in range(world):
        gr = torch.Generator().manual_seed(50 + r)
        ws += [(torch.randn(WIDTH, WIDTH, generator=gr) * 0.3).requires_grad_() for _ in range(2)]
    for mb in range(microbatches):
        inp, tgt = _micro_batch(mb)
        h = inp
        for w in ws:
            h = torch.tanh(h @ w.t())
        (torch.nn.functional.mse_loss(h, tgt) / microbatches).backward()
    want = torch.stack([w.grad for w in ws]).view(world, 2, WIDTH, WIDTH)
    for r in range(world):
        assert torch.allclose(everyone[r], want[r], atol=1e-5), r
    if defer:
        # every backward step but the last one queued its two weight gradients; with
        # defer_last the last one did too
        if defer_last:
            assert _LOG.count("queued") == 2 * microbatches and _LOG.count("now") == 0
        else:
            assert _LOG.count("queued") == 2 * (microbatches - 1) and _LOG.count("now") == 2
        if rank > 0:  # ... and ran them only after the input gradient was handed over
            assert sent_before_flush and all(sent_before_flush)
    else:
        assert _LOG.count("queued") == 0


@pytest.mark.parametrize("stages,microbatches,defer", [(2, 4, True), (2, 4, False),
                                                       (3, 5, "all"), (3, 5, True)])
def test_deferred_weight_gradients_match_and_follow_the_send(stages, microbatches, defer):
    run_ranks(_deferral_worker, stages, microbatches, defer)


def test_deferred_work_context_rules():
    q = DeferredWork()
    ran = []
    with q:
        assert DeferredWork.active() is q
        q.add(lambda: ran.append(1))
        q.add(lambda: ran.append(2))
        with pytest.raises(RuntimeError):
            with DeferredWork():
                pass
    assert DeferredWork.active() is None and ran == [] and len(q) == 2
    q.flush()
    assert ran == [1, 2] and len(q) == 0 and q.flushes == 1
    q.flush()
    assert q.flushes == 1
    with pytest.raises(ValueError):
        with q:
            q.add(lambda: ran.append(3))
            raise ValueError("step failed")
    assert len(q) == 0 and ran == [1, 2]      # a failed step drops its queue
