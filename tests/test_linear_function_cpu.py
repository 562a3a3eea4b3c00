"""The autograd logic of ``ops.gemm.LinearFunction`` on CPU, with the tcgen05 GEMM replaced by
a torch matmul of the same calling convention: forward, input gradient, weight gradient into
``main_grad`` or returned, and the deferred weight-gradient queue."""

import pytest
import torch

from bitscom_b200.ops import gemm as G
from bitscom_b200.parallel.deferred import DeferredWork


def _fake_gemm(a, b, *, a_mn_major=False, b_mn_major=False, out=None,
               out_dtype=torch.bfloat16, accumulate=False, max_ctas=0, residual=None):
    A = a.t() if a_mn_major else a          # [M, K]
    B = b if b_mn_major else b.t()          # [K, N]
    c = A.float() @ B.float()
    if residual is not None:
        c = c + residual.float()
    if out is None:
        return c.to(out_dtype)
    if accumulate:
        out.add_(c.to(out.dtype))
    else:
        out.copy_(c.to(out.dtype))
    return out


@pytest.fixture
def fake_gemm(monkeypatch):
    monkeypatch.setattr(G, "gemm", _fake_gemm)


def _case(main_grad):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 6, 16, generator=g).to(torch.bfloat16).requires_grad_()
    w = torch.nn.Parameter((torch.randn(24, 16, generator=g) * 0.2).to(torch.bfloat16))
    if main_grad:
        w.main_grad = torch.full((24, 16), 0.5)
    dy = torch.randn(2, 6, 24, generator=g).to(torch.bfloat16)
    return x, w, dy


@pytest.mark.parametrize("main_grad", [True, False])
def test_forward_and_gradients(fake_gemm, main_grad):
    x, w, dy = _case(main_grad)
    y = G.linear(x, w)
    assert y.shape == (2, 6, 24) and y._base is None           # not a view
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    assert torch.allclose(y.float(), (xr @ wr.t()).detach(), atol=0.05)
    assert torch.allclose(x.grad.float(), xr.grad, atol=0.05)
    if main_grad:
        assert w.grad is None
        assert torch.allclose(w.main_grad - 0.5, wr.grad, atol=0.05)
    else:
        assert torch.allclose(w.grad.float(), wr.grad, atol=0.1)


def test_residual_is_added_in_the_gemm_and_its_gradient_is_the_output_gradient(fake_gemm):
    x, w, dy = _case(True)
    res = torch.randn(2, 6, 24, generator=torch.Generator().manual_seed(5)).to(
        torch.bfloat16).requires_grad_()
    y = G.linear(x, w, residual=res)
    want = res.detach().float() + x.detach().float() @ w.detach().float().t()
    assert torch.allclose(y.float(), want, atol=0.05)
    y.backward(dy)
    assert torch.equal(res.grad, dy)
    assert x.grad is not None and w.grad is None


def test_rmsnorm_fork_adds_the_residual_gradient_inside_the_norm_backward():
    from bitscom_b200.ops import nn as K

    g = torch.Generator().manual_seed(11)
    x = torch.randn(10, 32, generator=g).to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * torch.randn(32, generator=g)).to(torch.bfloat16).requires_grad_()
    h, xr = K.rmsnorm_fork(x, w)
    (h.float().sum() * 2 + (xr.float() * 3).sum()).backward()
    x2 = x.detach().clone().requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    h2 = K.rmsnorm(x2, w2)
    (h2.float().sum() * 2 + (x2.float() * 3).sum()).backward()
    assert torch.equal(h, h2)
    assert torch.allclose(x.grad.float(), x2.grad.float(), atol=0.05)
    assert torch.allclose(w.grad.float(), w2.grad.float(), atol=0.05)
    # the residual branch alone
    x3 = x.detach().clone().requires_grad_()
    _, only = K.rmsnorm_fork(x3, w.detach())
    only.float().sum().backward()
    assert torch.equal(x3.grad, torch.ones_like(x3))


def test_deferred_weight_gradient_runs_at_flush(fake_gemm):
    x, w, dy = _case(True)
    queue = DeferredWork()
    with queue:
        G.linear(x, w).backward(dy)
    assert len(queue) == 1 and x.grad is not None
    assert torch.equal(w.main_grad, torch.full((24, 16), 0.5))   # nothing accumulated yet
    queue.flush()
    want = dy.float().reshape(-1, 24).t() @ x.detach().float().reshape(-1, 16)
    assert torch.allclose(w.main_grad - 0.5, want, atol=0.05)
    # weights without a flat gradient buffer are never deferred
    x2, w2, dy2 = _case(False)
    with DeferredWork() as q2:
        G.linear(x2, w2).backward(dy2)
    assert len(q2) == 0 and w2.grad is not None
