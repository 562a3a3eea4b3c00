"""Trainer kernels (RMSNorm, LayerNorm, RoPE, SwiGLU, bias + GELU, cross-entropy, embedding,
AdamW, SGD) against
plain PyTorch fp32 references of the same ops."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.ops import nn as K


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _close(a, b, rtol=2e-2, atol=2e-2):
    assert torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol), \
        f"max diff {(a.float() - b.float()).abs().max().item()}"


@pytest.mark.parametrize("rows,H", [(64, 256), (300, 4096), (7, 8192), (1000, 1024),
                                    (4097, 4096), (5, 8), (33, 16384)])
def test_rmsnorm_fwd_bwd(rows, H):
    x = _bf(rows, H, seed=1).requires_grad_()
    w = (1 + 0.1 * _bf(H, seed=2).float()).to(torch.bfloat16).requires_grad_()
    dy = _bf(rows, H, seed=3)
    y = K.rmsnorm(x, w, 1e-5)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad, atol=3e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=3e-2, atol=0.02 * rows ** 0.5 + 0.05)
    # fp32 main_grad accumulation
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(H, device="cuda")
    K.rmsnorm(x.detach(), w2, 1e-5).backward(dy)
    assert w2.grad is None
    assert torch.allclose(w2.main_grad, wr.grad, rtol=2e-2, atol=0.01 * rows ** 0.5 + 0.02)


def test_rmsnorm_fork_adds_the_residual_gradient_in_the_kernel():
    """``rmsnorm_fork`` returns (norm(x), x); in backward the gradient of the residual branch is
    added to the norm's input gradient inside the backward kernel."""
    rows, H = 777, 4096
    x = _bf(rows, H, seed=1).requires_grad_()
    w = (1 + 0.1 * _bf(H, seed=2).float()).to(torch.bfloat16).requires_grad_()
    dh, dres = _bf(rows, H, seed=3), _bf(rows, H, seed=4)
    h, xr = K.rmsnorm_fork(x, w, 1e-5)
    torch.autograd.backward([h, xr], [dh, dres])
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    K.rmsnorm(x2, w2, 1e-5).backward(dh)
    want = x2.grad.float() + dres.float()
    _close(x.grad, want, atol=3e-2)
    assert torch.allclose(w.grad.float(), w2.grad.float(), rtol=1e-2, atol=1e-2)


def _rope_ref(t, cos, sin):
    half = t.shape[-1] // 2
    a, b = t[..., :half], t[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)


@pytest.mark.parametrize("rows,H", [(64, 256), (1000, 1024), (37, 768), (5, 8), (8191, 1024)])
def test_layernorm_fwd_bwd(rows, H):
    x = (_bf(rows, H, seed=1).float() * 2 + 0.5).to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * _bf(H, seed=2).float()).to(torch.bfloat16).requires_grad_()
    b = (0.1 * _bf(H, seed=4).float()).to(torch.bfloat16).requires_grad_()
    dy = _bf(rows, H, seed=3)
    assert K.layernorm_supported(x)
    y = K.layernorm(x, w, b, 1e-5)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr, atol=3e-2)
    _close(x.grad, xr.grad, atol=4e-2)
    tol = 0.02 * rows ** 0.5 + 0.05
    assert torch.allclose(w.grad.float(), wr.grad, rtol=3e-2, atol=tol)
    assert torch.allclose(b.grad.float(), br.grad, rtol=3e-2, atol=tol)
    # fp32 main_grad accumulation: gradients land in the flat buffers, autograd sees None
    w2, b2 = w.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    w2.main_grad = torch.ones(H, device="cuda")
    b2.main_grad = torch.zeros(H, device="cuda")
    K.layernorm(x.detach(), w2, b2, 1e-5).backward(dy)
    assert w2.grad is None and b2.grad is None
    assert torch.allclose(w2.main_grad - 1, wr.grad, rtol=1e-2, atol=tol)
    assert torch.allclose(b2.main_grad, br.grad, rtol=1e-2, atol=tol)
    assert not K.layernorm_supported(torch.empty(2, 2048, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("rows,C", [(64, 256), (777, 4096), (3, 8)])
def test_bias_gelu_fwd_bwd(rows, C):
    x = (_bf(rows, C, seed=5).float() * 2).to(torch.bfloat16).requires_grad_()
    b = _bf(C, seed=6).requires_grad_()
    dy = _bf(rows, C, seed=7)
    y = K.bias_gelu(x, b)
    y.backward(dy)
    xr, br = x.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(xr + br, approximate="tanh")
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    assert torch.allclose(b.grad.float(), br.grad, rtol=3e-2, atol=0.03 * rows ** 0.5 + 0.05)
    b2 = b.detach().clone().requires_grad_()
    b2.main_grad = torch.zeros(C, device="cuda")
    K.bias_gelu(x.detach(), b2).backward(dy)
    assert b2.grad is None
    assert torch.allclose(b2.main_grad, br.grad, rtol=1e-2, atol=0.03 * rows ** 0.5 + 0.05)


def test_rope_fwd_bwd():
    B, S, nh, hd = 2, 64, 4, 128
    H = nh * hd
    qkv = _bf(B * S, 3 * H, seed=4).requires_grad_()
    cos, sin = K.rope_tables(S, hd)
    ref_in = qkv.detach().float().view(B, S, 3, nh, hd).requires_grad_()
    out = K.rope_qk_(qkv * 1.0, cos, sin, nh, hd, S)
    dy = _bf(B * S, 3 * H, seed=5)
    out.backward(dy)
    c, s = cos.view(1, S, 1, hd // 2), sin.view(1, S, 1, hd // 2)
    ref = torch.stack([_rope_ref(ref_in[:, :, 0], c, s), _rope_ref(ref_in[:, :, 1], c, s),
                       ref_in[:, :, 2]], 2)
    ref.backward(dy.float().view(B, S, 3, nh, hd))
    _close(out.view(B, S, 3, nh, hd), ref)
    _close(qkv.grad.view(B, S, 3, nh, hd), ref_in.grad)


def test_swiglu_fwd_bwd():
    T, F = 100, 512
    gu = _bf(T, 2 * F, seed=6).requires_grad_()
    dh = _bf(T, F, seed=7)
    h = K.swiglu(gu)
    h.backward(dh)
    r = gu.detach().float().requires_grad_()
    hr = torch.nn.functional.silu(r[:, :F]) * r[:, F:]
    hr.backward(dh.float())
    _close(h, hr)
    _close(gu.grad, r.grad, atol=3e-2)


@pytest.mark.parametrize("rows,V", [(64, 512), (33, 32000)])
def test_cross_entropy_loss_and_grad(rows, V):
    logits = _bf(rows, V, seed=8, scale=2.0)
    targets = torch.randint(0, V, (rows,), device="cuda")
    targets[::5] = 0  # ignored
    ref_in = logits.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, targets, ignore_index=0)
    ref.backward()
    work = logits.clone().requires_grad_()
    loss = K.cross_entropy(work * 1.0, targets, ignore_index=0)
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert torch.allclose(work.grad.float(), ref_in.grad, rtol=5e-2, atol=2e-4)


def test_embedding_fwd_bwd():
    V, H, T = 1000, 256, 300
    table = _bf(V, H, seed=9).requires_grad_()
    ids = torch.randint(0, V, (3, 100), device="cuda")
    out = K.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    dout = _bf(3, 100, H, seed=10)
    out.backward(dout)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids.view(-1), dout.float().view(-1, H))
    _close(table.grad, ref, atol=5e-2)


def test_flat_adamw_matches_torch():
    n = 4096 * 3
    master = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(master.clone())
    opt_ref = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    grad = torch.zeros(n, device="cuda")
    bf = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    opt = K.FlatAdamW(master, grad, bf, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(4):
        g = torch.randn(n, device="cuda") * 0.1
        grad.copy_(g * 4)           # un-averaged sum over 4 "ranks"
        ref_p.grad = g.clone()
        opt_ref.step()
        opt.step(grad_scale=0.25, zero_grad=True)
        assert float(grad.abs().sum()) == 0.0
        assert torch.allclose(master, ref_p.data, rtol=1e-5, atol=1e-6)
        assert torch.equal(bf, master.to(torch.bfloat16))


def test_flat_sgd_matches_torch():
    n = 1000
    p = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt_ref = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, weight_decay=5e-4)
    grad = torch.zeros(n, device="cuda")
    opt = K.FlatSGD(p, grad, lr=0.1, momentum=0.9, weight_decay=5e-4)
    for _ in range(3):
        g = torch.randn(n, device="cuda")
        grad.copy_(g)
        ref_p.grad = g.clone()
        opt_ref.step()
        opt.step()
        assert torch.allclose(p, ref_p.data, rtol=1e-5, atol=1e-6)
