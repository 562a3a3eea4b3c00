"""Tiny GPT-2 on the hand-written kernels (tcgen05 GEMM, head_dim-64 attention, LayerNorm,
bias + GELU, fused cross-entropy) against a plain fp32 PyTorch model with the same weights."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.models.gpt2 import GPT2, GPT2Config


def _reference_loss(model, ids, params):
    cfg = model.cfg
    B, S = ids.shape
    D, nh = cfg.d_model, cfg.n_head
    w = lambda n: params[n.replace(".", "_")]  # noqa: E731
    x = w("wte")[ids.reshape(-1)] + w("wpe")[:S].repeat(B, 1)
    for i in range(cfg.n_layer):
        h = F.layer_norm(x, (D,), w(f"h{i}.ln1_w"), w(f"h{i}.ln1_b"))
        qkv = h @ w(f"h{i}.wqkv").t() + w(f"h{i}.bqkv")
        q, k, v = (qkv[:, j * D:(j + 1) * D].view(B, S, nh, D // nh).transpose(1, 2)
                   for j in range(3))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + a.transpose(1, 2).reshape(B * S, D) @ w(f"h{i}.wo").t() + w(f"h{i}.bo")
        h = F.layer_norm(x, (D,), w(f"h{i}.ln2_w"), w(f"h{i}.ln2_b"))
        h = F.gelu(h @ w(f"h{i}.wfc").t() + w(f"h{i}.bfc"), approximate="tanh")
        x = x + h @ w(f"h{i}.wproj").t() + w(f"h{i}.bproj")
    x = F.layer_norm(x, (D,), w("lnf_w"), w("lnf_b"))
    logits = x @ w("wte").t()
    tgt = torch.full_like(ids, -100)
    tgt[:, :-1] = ids[:, 1:]
    return F.cross_entropy(logits.float(), tgt.reshape(-1), ignore_index=-100)


def test_tiny_gpt2_loss_and_grads_match_fp32_reference():
    cfg = GPT2Config.tiny()  # d_model 256, 4 heads: head_dim 64, seq 128
    model = GPT2(cfg, "cuda", seed=3)
    with torch.no_grad():  # make biases and LayerNorm parameters non-trivial
        g = torch.Generator(device="cuda").manual_seed(11)
        for name, view in model.flat.named_views():
            if view.dim() == 1:
                view.add_(torch.randn(view.shape, device="cuda", generator=g) * 0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq), device="cuda",
                        generator=torch.Generator(device="cuda").manual_seed(5))
    loss = model(ids, ids)
    loss.backward()
    model.collect_autograd_grads()
    torch.cuda.synchronize()

    params = {n: p.detach().float().requires_grad_() for n, p in model.p.items()}
    ref = _reference_loss(model, ids, params)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item()))
    for name in ("h0_wqkv", "h1_wfc", "h0_ln1_w", "h1_ln2_b", "h0_bfc", "h1_bqkv", "lnf_w", "wpe"):
        got, want = model.p[name].main_grad, params[name].grad
        scale = want.abs().max().item() + 1e-6
        err = (got - want).abs().max().item()
        assert err < 0.08 * scale + 2e-3, f"{name}: max err {err} vs scale {scale}"


def test_graphed_step_matches_eager_step():
    """Forward + backward captured in a CUDA graph gives the same loss and the same flat
    gradient as the eager step, on fresh inputs, replay after replay."""
    from bitscom_b200.utils.graphs import GraphedStep

    cfg = GPT2Config.tiny()
    eager, graphed = GPT2(cfg, "cuda", seed=3), GPT2(cfg, "cuda", seed=3)

    def make(model):
        def fwd_bwd(ids):
            loss = model(ids, targets=ids)
            loss.backward()
            model.collect_autograd_grads()
            return loss.detach()
        return fwd_bwd

    example = torch.zeros(2, cfg.seq, dtype=torch.int64, device="cuda")
    step = GraphedStep(make(graphed), [example], reset=lambda: graphed.flat.grads.zero_())
    run_eager = make(eager)
    gen = torch.Generator(device="cuda").manual_seed(9)
    for _ in range(3):
        ids = torch.randint(0, cfg.vocab_size, (2, cfg.seq), device="cuda", generator=gen)
        eager.flat.grads.zero_()
        graphed.flat.grads.zero_()
        want = run_eager(ids)
        got = step(ids)
        torch.cuda.synchronize()
        assert abs(got.item() - want.item()) < 1e-3
        ge, gg = eager.flat.grads, graphed.flat.grads
        # identical kernels in identical order; only fp32 atomics may reorder
        assert (ge - gg).abs().max().item() <= 1e-3 * ge.abs().max().item() + 1e-6
    assert step.replays == 3
