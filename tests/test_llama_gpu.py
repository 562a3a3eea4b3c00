"""Tiny Llama stage on the hand-written kernels against a plain fp32 PyTorch model."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.models.llama import LlamaConfig, LlamaStage, stage_layers
    from bitscom_b200.ops import nn as K


def _reference_loss(model, ids, cfg):
    """fp32 re-statement of the same network from the model's own bf16 weights."""
    P = {k: v.detach().float() for k, v in model.flat.named_views()}
    B, S = ids.shape
    H, nh, hd, F = cfg.hidden_size, cfg.num_heads, cfg.head_dim, cfg.intermediate_size
    cos, sin = K.rope_tables(S, hd)
    cos, sin = cos.view(1, S, 1, hd // 2), sin.view(1, S, 1, hd // 2)

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w

    def rope(t):
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    x = P["embed"][ids.view(-1)]
    for i in range(cfg.num_layers):
        h = norm(x, P[f"l{i}.norm1"])
        qkv = (h @ P[f"l{i}.wqkv"].t()).view(B, S, 3, nh, hd)
        q, k, v = rope(qkv[:, :, 0]), rope(qkv[:, :, 1]), qkv[:, :, 2]
        att = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + att.transpose(1, 2).reshape(B * S, H) @ P[f"l{i}.wo"].t()
        h = norm(x, P[f"l{i}.norm2"])
        gu = h @ P[f"l{i}.wgu"].t()
        x = x + (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ P[f"l{i}.wdown"].t()
    logits = norm(x, P["final_norm"]) @ P["embed"].t()
    tgt = torch.zeros_like(ids)
    tgt[:, :-1] = ids[:, 1:]
    return torch.nn.functional.cross_entropy(logits, tgt.view(-1), ignore_index=0)


def test_stage_layers_split():
    assert [stage_layers(32, s, 4) for s in range(4)] == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert [stage_layers(5, s, 2) for s in range(2)] == [(0, 3), (3, 5)]


@pytest.mark.parametrize("attention", ["sdpa", "tcgen05"])
def test_tiny_llama_loss_and_grads(attention):
    if attention == "tcgen05":
        from bitscom_b200.ops import attention as A
        if not A.available():
            pytest.skip("attention kernel not built")
    cfg = LlamaConfig.tiny(attention=attention, hidden_size=256, num_heads=2, max_seq=128)
    model = LlamaStage(cfg, device="cuda", seed=3)
    ids = torch.randint(1, cfg.vocab_size, (2, 128), device="cuda")
    loss = model(ids, targets=ids)
    loss.backward()
    ref = _reference_loss(model, ids, cfg)
    assert abs(loss.item() - ref.item()) < 0.05, (loss.item(), ref.item())
    g = model.flat.grads
    assert torch.isfinite(g).all() and g.abs().sum() > 0
    # one optimizer step lowers the loss on the same batch
    opt = K.FlatAdamW(model.flat.master, model.flat.grads, model.flat.params, lr=1e-3)
    opt.step()
    loss2 = model(ids, targets=ids)
    assert loss2.item() < loss.item()


@pytest.mark.skipif(os.environ.get("BITSCOM_EXPERIMENTAL", "0") != "1",
                    reason="consistency check of the ops' host paths against the kernels; "
                           "set BITSCOM_EXPERIMENTAL=1 to run it")
def test_host_paths_follow_the_kernels():
    """The same tiny model (the same weights) on the GPU through the kernels and on the CPU
    through the ops' host paths: loss and flat gradient agree to bf16 accuracy."""
    cfg = LlamaConfig.tiny(attention="sdpa", hidden_size=256, num_heads=2, max_seq=128)
    ids = torch.randint(1, cfg.vocab_size, (2, 128), generator=torch.Generator().manual_seed(5))
    gpu = LlamaStage(cfg, device="cuda", seed=3)
    cpu = LlamaStage(cfg, device="cpu", seed=3)
    with torch.no_grad():      # the two devices' generators differ: copy the weights over
        cpu.flat.params.copy_(gpu.flat.params.cpu())
    cpu.flat.sync_master_from_params()
    results = {}
    for device, model in (("cuda", gpu), ("cpu", cpu)):
        loss = model(ids.to(device), targets=ids.to(device))
        loss.backward()
        results[device] = (float(loss), model.flat.grads.detach().float().cpu().clone())
    assert abs(results["cuda"][0] - results["cpu"][0]) < 0.02
    g_gpu, g_cpu = results["cuda"][1], results["cpu"][1]
    assert (g_gpu - g_cpu).norm() < 0.05 * g_cpu.norm()


def test_trainer_cli_trains_on_a_text_file(tmp_path, capsys):
    """The trainer's command line with the reference's flags, fed from a local text file
    through the byte tokenizer and the prefetching loader: two epochs, the loss goes down."""
    import json

    from bitscom_b200.trainer import llama_dp_pp

    text = tmp_path / "docs.txt"
    text.write_text("\n".join("the quick brown fox jumps over the lazy dog " * 4
                              for _ in range(16)))
    llama_dp_pp.main(["--model", "tiny", "--dataset", str(text), "--tokenizer", "bytes",
                      "--seq_length", "128", "--micro_batches", "2", "--batch_size", "2",
                      "--epochs", "3", "--max_steps", "12", "--lr", "3e-3",
                      "--simulate_quantization", "--dataset_config", "ignored"])
    rows = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(rows) == 12 and rows[-1]["epoch"] == 2
    assert rows[-1]["loss"] < rows[0]["loss"] - 0.5
