"""GPT-2 decoder (medium by default: 24 layers, d_model 1024, 16 heads, vocab 50257,
sequence 1024) for the sharded-training workload.  Linear layers run on the tcgen05 GEMM
(``ops.gemm``), attention on the tcgen05 flash kernel (head_dim 64), LayerNorm and
bias + GELU on the hand-written elementwise kernels.  Parameters are views of one flat
buffer so that ZeRO-style sharding is a contiguous range per rank.  The reference's GPT-2
benchmark uses a 4-layer, 256-wide HF model (``benchmarks/multimodel_stochastic_e2e_curve
.py:534-539``); there is no sharded trainer in the reference."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from ..ops import attention as A
from ..ops import gemm as G
from ..ops import nn as K
from ..parallel.flat import FlatParameters


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    seq: int = 1024
    init_std: float = 0.02

    @property
    def padded_vocab(self) -> int:
        return -(-self.vocab_size // 256) * 256

    @staticmethod
    def medium(**kw) -> "GPT2Config":
        return GPT2Config(**kw)

    @staticmethod
    def tiny(**kw) -> "GPT2Config":
        base = dict(vocab_size=512, n_layer=2, d_model=256, n_head=4, seq=128)
        base.update(kw)
        return GPT2Config(**base)


class GPT2(torch.nn.Module):
    def __init__(self, cfg: GPT2Config, device="cuda", seed: int = 0, pad_to: int = 256,
                 fused_ops: bool = True):
        super().__init__()
        self.cfg = cfg
        # False: LayerNorm, GELU and attention from torch (the library baseline for A/B runs)
        self.fused_ops = fused_ops
        D, V = cfg.d_model, cfg.padded_vocab
        shapes: Dict[str, Tuple[int, ...]] = {"wte": (V, D), "wpe": (cfg.seq, D)}
        for i in range(cfg.n_layer):
            shapes[f"h{i}.ln1_w"] = (D,)
            shapes[f"h{i}.ln1_b"] = (D,)
            shapes[f"h{i}.wqkv"] = (3 * D, D)
            shapes[f"h{i}.bqkv"] = (3 * D,)
            shapes[f"h{i}.wo"] = (D, D)
            shapes[f"h{i}.bo"] = (D,)
            shapes[f"h{i}.ln2_w"] = (D,)
            shapes[f"h{i}.ln2_b"] = (D,)
            shapes[f"h{i}.wfc"] = (4 * D, D)
            shapes[f"h{i}.bfc"] = (4 * D,)
            shapes[f"h{i}.wproj"] = (D, 4 * D)
            shapes[f"h{i}.bproj"] = (D,)
        shapes["lnf_w"] = (D,)
        shapes["lnf_b"] = (D,)
        self.flat = FlatParameters(shapes, device, pad_to=pad_to)
        self.p = torch.nn.ParameterDict(
            {n.replace(".", "_"): self.flat.make_parameter(n) for n in shapes})
        gen = torch.Generator(device=self.flat.params.device).manual_seed(seed)
        with torch.no_grad():
            for name, view in self.flat.named_views():
                if name.endswith("_w") and "ln" in name:
                    view.fill_(1.0)
                elif name.split(".")[-1].startswith("b") or name.endswith("_b"):
                    view.zero_()
                else:
                    view.copy_(torch.randn(view.shape, device=view.device, generator=gen)
                               * cfg.init_std)
        self.flat.sync_master_from_params()

    def _w(self, name):
        return self.p[name.replace(".", "_")]

    def _bias_grad_hook(self, name):
        return self._w(name)

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None):
        cfg = self.cfg
        B, S = ids.shape
        D, nh = cfg.d_model, cfg.n_head
        x = K.embedding(ids.reshape(-1), self._w("wte")) + self._w("wpe")[:S].repeat(B, 1)
        hd = D // nh
        fused_attn = self.fused_ops and A.available() and A.supported(S, hd)
        ln = K.layernorm if self.fused_ops and K.layernorm_supported(x) else (
            lambda t, w, b: F.layer_norm(t, (D,), w, b))
        gelu = K.bias_gelu if self.fused_ops else (
            lambda t, b: F.gelu(t + b, approximate="tanh"))
        for i in range(cfg.n_layer):
            if self.on_layer_backward is not None and x.requires_grad:
                # fires once the gradient w.r.t. this layer's input exists: every gradient of
                # the layer's own parameters has been produced by then
                x.register_hook(self._make_hook(i))
            h = ln(x, self._w(f"h{i}.ln1_w"), self._w(f"h{i}.ln1_b"))
            qkv = G.linear(h, self._w(f"h{i}.wqkv")) + self._w(f"h{i}.bqkv")
            if fused_attn:
                a = A.attention(qkv, B, S, nh, hd)
            else:
                q, k, v = (qkv[:, j * D:(j + 1) * D].view(B, S, nh, hd).transpose(1, 2)
                           for j in range(3))
                a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
                a = a.transpose(1, 2).reshape(B * S, D)
            x = x + G.linear(a, self._w(f"h{i}.wo")) + self._w(f"h{i}.bo")
            h = ln(x, self._w(f"h{i}.ln2_w"), self._w(f"h{i}.ln2_b"))
            h = gelu(G.linear(h, self._w(f"h{i}.wfc")), self._w(f"h{i}.bfc"))
            x = x + G.linear(h, self._w(f"h{i}.wproj")) + self._w(f"h{i}.bproj")
        x = ln(x, self._w("lnf_w"), self._w("lnf_b"))
        logits = G.linear(x, self._w("wte"))
        if targets is None:
            return logits.view(B, S, -1)
        shifted = torch.full_like(targets, -100)
        shifted[:, :-1] = targets[:, 1:]
        return K.cross_entropy(logits, shifted.reshape(-1), ignore_index=-100)

    on_layer_backward = None  # optional callable(layer_index), set by a trainer

    def _make_hook(self, layer_index: int):
        cb = self.on_layer_backward

        def hook(grad):
            cb(layer_index)
            return None

        return hook

    def collect_autograd_grads(self, prefix: Optional[str] = None) -> None:
        """Parameters updated by torch ops (LayerNorm, biases, position embedding) receive
        ``.grad``; fold them into the flat fp32 gradient buffer.  ``prefix`` limits the pass
        to the parameters whose name starts with it (one layer: ``"h3."``)."""
        want = None if prefix is None else prefix.replace(".", "_")
        for name, p in self.p.items():
            if p.grad is not None and (want is None or name.startswith(want)):
                p.main_grad.add_(p.grad.float())
                p.grad = None
