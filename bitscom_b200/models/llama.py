"""Llama decoder on hand-written sm_100a kernels.

Architecture of the reference trainer's model config
(``benchmarks/train_llama7b_dp_pp_lowbit.py:222-231``: vocab 32000, hidden 4096, FFN
11008 SwiGLU, 32 layers, 32 heads, RMSNorm, RoPE theta 1e4, tied embeddings) — the
reference imports the module itself from an external package; this one is written for
B200: every linear layer is the tcgen05/TMEM GEMM (forward, data gradient and weight
gradient), attention is the tcgen05 flash kernel, RMSNorm / RoPE / SwiGLU / softmax
cross-entropy / embedding are single-pass kernels, parameters live in one flat buffer
(``bitscom_b200.parallel.flat``) and weight gradients accumulate in fp32.

A model is built per pipeline stage: ``LlamaStage(cfg, first_layer, last_layer, ...)``
holds the embedding on the first stage and the final norm + LM head on the last.
"""

from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from ..ops import gemm as G
from ..ops import nn as K
from ..parallel.flat import FlatParameters


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    max_seq: int = 2048
    tie_embeddings: bool = True
    attention: str = "tcgen05"   # "tcgen05" (own kernel) or "sdpa" (library fallback)
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @staticmethod
    def llama7b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        base = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_layers=2,
                    num_heads=2, max_seq=256)
        base.update(kw)
        return LlamaConfig(**base)

    def params_per_layer(self) -> int:
        H, F = self.hidden_size, self.intermediate_size
        return 4 * H * H + 3 * H * F + 2 * H

    def total_params(self) -> int:
        emb = self.vocab_size * self.hidden_size
        return self.num_layers * self.params_per_layer() + emb * (1 if self.tie_embeddings else 2) \
            + self.hidden_size


def stage_layers(num_layers: int, stage: int, num_stages: int) -> Tuple[int, int]:
    """Contiguous layer range of a pipeline stage; earlier stages take the remainder
    (same split as the reference, ``train_llama7b_dp_pp_lowbit.py:127-131``)."""
    per, rem = divmod(num_layers, num_stages)
    start = stage * per + min(stage, rem)
    return start, start + per + (1 if stage < rem else 0)


def _attention(qkv: torch.Tensor, batch: int, seq: int, heads: int, head_dim: int, impl: str):
    if impl == "tcgen05":
        from ..ops import attention as A

        return A.attention(qkv, batch, seq, heads, head_dim)
    H = heads * head_dim
    q, k, v = (qkv[..., i * H:(i + 1) * H].view(batch, seq, heads, head_dim).transpose(1, 2)
               for i in range(3))
    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.transpose(1, 2).reshape(batch * seq, H)


class LlamaStage(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, stage: int = 0, num_stages: int = 1,
                 device="cuda", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.stage, self.num_stages = stage, num_stages
        self.is_first, self.is_last = stage == 0, stage == num_stages - 1
        self.layer_range = stage_layers(cfg.num_layers, stage, num_stages)
        H, F, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size

        shapes: Dict[str, Tuple[int, ...]] = {}
        if self.is_first:
            shapes["embed"] = (V, H)
        for i in range(*self.layer_range):
            shapes[f"l{i}.norm1"] = (H,)
            shapes[f"l{i}.wqkv"] = (3 * H, H)
            shapes[f"l{i}.wo"] = (H, H)
            shapes[f"l{i}.norm2"] = (H,)
            shapes[f"l{i}.wgu"] = (2 * F, H)
            shapes[f"l{i}.wdown"] = (H, F)
        if self.is_last:
            shapes["final_norm"] = (H,)
            if not (cfg.tie_embeddings and self.is_first):
                shapes["lm_head"] = (V, H)
        self.flat = FlatParameters(shapes, device)
        self.p = torch.nn.ParameterDict(
            {name.replace(".", "_"): self.flat.make_parameter(name) for name in shapes})
        self.reset_parameters(seed)
        self._rope: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None

    def reset_parameters(self, seed: int = 0) -> None:
        """Every tensor draws from a stream keyed by (seed, its name), so a parameter has the
        same initial value whichever pipeline stage owns it: a model split over stages starts
        from the same weights as the unsplit one."""
        gen = torch.Generator(device=self.flat.params.device)
        with torch.no_grad():
            for name, view in self.flat.named_views():
                if "norm" in name:
                    view.fill_(1.0)
                else:
                    gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (1 << 62))
                    view.copy_(torch.randn(view.shape, device=view.device, generator=gen,
                                           dtype=torch.float32) * self.cfg.init_std)
        self.flat.sync_master_from_params()

    def _w(self, name: str) -> torch.nn.Parameter:
        return self.p[name.replace(".", "_")]

    def _rope_tables(self, seq: int, device):
        if self._rope is None or self._rope[2] != seq:
            cos, sin = K.rope_tables(seq, self.cfg.head_dim, self.cfg.rope_theta, device)
            self._rope = (cos, sin, seq)
        return self._rope[0], self._rope[1]

    def layer(self, i: int, x: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        cfg = self.cfg
        cos, sin = self._rope_tables(seq, x.device)
        # residual adds live in the epilogue of the output / down projections, and the two
        # gradients that meet at each norm's input are added inside the norm's backward kernel
        h, x = K.rmsnorm_fork(x, self._w(f"l{i}.norm1"), cfg.rms_eps)
        qkv = G.linear(h, self._w(f"l{i}.wqkv"))
        qkv = K.rope_qk_(qkv, cos, sin, cfg.num_heads, cfg.head_dim, seq)
        a = _attention(qkv, batch, seq, cfg.num_heads, cfg.head_dim, cfg.attention)
        x = G.linear(a, self._w(f"l{i}.wo"), residual=x)
        h, x = K.rmsnorm_fork(x, self._w(f"l{i}.norm2"), cfg.rms_eps)
        gu = G.linear(h, self._w(f"l{i}.wgu"))
        x = G.linear(K.swiglu(gu), self._w(f"l{i}.wdown"), residual=x)
        return x

    def forward(self, inp: torch.Tensor, targets: Optional[torch.Tensor] = None,
                ignore_index: int = 0, loss_scale: float = 1.0):
        """First stage: ``inp`` are token ids ``[batch, seq]``; other stages: hidden states
        ``[batch * seq, hidden]`` (pass batch/seq through ``set_shape``).  The last stage
        returns the mean next-token loss when ``targets [batch, seq]`` are given, else the
        logits; earlier stages return hidden states."""
        if self.is_first:
            batch, seq = inp.shape
            x = K.embedding(inp.reshape(-1), self._w("embed"))
        else:
            batch, seq = self._shape
            x = inp
        self._shape = (batch, seq)
        for i in range(*self.layer_range):
            if self.on_layer_backward is not None and x.requires_grad:
                # fires once the gradient w.r.t. this layer's input exists, i.e. the layer's
                # own weight gradients have been enqueued
                x.register_hook(self._make_hook(i))
            x = self.layer(i, x, batch, seq)
        if not self.is_last:
            return x
        x = K.rmsnorm(x, self._w("final_norm"), self.cfg.rms_eps)
        head = self._w("lm_head") if "lm_head" in self.p else self._w("embed")
        logits = G.linear(x, head)
        if targets is None:
            return logits.view(batch, seq, -1)
        # next-token prediction: position t predicts token t+1; the last position of every
        # sequence has no target (reference loss: train_llama7b_dp_pp_lowbit.py:158-165)
        shifted = torch.full_like(targets, ignore_index)
        shifted[:, :-1] = targets[:, 1:]
        return K.cross_entropy(logits, shifted.reshape(-1), ignore_index, loss_scale)

    def _make_hook(self, layer_index: int):
        cb = self.on_layer_backward

        def hook(grad):
            cb(layer_index)
            return None

        return hook

    on_layer_backward = None  # optional callable(layer_index), set by the trainer

    def set_shape(self, batch: int, seq: int) -> None:
        self._shape = (batch, seq)

    _shape: Tuple[int, int] = (1, 1)
