"""Small encoder / decoder transformers in plain torch modules, device-agnostic, for the
convergence benchmarks (they run on CPU ranks over gloo as well as on GPUs).  They stand in
for the Hugging Face ``BertForSequenceClassification`` and ``GPT2LMHeadModel`` instances the
reference builds with hidden 256, 4 layers, 4 heads
(``benchmarks/multimodel_stochastic_e2e_curve.py:48-74``).  These are not the hot-path
models: the Llama and GPT-2 medium trainers use the hand-written kernels."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, d: int, heads: int, causal: bool, pre_norm: bool, eps: float):
        super().__init__()
        self.heads, self.causal, self.pre_norm = heads, causal, pre_norm
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln1 = nn.LayerNorm(d, eps=eps)
        self.fc1 = nn.Linear(d, 4 * d)
        self.fc2 = nn.Linear(4 * d, d)
        self.ln2 = nn.LayerNorm(d, eps=eps)

    def _attn(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=self.causal)
        return self.proj(y.transpose(1, 2).reshape(b, s, d))

    def _mlp(self, x):
        return self.fc2(F.gelu(self.fc1(x)))

    def forward(self, x):
        if self.pre_norm:  # GPT-2 ordering
            x = x + self._attn(self.ln1(x))
            return x + self._mlp(self.ln2(x))
        x = self.ln1(x + self._attn(x))  # BERT ordering
        return self.ln2(x + self._mlp(x))


def _init(module: nn.Module, std: float = 0.02) -> None:
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=std)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)


class BertClassifier(nn.Module):
    """Post-norm encoder with learned positions, a tanh pooler over token 0 and a linear
    classifier; ``forward(ids, labels)`` returns the cross-entropy loss."""

    def __init__(self, vocab: int = 30522, hidden: int = 256, layers: int = 4, heads: int = 4,
                 max_pos: int = 512, num_labels: int = 2):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.ln = nn.LayerNorm(hidden, eps=1e-12)
        self.blocks = nn.ModuleList(_Block(hidden, heads, False, False, 1e-12)
                                    for _ in range(layers))
        self.pool = nn.Linear(hidden, hidden)
        self.cls = nn.Linear(hidden, num_labels)
        _init(self)

    def forward(self, ids: torch.Tensor, labels: torch.Tensor = None):
        pos = torch.arange(ids.shape[1], device=ids.device)
        x = self.ln(self.tok(ids) + self.pos(pos))
        for blk in self.blocks:
            x = blk(x)
        logits = self.cls(torch.tanh(self.pool(x[:, 0])))
        return logits if labels is None else F.cross_entropy(logits, labels)


class GPT2LM(nn.Module):
    """Pre-norm causal decoder with tied input / output embeddings; ``forward(ids,
    labels)`` returns the shifted next-token cross-entropy loss."""

    def __init__(self, vocab: int = 50257, hidden: int = 256, layers: int = 4, heads: int = 4,
                 max_pos: int = 512):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.blocks = nn.ModuleList(_Block(hidden, heads, True, True, 1e-5)
                                    for _ in range(layers))
        self.ln_f = nn.LayerNorm(hidden, eps=1e-5)
        _init(self)
        for blk in self.blocks:  # GPT-2 scales the residual projections
            nn.init.normal_(blk.proj.weight, std=0.02 / math.sqrt(2 * layers))
            nn.init.normal_(blk.fc2.weight, std=0.02 / math.sqrt(2 * layers))

    def forward(self, ids: torch.Tensor, labels: torch.Tensor = None):
        pos = torch.arange(ids.shape[1], device=ids.device)
        x = self.tok(ids) + self.pos(pos)
        for blk in self.blocks:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.tok.weight)
        if labels is None:
            return logits
        return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]),
                               labels[:, 1:].reshape(-1))
