"""Flat parameter storage: one bf16 working buffer, one fp32 master copy and one fp32
gradient buffer per model (or pipeline stage), with every parameter a view.

Why flat: (1) the optimizer is one fused kernel over the whole buffer; (2) gradient
buckets for the low-bit all-reduce are *slices* of the flat fp32 gradient buffer, so
bucketing copies nothing (the reference's benchmarks ``torch.cat`` every bucket and
scatter it back, ``benchmarks/multimodel_stochastic_e2e_curve.py:207-244``) and error
feedback residuals have a stable identity: the bucket index; (3) ZeRO-style sharding
is a contiguous range per rank.
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch

ALIGN = 256  # elements; keeps every parameter 16-byte aligned in all three buffers


class FlatParameters:
    def __init__(self, shapes: Dict[str, Tuple[int, ...]], device, dtype=torch.bfloat16,
                 pad_to: int = ALIGN, with_master: bool = True):
        self.dtype = dtype
        self.offsets: Dict[str, Tuple[int, int, Tuple[int, ...]]] = {}
        cursor = 0
        for name, shape in shapes.items():
            n = 1
            for s in shape:
                n *= s
            self.offsets[name] = (cursor, n, tuple(shape))
            cursor += -(-n // ALIGN) * ALIGN
        self.used = cursor  # elements before the padding to ``pad_to`` (the same for every pad_to)
        self.numel = -(-cursor // pad_to) * pad_to
        self.params = torch.zeros(self.numel, dtype=dtype, device=device)
        self.grads = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.master = torch.zeros(self.numel, dtype=torch.float32, device=device) \
            if with_master and dtype != torch.float32 else (self.params if dtype == torch.float32
                                                            else None)

    def view(self, name: str) -> torch.Tensor:
        off, n, shape = self.offsets[name]
        return self.params[off:off + n].view(shape)

    def grad_view(self, name: str) -> torch.Tensor:
        off, n, shape = self.offsets[name]
        return self.grads[off:off + n].view(shape)

    def make_parameter(self, name: str) -> torch.nn.Parameter:
        p = torch.nn.Parameter(self.view(name))
        p.main_grad = self.grad_view(name)
        return p

    def sync_master_from_params(self) -> None:
        if self.master is not None and self.master is not self.params:
            self.master.copy_(self.params)

    def buckets(self, bucket_elems: int, multiple_of: int = 1) -> List[Tuple[int, int]]:
        """(start, length) slices of the flat buffers, each ``bucket_elems`` long (rounded
        up to ``multiple_of``) except the last."""
        size = max(multiple_of, -(-bucket_elems // multiple_of) * multiple_of)
        return [(s, min(size, self.numel - s)) for s in range(0, self.numel, size)]

    def named_views(self) -> Iterable[Tuple[str, torch.Tensor]]:
        for name in self.offsets:
            yield name, self.view(name)
