"""Single-process golden model of the low-bit collectives.

Given every rank's input it plays the wire protocol with the host quantizer
(``bitscom_b200.quantization`` on CPU) and returns what every rank must end up with,
bit for bit under nearest rounding and under seeded stochastic rounding.  It is the
same construction as the reference's own distributed test oracle
(``tests/test_lowbit_allreduce_reference.py:81-164``: quantize shards per rank, sum in
ascending source order in fp32, re-quantize, concatenate) extended with first- and
second-stage error feedback (``cpp/src/process_group_lowbit.cc:696-770,1136-1170``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..quantization import (quantize_pack_tensor_blockwise, stage1_stream,
                            unpack_dequantize_tensor_blockwise)


@dataclass
class SimState:
    """Residuals of all ranks for one bucket."""

    stage1: List[Optional[torch.Tensor]] = field(default_factory=list)
    stage2: List[Optional[torch.Tensor]] = field(default_factory=list)


def _codec(x, bits, block, sr, seed, offset, stream):
    p, s, _ = quantize_pack_tensor_blockwise(
        x, bits, block_size=block, stochastic_rounding=sr, sr_seed=seed, sr_offset=offset,
        sr_stream=stream)
    d = unpack_dequantize_tensor_blockwise(p, s, bits, x.numel(), block_size=block,
                                           dtype=torch.float32)
    return p, s, d


def simulate_all_reduce(inputs: List[torch.Tensor], bits: int, block: int, *,
                        stochastic: bool = False, seed: Optional[int] = None,
                        state: Optional[SimState] = None, stage2: bool = False,
                        post_scale: float = 1.0) -> List[torch.Tensor]:
    """Returns the per-rank results (identical tensors) in each input's dtype."""
    world = len(inputs)
    n = int(inputs[0].numel())
    S = -(-n // world)
    padded = S * world
    use_ef = state is not None
    if use_ef and not state.stage1:
        state.stage1 = [torch.zeros(padded) for _ in range(world)]
        state.stage2 = [torch.zeros(S) for _ in range(world)]

    sent = [[None] * world for _ in range(world)]  # sent[i][j] = dequant(shard j of rank i)
    for i, t in enumerate(inputs):
        flat = t.detach().cpu().reshape(-1)
        flat = torch.nn.functional.pad(flat, (0, padded - n))
        if use_ef:
            flat = flat.to(torch.float32) + state.stage1[i]
        for j in range(world):
            shard = flat[j * S:(j + 1) * S]
            _, _, d = _codec(shard, bits, block, stochastic, seed, j * S, stage1_stream(i))
            sent[i][j] = d
            if use_ef:
                state.stage1[i][j * S:(j + 1) * S] = shard.to(torch.float32) - d

    parts = []
    for j in range(world):
        acc = torch.zeros(S)
        for i in range(world):
            acc.add_(sent[i][j])
        if use_ef and stage2:
            acc = acc + state.stage2[j]
        _, _, d = _codec(acc, bits, block, stochastic, seed, j * S, 1)
        if use_ef and stage2:
            state.stage2[j] = acc - d
        parts.append(d)
    full = torch.cat(parts)[:n]
    outs = []
    for t in inputs:
        r = full.view(t.shape).to(t.dtype)
        if post_scale != 1.0:
            r = r * post_scale
        outs.append(r)
    return outs


def simulate_reduce_scatter(inputs: List[torch.Tensor], bits: int, block: int, *,
                            stochastic: bool = False, seed: Optional[int] = None,
                            state: Optional[SimState] = None,
                            out_dtype: Optional[torch.dtype] = None) -> List[torch.Tensor]:
    """inputs[i] is rank i's flat ``[W * n]`` tensor; returns rank j's ``[n]`` output."""
    world = len(inputs)
    total = int(inputs[0].numel())
    n = total // world
    use_ef = state is not None
    if use_ef and not state.stage1:
        state.stage1 = [torch.zeros(total) for _ in range(world)]
    sent = [[None] * world for _ in range(world)]
    for i, t in enumerate(inputs):
        flat = t.detach().cpu().reshape(-1)
        if use_ef:
            flat = flat.to(torch.float32) + state.stage1[i]
        for j in range(world):
            shard = flat[j * n:(j + 1) * n]
            _, _, d = _codec(shard, bits, block, stochastic, seed, j * n, stage1_stream(i))
            sent[i][j] = d
            if use_ef:
                state.stage1[i][j * n:(j + 1) * n] = shard.to(torch.float32) - d
    outs = []
    for j in range(world):
        acc = torch.zeros(n)
        for i in range(world):
            acc.add_(sent[i][j])
        outs.append(acc.to(out_dtype or inputs[0].dtype))
    return outs


def simulate_all_gather(inputs: List[torch.Tensor], bits: int, block: int, *,
                        stochastic: bool = False, seed: Optional[int] = None,
                        state: Optional[SimState] = None,
                        out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """inputs[j] is rank j's ``[n]`` shard; returns the ``[W * n]`` tensor all ranks get."""
    world = len(inputs)
    n = int(inputs[0].numel())
    use_ef = state is not None
    if use_ef and not state.stage2:
        state.stage2 = [torch.zeros(n) for _ in range(world)]
    parts = []
    for j, t in enumerate(inputs):
        x = t.detach().cpu().reshape(-1)
        if use_ef:
            x = x.to(torch.float32) + state.stage2[j]
        _, _, d = _codec(x, bits, block, stochastic, seed, j * n, 1)
        if use_ef:
            state.stage2[j] = x.to(torch.float32) - d
        parts.append(d)
    return torch.cat(parts).to(out_dtype or inputs[0].dtype)
