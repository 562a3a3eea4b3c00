"""ZeRO-1 style sharded optimizer on low-bit collectives.

Every rank keeps the whole bf16 model but only ``1/W`` of the fp32 master weights and
optimizer moments.  One step is

  low-bit reduce-scatter of the flat fp32 gradient  ->  each rank holds the summed
      gradient of its shard (error feedback on the sender side),
  fused AdamW on the shard, which also writes the bf16 copy of the shard straight into its
      place in the flat parameter buffer,
  low-bit all-gather of that bf16 shard into the flat parameter buffer IN PLACE (the shard is
      a slice of the output; error feedback on the owner side, so quantization error of the
      broadcast parameters is carried to the next step instead of accumulating).  No fp32
      staging buffer of the whole model and no conversion pass afterwards.

The reference has only the low-bit reduce-scatter primitive in its C++ backend
(``cpp/src/process_group_lowbit.cc:1670-1777``) and forwards all-gather to NCCL; sharded
training on top of both is new here.
"""

from __future__ import annotations

from typing import List

import torch

from ..ops import nn as K
from .flat import FlatParameters


class ShardedAdamW:
    def __init__(self, flat: FlatParameters, lowbit_group, *, lr=1e-4, betas=(0.9, 0.999),
                 eps=1e-8, weight_decay=0.01, param_bits_group=None):
        self.flat = flat
        self.group = lowbit_group              # gradients: reduce-scatter
        self.pgroup = param_bits_group or lowbit_group  # parameters: all-gather
        self.world = lowbit_group.world_size
        self.rank = lowbit_group.rank
        n = flat.numel
        if n % (self.world * 256):
            raise ValueError("flat buffer must be padded to world * 256 elements")
        self.shard = n // self.world
        lo = self.rank * self.shard
        dev = flat.params.device
        self.master_shard = flat.params[lo:lo + self.shard].float().clone()
        self.grad_shard = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        # the optimizer kernel refreshes the bf16 working copy of the shard where it lives
        self.param_shard = flat.params[lo:lo + self.shard]
        self.opt = K.FlatAdamW(self.master_shard, self.grad_shard, self.param_shard, lr=lr,
                               betas=betas, eps=eps, weight_decay=weight_decay)

    def step(self) -> None:
        flat = self.flat
        if self.world > 1:
            self.group.reduce_scatter_lowbit(self.grad_shard, flat.grads, ef_key="zero_grads")
        else:
            self.grad_shard.copy_(flat.grads)
        self.opt.step(grad_scale=1.0 / self.world, zero_grad=True)
        flat.grads.zero_()
        if self.world > 1:
            # in place: every rank, the owner included, ends up with the dequantized shard, so
            # all replicas of the bf16 model stay bit-identical
            self.pgroup.all_gather_lowbit(flat.params, self.param_shard, ef_key="zero_params")

    def state_dict(self):
        return {"opt": self.opt.state_dict(), "master_shard": self.master_shard}

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd["opt"])   # also refreshes the bf16 copy of the shard
        self.master_shard.copy_(sd["master_shard"])


def reshard_state(states: List[dict], new_world: int, numel: int) -> List[dict]:
    """Re-partition the optimizer state of a sharded run for another world size.

    ``states`` are the ``ShardedAdamW.state_dict()`` of every rank of the old run, in rank
    order (for example read back from the per-rank checkpoint files after a restart with
    fewer ranks); ``numel`` is the unpadded number of parameters.  Returns one state dict per
    rank of the new run.  The flat buffer of a run is padded to ``world * 256`` elements, so
    the padded lengths of the two runs may differ: padding holds zero parameters with zero
    moments and is cut or added at the end."""
    if not states:
        raise ValueError("no states given")
    steps = {int(s["opt"]["step"]) for s in states}
    if len(steps) != 1:
        raise ValueError(f"the ranks' states are from different steps: {sorted(steps)}")
    unit = new_world * 256
    padded = -(-int(numel) // unit) * unit
    step = steps.pop()
    out: List[dict] = [{"opt": {"step": step}} for _ in range(new_world)]

    def repartition(pick):
        full = torch.cat([pick(s).reshape(-1).to(torch.float32).cpu() for s in states])
        if full.numel() < numel:
            raise ValueError("the states hold fewer elements than numel")
        full = full[:numel]
        if padded > numel:
            full = torch.cat([full, torch.zeros(padded - numel)])
        return list(full.view(new_world, padded // new_world).unbind(0))

    for name in ("exp_avg", "exp_avg_sq", "master"):
        for r, piece in enumerate(repartition(lambda s, name=name: s["opt"][name])):
            out[r]["opt"][name] = piece.clone()
    for r in range(new_world):
        out[r]["master_shard"] = out[r]["opt"]["master"].clone()
    return out
