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

from typing import Dict, List, Optional, Sequence

import torch

from ..ops import nn as K
from .flat import FlatParameters


class ShardedAdamW:
    def __init__(self, flat: FlatParameters, lowbit_group, *, lr=1e-4, betas=(0.9, 0.999),
                 eps=1e-8, weight_decay=0.01, param_bits_group=None, key=None):
        # key: distinguishes the error-feedback residuals of several instances that share the
        # same groups (one instance per bucket in BucketedShardedAdamW)
        self._grad_key = "zero_grads" if key is None else ("zero_grads", key)
        self._param_key = "zero_params" if key is None else ("zero_params", key)
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

    def reduce_grads(self) -> None:
        """Summed gradient of this rank's shard -> ``grad_shard`` (on the current stream)."""
        if self.world > 1:
            self.group.reduce_scatter_lowbit(self.grad_shard, self.flat.grads,
                                             ef_key=self._grad_key)
        else:
            self.grad_shard.copy_(self.flat.grads)

    def update(self) -> None:
        """AdamW on the shard; clears the gradient buffers."""
        self.opt.step(grad_scale=1.0 / self.world, zero_grad=True)
        self.flat.grads.zero_()

    def gather_params(self) -> None:
        if self.world > 1:
            # in place: every rank, the owner included, ends up with the dequantized shard, so
            # all replicas of the bf16 model stay bit-identical
            self.pgroup.all_gather_lowbit(self.flat.params, self.param_shard,
                                          ef_key=self._param_key)

    def step(self) -> None:
        self.reduce_grads()
        self.update()
        self.gather_params()

    def state_dict(self):
        return {"opt": self.opt.state_dict(), "master_shard": self.master_shard}

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd["opt"])   # also refreshes the bf16 copy of the shard
        self.master_shard.copy_(sd["master_shard"])


class FlatSlice:
    """``[start, start + length)`` of a flat parameter set, with the attributes the sharded
    optimizer reads."""

    def __init__(self, flat, start: int, length: int):
        self.numel = int(length)
        self.params = flat.params[start:start + length]
        self.grads = flat.grads[start:start + length]


def bucket_cuts(starts: Sequence[int], numel: int, world: int) -> List[int]:
    """Cut points ``[0, ..., numel]`` of the buckets for parameter groups that begin at
    ``starts``: every cut is rounded UP to ``world * 256`` elements (a bucket is shared out
    in whole quantization blocks), empty buckets are dropped."""
    unit = world * 256
    if numel % unit:
        raise ValueError("flat buffer must be padded to world * 256 elements")
    cuts = {0, int(numel)}
    for s in starts:
        cuts.add(min(-(-int(s) // unit) * unit, int(numel)))
    return sorted(cuts)


class BucketedShardedAdamW:
    """``ShardedAdamW`` bucket by bucket, with the collectives off the critical path.

    The flat buffer is cut at ``cuts`` (see ``bucket_cuts``); every bucket is shared out over
    the ranks on its own, so a rank owns ``1/W`` of EVERY bucket.  Backward announces finished
    parameter groups with ``ready_from(offset)``: the buckets that lie entirely behind the
    (rounded-up) offset are reduce-scattered on a side stream while backward goes on.
    ``step`` launches what is left, then walks the buckets in forward order: AdamW on the
    bucket's shard (compute stream) as soon as its reduce-scatter has landed, and the low-bit
    all-gather of the bucket's parameters on the side stream behind it, under the next
    bucket's AdamW.  All collectives run on ONE side stream, in an order that is the same on
    every rank: they share one symmetric-memory communicator, which holds one call at a time.
    Rounding the cuts up puts the first elements of group g into bucket g - 1; backward
    finishes groups in descending order, so bucket g - 1, launched after group g - 1, finds
    them final."""

    def __init__(self, flat: FlatParameters, lowbit_group, cuts: Sequence[int], *,
                 overlap: bool = True, **kw):
        self.flat, self.world, self.rank = flat, lowbit_group.world_size, lowbit_group.rank
        self.cuts = [int(c) for c in cuts]
        if self.cuts[0] != 0 or self.cuts[-1] != flat.numel or sorted(set(self.cuts)) != self.cuts:
            raise ValueError("cuts must rise from 0 to the buffer length")
        self.parts = [ShardedAdamW(FlatSlice(flat, lo, hi - lo), lowbit_group, key=b, **kw)
                      for b, (lo, hi) in enumerate(zip(self.cuts, self.cuts[1:]))]
        cuda = flat.params.is_cuda
        self.stream = torch.cuda.Stream(device=flat.params.device) if cuda and overlap else None
        self._launched = [False] * len(self.parts)
        self._events: List[Optional[torch.cuda.Event]] = [None] * len(self.parts)

    @property
    def master_shards(self) -> List[torch.Tensor]:
        return [p.master_shard for p in self.parts]

    def _reduce(self, b: int) -> None:
        if self._launched[b]:
            return
        self._launched[b] = True
        if self.stream is None:
            self.parts[b].reduce_grads()
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.flat.params.device))
        with torch.cuda.stream(self.stream):
            self.parts[b].reduce_grads()
            self._events[b] = self.stream.record_event()

    def ready_from(self, offset: int) -> None:
        """Every gradient at flat index >= ``offset`` is final on the current stream."""
        unit = self.world * 256
        lo = -(-int(offset) // unit) * unit
        for b in range(len(self.parts) - 1, -1, -1):
            if self.cuts[b] < lo:
                break
            self._reduce(b)

    def step(self) -> None:
        for b in range(len(self.parts) - 1, -1, -1):
            self._reduce(b)
        cur = torch.cuda.current_stream(self.flat.params.device) if self.stream else None
        for b, part in enumerate(self.parts):
            if cur is not None:
                cur.wait_event(self._events[b])
            part.update()
            if cur is not None:
                self.stream.wait_event(cur.record_event())
                with torch.cuda.stream(self.stream):
                    part.gather_params()
            else:
                part.gather_params()
        if cur is not None:
            cur.wait_stream(self.stream)
        self._launched = [False] * len(self.parts)

    def state_dict(self) -> dict:
        return {"cuts": list(self.cuts), "buckets": [p.state_dict() for p in self.parts]}

    def load_state_dict(self, sd: dict) -> None:
        if list(sd["cuts"]) != self.cuts:
            raise ValueError("the state was saved with other bucket cuts: re-partition it "
                             "with reshard_bucketed_state first")
        for part, piece in zip(self.parts, sd["buckets"]):
            part.load_state_dict(piece)


def reshard_bucketed_state(states: List[dict], new_world: int, new_cuts: Sequence[int],
                           numel: int) -> List[dict]:
    """``reshard_state`` for ``BucketedShardedAdamW``: ``states`` are all old ranks' state
    dicts (same cuts), the result is one state dict per new rank for buckets cut at
    ``new_cuts``.  The old and the new run may differ in world size, in their cuts and in the
    padding at the end of the buffer; ``numel`` is the unpadded number of parameters."""
    if not states:
        raise ValueError("no states given")
    old_cuts = list(states[0]["cuts"])
    if any(list(s["cuts"]) != old_cuts for s in states):
        raise ValueError("the ranks' states were saved with different bucket cuts")
    steps = {int(b["opt"]["step"]) for s in states for b in s["buckets"]}
    if len(steps) != 1:
        raise ValueError(f"the states are from different steps: {sorted(steps)}")
    step = steps.pop()
    new_cuts = [int(c) for c in new_cuts]
    total = max(old_cuts[-1], new_cuts[-1])
    full: Dict[str, torch.Tensor] = {}
    for name in ("exp_avg", "exp_avg_sq", "master"):
        buf = torch.zeros(total, dtype=torch.float32)
        for b, (lo, hi) in enumerate(zip(old_cuts, old_cuts[1:])):
            buf[lo:hi] = torch.cat([s["buckets"][b]["opt"][name].reshape(-1).float().cpu()
                                    for s in states])
        buf[numel:] = 0.0     # padding: zero parameters with zero moments
        full[name] = buf
    out = [{"cuts": new_cuts, "buckets": []} for _ in range(new_world)]
    for lo, hi in zip(new_cuts, new_cuts[1:]):
        if (hi - lo) % (new_world * 256):
            raise ValueError("new cuts must be multiples of new_world * 256")
        shard = (hi - lo) // new_world
        for r in range(new_world):
            a = lo + r * shard
            opt = {"step": step}
            for name in ("exp_avg", "exp_avg_sq", "master"):
                opt[name] = full[name][a:a + shard].clone()
            out[r]["buckets"].append({"opt": opt, "master_shard": opt["master"].clone()})
    return out


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
