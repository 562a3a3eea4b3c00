"""Low-bit reduce-scatter and all-gather: the two halves of the low-bit all-reduce as
collectives of their own, for ZeRO/FSDP-style sharded training.

The reference has a low-bit ``reduce_scatter`` only inside its C++ backend
(``cpp/src/process_group_lowbit.cc:1670-1777``: pack every input shard, two all-to-alls,
dequantize and sum in source order) and forwards ``allgather`` to NCCL uncompressed
(``:1660-1668``).  Here both run through the fused sm_100a kernel on CUDA and through
list / single-tensor collectives elsewhere, with optional error feedback:

* reduce-scatter: residual over the whole ``[W * n]`` input (stage-1 semantics);
* all-gather: residual over this rank's ``[n]`` shard (stage-2 semantics).
"""

from __future__ import annotations

from typing import Hashable, Optional

import torch
import torch.distributed as dist

from ..quantization import (quantize_pack_tensor_blockwise, stage1_stream,
                            unpack_dequantize_tensor_blockwise)


def _immediate(async_op: bool):
    from ..api import _ImmediateWork

    return _ImmediateWork() if async_op else None


def _single(group) -> bool:
    from ..api import _uses_single_tensor_alltoall

    return _uses_single_tensor_alltoall(group)


def lowbit_reduce_scatter(owner, output: torch.Tensor, input: torch.Tensor, *,
                          group=None, ef_key: Optional[Hashable] = None,
                          async_op: bool = False):
    group = group or owner.pg
    world = dist.get_world_size(group)
    n = int(output.numel())
    if int(input.numel()) != world * n:
        raise ValueError(f"input must hold world*output elements ({world}*{n}), "
                         f"got {int(input.numel())}")
    if n == 0:
        return _immediate(async_op)
    bits, block, sr = owner.bitwidth, owner.block_size, owner.stochastic_rounding
    ef = owner._ef_for(input, ef_key)
    seed = owner._next_sr_seed()

    comm = owner._fused_comm(input, group) if input.is_contiguous() and output.is_contiguous() \
        else None
    if comm is not None:
        return comm.reduce_scatter(output, input, bitwidth=bits, block_size=block,
                                   stochastic=sr, seed=seed, ef=ef, async_op=async_op)

    flat = input.contiguous().view(-1)
    if ef is not None:
        from ..api import ShardPlan

        ef.ensure(ShardPlan(world, world * n), flat.device, False)
        flat = flat.to(torch.float32) + ef.stage1
    packed, scales = [], []
    for j in range(world):
        shard = flat[j * n:(j + 1) * n]
        p, s, _ = quantize_pack_tensor_blockwise(
            shard, bits, block_size=block, stochastic_rounding=sr, sr_seed=seed,
            sr_offset=j * n, sr_stream=stage1_stream(dist.get_rank(group)))
        packed.append(p)
        scales.append(s)
        if ef is not None:
            ef.stage1[j * n:(j + 1) * n] = shard - unpack_dequantize_tensor_blockwise(
                p, s, bits, n, block_size=block, dtype=torch.float32, device=flat.device)
    if _single(group):
        sp, ss = torch.stack(packed), torch.stack(scales)
        rp, rs = torch.empty_like(sp), torch.empty_like(ss)
        dist.all_to_all_single(rp, sp, group=group)
        dist.all_to_all_single(rs, ss, group=group)
    else:
        rp = [torch.empty_like(packed[0]) for _ in range(world)]
        rs = [torch.empty_like(scales[0]) for _ in range(world)]
        dist.all_to_all(rp, packed, group=group)
        dist.all_to_all(rs, scales, group=group)
    acc = torch.zeros(n, dtype=torch.float32, device=flat.device)
    for src in range(world):
        acc.add_(unpack_dequantize_tensor_blockwise(
            rp[src], rs[src], bits, n, block_size=block, dtype=torch.float32,
            device=flat.device))
    output.copy_(acc.view_as(output).to(output.dtype))
    return _immediate(async_op)


def lowbit_all_gather(owner, output: torch.Tensor, input: torch.Tensor, *,
                      group=None, ef_key: Optional[Hashable] = None,
                      async_op: bool = False):
    group = group or owner.pg
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = int(input.numel())
    if int(output.numel()) != world * n:
        raise ValueError(f"output must hold world*input elements ({world}*{n}), "
                         f"got {int(output.numel())}")
    if n == 0:
        return _immediate(async_op)
    bits, block, sr = owner.bitwidth, owner.block_size, owner.stochastic_rounding
    ef = owner._ef_for(input, ef_key)
    seed = owner._next_sr_seed()

    comm = owner._fused_comm(input, group) if input.is_contiguous() and output.is_contiguous() \
        else None
    if comm is not None:
        return comm.all_gather(output, input, bitwidth=bits, block_size=block,
                               stochastic=sr, seed=seed, ef=ef, async_op=async_op)

    src = input.contiguous().view(-1)
    if ef is not None:
        if ef.stage2 is None or ef.stage2.numel() != n:
            ef.stage2 = torch.zeros(n, dtype=torch.float32, device=src.device)
        src = src.to(torch.float32) + ef.stage2
    p, s, _ = quantize_pack_tensor_blockwise(
        src, bits, block_size=block, stochastic_rounding=sr, sr_seed=seed,
        sr_offset=rank * n, sr_stream=1)
    if ef is not None:
        ef.stage2 = src - unpack_dequantize_tensor_blockwise(
            p, s, bits, n, block_size=block, dtype=torch.float32, device=src.device)
    gp = [torch.empty_like(p) for _ in range(world)]
    gs = [torch.empty_like(s) for _ in range(world)]
    dist.all_gather(gp, p, group=group)
    dist.all_gather(gs, s, group=group)
    out = output.view(-1)
    for j in range(world):
        out[j * n:(j + 1) * n] = unpack_dequantize_tensor_blockwise(
            gp[j], gs[j], bits, n, block_size=block, dtype=torch.float32,
            device=src.device).to(out.dtype)
    return _immediate(async_op)
