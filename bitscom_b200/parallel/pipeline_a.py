"""Hierarchical low-bit all-reduce, "pipeline-A".

Behaviour of the reference's ``_hierarchical_lowbit_allreduce_pipeline_a``
(``python/bitscom/api.py:877-1163``): the flat bucket is cut into chunks
(``chunk_size`` elements, default a quarter of the bucket) and every chunk goes through

  local     dense ``reduce`` onto the local leader (or, with ``local_quantize``, a
            quantized all-gather that the leader dequantizes and sums),
  inter     the leaders run the flat low-bit all-reduce over ``inter_group`` on fp32,
            everybody then meets in a barrier on ``local_group``,
  finalize  the leader broadcasts the result inside ``local_group`` (dense, or packed
            bytes + scales with ``local_quantize``).

The leader of a local group is its first rank (the rank with ``global_rank % local_size
== 0`` in the reference's layout).  On CUDA, when there are fewer local ranks than global
ranks, chunks are software-pipelined over two streams: local(i) and finalize(i-2) on one,
inter(i-1) on the other.

Beyond the reference: the inter phase carries error feedback (both stages) with residuals
kept per (bucket, chunk); on CUDA nothing blocks the host: the caller's stream is ordered
after both lanes with events, and the per-chunk barrier of the reference (which blocks the
host under NCCL and orders nothing that the finalize broadcast does not order already) is
kept for CPU groups only.

The schedule below is data: a list of (lane, phase, chunk) steps with their
dependencies, executed either on one stream in order or on two streams with events.
The inter stage uses the fused sm_100a all-reduce kernel when the leaders' tensors are
on CUDA and the inter group sits on one NVSwitch domain.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..quantization import quantize_pack_tensor_blockwise, unpack_dequantize_tensor_blockwise

Step = Tuple[str, str, int]  # (lane, phase, chunk index)


def build_schedule(num_chunks: int) -> List[Step]:
    """Issue order of the two-lane software pipeline (warm-up, steady state, drain)."""
    steps: List[Step] = []
    for i in range(num_chunks + 2):
        if 0 <= i - 2 < num_chunks:
            steps.append(("intra", "finalize", i - 2))
        if i < num_chunks:
            steps.append(("intra", "local", i))
        if 0 <= i - 1 < num_chunks:
            steps.append(("inter", "inter", i - 1))
    return steps


def run_pipeline_a(owner, tensor: torch.Tensor, *, local_group, inter_group,
                   chunk_size: Optional[int], local_quantize: bool, ef_key=None) -> None:
    flat = tensor.contiguous().view(-1)
    if flat.numel() == 0:
        return
    chunk_elems = int(chunk_size) if chunk_size is not None else max(1, flat.numel() // 4)
    chunks = owner._split_flat_chunks(flat, chunk_elems)
    n = len(chunks)

    global_rank = dist.get_rank(owner.pg)
    local_rank = dist.get_rank(local_group)
    local_size = dist.get_world_size(local_group)
    global_size = dist.get_world_size(owner.pg)
    leader = local_rank == 0
    # dst / src of the local collectives are ranks of the DEFAULT group: owner.pg may be a
    # strided subgroup (a data-parallel group of a dp x pp mesh), where
    # ``global_rank - local_rank`` names somebody else
    leader_global = dist.get_global_rank(local_group, 0)
    bits, block, sr = owner.bitwidth, owner.block_size, owner.stochastic_rounding
    owner._comm_debug(
        f"pipeline_a start numel={int(flat.numel())} chunks={n} chunk_elems={chunk_elems} "
        f"local_rank={local_rank} local_size={local_size} global_rank={global_rank} "
        f"global_size={global_size} is_local_leader={leader}")

    reduced: List[Optional[torch.Tensor]] = [None] * n   # fp32 on the leader
    shapes: List[Optional[Tuple[torch.Tensor, torch.Tensor, int]]] = [None] * n

    def local_phase(i: int) -> None:
        chunk = chunks[i]
        if not local_quantize:
            dist.reduce(chunk, dst=leader_global, group=local_group, op=dist.ReduceOp.SUM)
            return
        p, s, numel = quantize_pack_tensor_blockwise(
            chunk, bits, block_size=block, stochastic_rounding=sr)
        shapes[i] = (p, s, numel)
        all_p = [torch.empty_like(p) for _ in range(local_size)]
        all_s = [torch.empty_like(s) for _ in range(local_size)]
        dist.all_gather(all_p, p, group=local_group)
        dist.all_gather(all_s, s, group=local_group)
        if leader:
            acc = torch.zeros(numel, dtype=torch.float32, device=chunk.device)
            for k in range(local_size):
                acc.add_(unpack_dequantize_tensor_blockwise(
                    all_p[k], all_s[k], bits, numel, block_size=block,
                    dtype=torch.float32, device=chunk.device))
            reduced[i] = acc

    def inter_phase(i: int) -> None:
        chunk = chunks[i]
        if leader:
            src = reduced[i] if local_quantize else chunk.to(dtype=torch.float32)
            # residuals belong to the chunk of the caller's bucket, not to the staging copy
            ef = owner._ef_for(chunk, None if ef_key is None else (ef_key, "chunk", i))
            comm = owner._fused_comm(src, inter_group) if src.is_cuda else None
            if comm is not None:  # in place on the fp32 staging copy
                comm.all_reduce(src, bitwidth=bits, block_size=block, stochastic=sr,
                                seed=owner._next_sr_seed(), ef=ef,
                                stage2=owner.stage2_error_feedback)
                reduced[i] = src
            elif ef is not None:
                reduced[i] = owner._lowbit_allreduce_via_alltoall_group(src, inter_group, ef)
            else:
                reduced[i] = owner._lowbit_allreduce_via_alltoall_group(src, inter_group)
        if not chunk.is_cuda:
            dist.barrier(group=local_group)

    def finalize_phase(i: int) -> None:
        chunk = chunks[i]
        if leader and chunk.is_cuda and reduced[i] is not None:
            # produced on the inter lane, read here: tell the allocator
            reduced[i].record_stream(torch.cuda.current_stream(chunk.device))
        if not local_quantize:
            buf = reduced[i].to(dtype=chunk.dtype) if leader else torch.empty_like(chunk)
            dist.broadcast(buf, src=leader_global, group=local_group)
            chunk.copy_(buf)
            return
        p0, s0, numel = shapes[i]
        if leader:
            p, s, _ = quantize_pack_tensor_blockwise(
                reduced[i], bits, block_size=block, stochastic_rounding=sr)
        else:
            p, s = torch.empty_like(p0), torch.empty_like(s0)
        dist.broadcast(p, src=leader_global, group=local_group)
        dist.broadcast(s, src=leader_global, group=local_group)
        chunk.copy_(unpack_dequantize_tensor_blockwise(
            p, s, bits, numel, block_size=block, dtype=torch.float32,
            device=chunk.device).to(dtype=chunk.dtype))

    phases = {"local": local_phase, "inter": inter_phase, "finalize": finalize_phase}

    if not owner._should_use_dual_stream_pipeline(
            is_cuda=flat.is_cuda, local_size=local_size, global_size=global_size):
        for i in range(n):
            local_phase(i)
            inter_phase(i)
            finalize_phase(i)
    else:
        lanes = {"intra": torch.cuda.Stream(device=flat.device),
                 "inter": torch.cuda.Stream(device=flat.device)}
        for s in lanes.values():
            s.wait_stream(torch.cuda.current_stream(flat.device))
        local_done = [torch.cuda.Event() for _ in range(n)]
        inter_done = [torch.cuda.Event() for _ in range(n)]
        for lane, phase, i in build_schedule(n):
            stream = lanes[lane]
            with torch.cuda.stream(stream):
                if phase == "inter":
                    stream.wait_event(local_done[i])
                elif phase == "finalize":
                    stream.wait_event(inter_done[i])
                phases[phase](i)
                if phase == "local":
                    local_done[i].record(stream)
                elif phase == "inter":
                    inter_done[i].record(stream)
        cur = torch.cuda.current_stream(flat.device)
        for s in lanes.values():
            cur.wait_stream(s)  # stream-ordered completion: the host does not wait
        flat.record_stream(lanes["intra"])
        flat.record_stream(lanes["inter"])

    if flat.data_ptr() != tensor.data_ptr():
        tensor.copy_(flat.view_as(tensor))
    owner._comm_debug("pipeline_a done")
