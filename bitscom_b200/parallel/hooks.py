"""Gradient synchronisation for data parallelism, overlapped with backward.

The reference synchronises gradients after backward, one parameter (or one ``torch.cat``
bucket) at a time, fully exposed (``benchmarks/train_llama7b_dp_pp_lowbit.py:168-178``,
``benchmarks/multimodel_stochastic_e2e_curve.py:207-244``); overlap is left to an
external hook that calls ``all_reduce_stream``.  Here:

* ``GradBucketSync`` works on slices of a flat fp32 gradient buffer: when a slice is
  final (``on_ready``) the fused low-bit all-reduce kernel is enqueued on a side stream
  behind an event, with the 1/world scaling fused in, and error-feedback residuals keyed
  by slice index;
* ``lowbit_ddp_comm_hook`` plugs the same kernel into ``torch.nn.parallel
  .DistributedDataParallel.register_comm_hook`` (25 MB buckets by default in DDP).
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils import timing as _timing


class GradBucketSync:
    def __init__(self, lowbit_group, flat_grads: torch.Tensor,
                 ranges: Sequence[Tuple[int, int]], *, mode: str = "flat",
                 local_group=None, inter_group=None, chunk_size: Optional[int] = None,
                 average: bool = True, overlap: bool = True, max_ctas: Optional[int] = None,
                 key_prefix: Optional[tuple] = None):
        if mode not in ("flat", "pipeline_a", "dense"):
            raise ValueError(f"unknown mode {mode!r}")
        self.group = lowbit_group
        self.flat = flat_grads
        self.ranges = list(ranges)
        self.mode = mode
        self.local_group, self.inter_group = local_group, inter_group
        self.chunk_size = chunk_size
        self.world = lowbit_group.world_size
        self.post_scale = 1.0 / self.world if average else 1.0
        self.overlap = overlap and flat_grads.is_cuda
        # grid cap of the fused kernel for buckets launched WHILE backward is still running:
        # the cooperative grid must fit next to the compute kernels that own the SMs then
        self.max_ctas = max_ctas
        # error-feedback residuals are kept per key by the group: two synchronisers that share
        # a group (one per model chunk) need distinct prefixes
        self.key_prefix = tuple(key_prefix) if key_prefix else ()
        self._overlapping = False
        self.stream = torch.cuda.Stream(device=flat_grads.device) if flat_grads.is_cuda else None
        self._works: List = []
        self._launched = set()

    def _bucket(self, idx: int) -> torch.Tensor:
        start, length = self.ranges[idx]
        return self.flat[start:start + length]

    def _launch(self, idx: int) -> None:
        bucket = self._bucket(idx)
        key = self.key_prefix + ("bucket", idx)
        if self.mode == "dense":
            dist.all_reduce(bucket, group=self.group.pg)
            if self.post_scale != 1.0:
                bucket.mul_(self.post_scale)
        elif self.mode == "pipeline_a" and self.local_group is not None:
            self.group.all_reduce(bucket, local_group=self.local_group,
                                  inter_group=self.inter_group, chunk_size=self.chunk_size,
                                  ef_key=key)
            if self.post_scale != 1.0:
                bucket.mul_(self.post_scale)
        elif bucket.is_cuda:
            self._works.append(self.group.all_reduce_stream(
                bucket, stream=torch.cuda.current_stream(bucket.device),
                post_scale=self.post_scale, ef_key=key,
                max_ctas=self.max_ctas if self._overlapping else None))
        else:
            self.group.all_reduce(bucket, ef_key=key)
            if self.post_scale != 1.0:
                bucket.mul_(self.post_scale)
        _timing.add("grad_buckets_synced")

    def on_ready(self, idx: int) -> None:
        """Gradients of slice ``idx`` are final on the current stream."""
        if self.world <= 1 or idx in self._launched:
            return
        self._launched.add(idx)
        if not self.overlap:
            self._launch(idx)
            return
        cur = torch.cuda.current_stream(self.flat.device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            self._launch(idx)

    def on_ready_overlapped(self, idx: int) -> None:
        """``on_ready`` for a bucket that becomes final while compute kernels keep running (a
        layer of the last micro-batch's backward): launched with the grid cap."""
        self._overlapping = True
        try:
            self.on_ready(idx)
        finally:
            self._overlapping = False

    def check(self, wait: bool = False) -> None:
        """Raise ``FusedCollectiveError`` if a fused kernel of this group gave up on a bounded
        wait (it then returned early and the bucket holds partial sums).  ``wait=False`` costs
        no synchronisation: it polls the events of the launched buckets and the communicators'
        host-mapped status records, so it reports what has failed SO FAR; ``wait=True`` first
        waits for every launched bucket (use it before gradients are consumed for something
        that cannot be undone, such as writing a checkpoint)."""
        pending = []
        for work in self._works:
            if wait:
                work.wait()
            elif not work.is_completed():
                pending.append(work)
        self._works = pending
        self.group.check_status()

    def finish(self) -> None:
        """Launch whatever has not been launched yet and order the current stream after
        all of it.  Failures that are already on record (an earlier step's bucket that ran
        into its time limit) raise here, before this step's optimizer runs; the handles of
        this step's buckets are kept and looked at again by the next ``finish`` / ``check``."""
        if self.world > 1:
            for idx in range(len(self.ranges)):
                self.on_ready(idx)
            if self.overlap:
                torch.cuda.current_stream(self.flat.device).wait_stream(self.stream)
            self.check(wait=False)
        self._launched.clear()


class _HookState:
    def __init__(self, lowbit_group, average: bool = True):
        self.group = lowbit_group
        self.average = average
        self.stream: Optional[torch.cuda.Stream] = None


def make_ddp_hook_state(lowbit_group, average: bool = True) -> _HookState:
    return _HookState(lowbit_group, average)


def lowbit_ddp_comm_hook(state, bucket):  # unannotated: DDP compares annotations by identity
    """DDP communication hook: low-bit all-reduce of the bucket on a side stream.

    The returned future is CUDA-aware: its completion event is recorded on the side
    stream, so DDP's finalisation waits for the collective without blocking backward.
    Residuals are keyed by the bucket index, which DDP keeps stable after its first
    iteration.
    """
    buf = bucket.buffer()
    group = state.group
    world = group.world_size
    scale = 1.0 / world if state.average else 1.0
    if not buf.is_cuda:
        group.all_reduce(buf, ef_key=("ddp", bucket.index()))
        if scale != 1.0:
            buf.mul_(scale)
        fut: torch.futures.Future = torch.futures.Future()
        fut.set_result(buf)
        return fut
    if state.stream is None:
        state.stream = torch.cuda.Stream(device=buf.device)
    state.stream.wait_stream(torch.cuda.current_stream(buf.device))
    with torch.cuda.stream(state.stream):
        if group.bitwidth < 8 and world > 1:
            group.all_reduce_stream(buf, stream=state.stream, post_scale=scale,
                                    ef_key=("ddp", bucket.index()))
        else:
            dist.all_reduce(buf, group=group.pg)
            if scale != 1.0:
                buf.mul_(scale)
        fut = torch.futures.Future(devices=[buf.device])
        fut.set_result(buf)
    return fut
