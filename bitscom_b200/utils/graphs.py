"""CUDA-graph capture of a fixed-shape training step.

Small models are bound by launch overhead, not by the GPU: GPT-2 medium issues about 1,500
kernels per step, each behind tens of microseconds of Python and autograd dispatch.
``GraphedStep`` runs a step function a few times eagerly (so that lazily created scratch
buffers, kernel attributes and allocator pools exist), captures one more run into a
``torch.cuda.CUDAGraph`` and from then on replays it: one launch per step.

What may be captured: forward + backward of a model built on this package's kernels (they
take the current stream, encode their TMA tensor maps on the host at launch time, which
bakes the static addresses into the graph, and allocate nothing outside torch's allocator),
``collect_autograd_grads``-style accumulation into flat buffers, and the flat optimizer.
What must stay outside: collectives (NCCL and the fused low-bit kernel, whose peers are not
part of this GPU's graph), anything that reads a value back to the host, and anything whose
shapes change between steps.

The reference has no counterpart (its trainers are eager torch programs).
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple, Union

import torch

Tensors = Union[torch.Tensor, Tuple[torch.Tensor, ...]]


class GraphedStep:
    """``step = GraphedStep(fn, example_inputs)``; ``out = step(*inputs)``.

    ``fn(*static_inputs)`` must do all its work on the current stream with fixed shapes and
    return a tensor or a tuple of tensors.  Inputs are copied into static buffers before each
    replay; the returned tensors are the graph's own output buffers (overwritten by the next
    call, clone them to keep a value).  ``reset`` is called after the eager warm-up runs and
    again after capture, e.g. to zero gradient accumulators those runs have touched.
    """

    def __init__(self, fn: Callable[..., Tensors], example_inputs: Sequence[torch.Tensor],
                 warmup: int = 3, reset: Optional[Callable[[], None]] = None,
                 capture_error_mode: str = "relaxed"):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device")
        self.fn = fn
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if reset is not None:
            reset()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode=capture_error_mode):
            self.static_outputs = fn(*self.static_inputs)
        if reset is not None:
            reset()
        self.replays = 0

    def __call__(self, *inputs: torch.Tensor) -> Tensors:
        if len(inputs) != len(self.static_inputs):
            raise ValueError(f"expected {len(self.static_inputs)} inputs, got {len(inputs)}")
        for dst, src in zip(self.static_inputs, inputs):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError("a graphed step needs the shapes and dtypes it was captured with")
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_outputs
