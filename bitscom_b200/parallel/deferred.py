"""Deferred weight-gradient work for pipeline parallelism.

In 1F1B a stage's backward step produces two things: the gradient of its input, which the
previous stage is waiting for, and the weight gradients, which nothing downstream needs
before the optimizer step.  Inside a ``DeferredWork`` context the linear layers only queue
their weight-gradient GEMMs; the pipeline runner sends the input gradient first and runs the
queue while the transfer is in flight, which takes the weight-gradient time off the critical
path between stages (the "zero-bubble" split of backward into B and W).  The reference's
trainer uses torch's GPipe schedule and has nothing comparable
(``benchmarks/train_llama7b_dp_pp_lowbit.py:240-264``).

Queued closures keep their operands (the layer input and the output gradient) alive until
``flush``; nothing may modify those tensors in between.
"""

from __future__ import annotations

from typing import Callable, List, Optional


class DeferredWork:
    _active: Optional["DeferredWork"] = None  # process-wide: autograd runs on its own thread

    def __init__(self) -> None:
        self._items: List[Callable[[], None]] = []
        self.queued = 0
        self.flushes = 0

    @classmethod
    def active(cls) -> Optional["DeferredWork"]:
        return cls._active

    def add(self, fn: Callable[[], None]) -> None:
        self._items.append(fn)
        self.queued += 1

    def __len__(self) -> int:
        return len(self._items)

    def flush(self) -> None:
        """Run everything queued so far, in the order it was queued."""
        items, self._items = self._items, []
        for fn in items:
            fn()
        if items:
            self.flushes += 1

    def __enter__(self) -> "DeferredWork":
        if DeferredWork._active is not None:
            raise RuntimeError("DeferredWork contexts do not nest")
        DeferredWork._active = self
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        DeferredWork._active = None
        if exc_type is not None:
            self._items.clear()  # the step failed: do not touch the gradient buffers
        return False
