"""Prefetching loader: a background thread assembles the next steps' batches in pinned host
memory while the GPU works on the current one, so that the step's host-to-device copy is a
plain asynchronous copy from memory that is already resident.

A step's batch has the trainer's shape ``[micro_batches, micro_batch_size, seq_length]``
(int64).  The reference leaves this to ``torch.utils.data.DataLoader(pin_memory=True,
num_workers=...)`` (``benchmarks/train_llama7b_dp_pp_lowbit.py:107-115``); here the ring of
pinned buffers is owned by the loader, allocated once and reused, and nothing is pickled
between processes."""

from __future__ import annotations

import queue
import threading
from typing import Iterator, List, Optional

import torch

from .dataset import DistributedBatchSampler, PackedTokenDataset, TextLineDataset
from .tokenizer import load_tokenizer


class SyntheticTokens:
    """Uniform token ids in ``[1, vocab)``: item ``i`` is a function of ``(seed, i)`` only."""

    def __init__(self, vocab_size: int, seq_length: int, num_items: int = 1 << 20, seed: int = 0):
        self.vocab, self.seq_length, self.n, self.seed = vocab_size, seq_length, num_items, seed

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, idx: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(self.seed * 1000003 + idx)
        return torch.randint(1, self.vocab, (self.seq_length,), generator=g)


class PrefetchLoader:
    """Iterates over one epoch of step batches ``[micro_batches, micro_batch_size, seq]``.

    ``depth`` host buffers (pinned when a GPU is present) circulate between the producer thread
    and the consumer.  A buffer handed out is not refilled before the consumer has taken two
    more batches, and, when the consumer calls :meth:`mark_consumed` after enqueuing its
    asynchronous device copy, not before that copy has actually run (a CUDA event guards the
    buffer)."""

    def __init__(self, dataset, sampler: DistributedBatchSampler, micro_batches: int,
                 micro_batch_size: int, depth: int = 4, pin: Optional[bool] = None):
        if sampler.batch != micro_batches * micro_batch_size:
            raise ValueError("the sampler's batch must be micro_batches * micro_batch_size")
        if depth < 3:
            raise ValueError("depth must be at least 3 (in use, cooling down, being filled)")
        self.dataset, self.sampler = dataset, sampler
        self.shape = (micro_batches, micro_batch_size, dataset.seq_length)
        self.pinned = torch.cuda.is_available() if pin is None else bool(pin)
        self.buffers = [torch.empty(self.shape, dtype=torch.int64) for _ in range(depth)]
        if self.pinned:
            self.buffers = [b.pin_memory() for b in self.buffers]
        self.depth = depth
        self._events = [None] * depth
        self._last_slot: Optional[int] = None

    def __len__(self) -> int:
        return len(self.sampler)

    def set_epoch(self, epoch: int) -> None:
        self.sampler.set_epoch(epoch)

    def mark_consumed(self) -> None:
        """Call after enqueuing the device copy of the batch most recently taken: records an
        event on the current stream; the buffer is not refilled before it has completed."""
        if self._last_slot is not None and torch.cuda.is_available():
            ev = torch.cuda.Event()
            ev.record()
            self._events[self._last_slot] = ev

    def __iter__(self) -> Iterator[torch.Tensor]:
        free: "queue.Queue[Optional[int]]" = queue.Queue()
        ready: "queue.Queue[object]" = queue.Queue()
        for i in range(self.depth):
            free.put(i)
        stop = threading.Event()

        def produce():
            try:
                for indices in self.sampler:
                    slot = free.get()
                    if slot is None or stop.is_set():
                        return
                    ev, self._events[slot] = self._events[slot], None
                    if ev is not None:
                        ev.synchronize()
                    flat = self.buffers[slot].view(-1, self.shape[2])
                    for row, idx in enumerate(indices):
                        flat[row].copy_(self.dataset[idx])
                    ready.put(slot)
                ready.put(None)
            except BaseException as exc:  # surface loader errors in the training thread
                ready.put(exc)

        thread = threading.Thread(target=produce, name="bitscom-prefetch", daemon=True)
        thread.start()
        cooling: List[int] = []  # slots handed out earlier, oldest first
        try:
            while True:
                item = ready.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                self._last_slot = item
                yield self.buffers[item]
                cooling.append(item)
                while len(cooling) > 1:  # the batch before the previous one may be refilled
                    free.put(cooling.pop(0))
        finally:
            stop.set()
            free.put(None)  # wake a producer blocked on an empty free list
            thread.join(timeout=5)
            self._last_slot = None


def build_loader(dataset_spec: str, tokenizer_spec: str, *, seq_length: int, vocab_size: int,
                 micro_batches: int, micro_batch_size: int, dp_size: int = 1, dp_rank: int = 0,
                 seed: int = 0, shuffle: bool = True, depth: int = 4) -> PrefetchLoader:
    """``dataset_spec``: ``synthetic``, a text file (one document per line, tokenized with
    ``tokenizer_spec``), or a token file (``.bin`` / ``.u16`` / ``.i32`` / ``.i64`` / ``.npy``)."""
    if dataset_spec == "synthetic":
        ds = SyntheticTokens(vocab_size, seq_length, seed=seed)
    elif dataset_spec.endswith((".bin", ".u16", ".i32", ".i64", ".npy")):
        ds = PackedTokenDataset(dataset_spec, seq_length)
    else:
        tok = load_tokenizer(tokenizer_spec)
        if tok.vocab_size > vocab_size:
            raise ValueError(f"tokenizer vocabulary {tok.vocab_size} exceeds the model's "
                             f"{vocab_size}")
        ds = TextLineDataset(dataset_spec, tok, seq_length)
    sampler = DistributedBatchSampler(len(ds), micro_batches * micro_batch_size, dp_size, dp_rank,
                                      shuffle=shuffle, seed=seed)
    return PrefetchLoader(ds, sampler, micro_batches, micro_batch_size, depth=depth)
