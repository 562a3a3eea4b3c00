"""Datasets and the data-parallel sampler.

``TextLineDataset`` keeps the reference's per-document behaviour
(``benchmarks/train_llama7b_dp_pp_lowbit.py:19-57``): one document per item, truncated to the
sequence length and padded with the pad id, which the loss ignores.  ``PackedTokenDataset``
is the throughput path: a token file cut into back-to-back windows, memory-mapped, no padding.
``DistributedBatchSampler`` deals whole batches to data-parallel ranks the way
``torch.utils.data.DistributedSampler`` deals items (``:100-106`` of the same file): every
rank sees the same number of batches, the order is a function of (seed, epoch) only."""

from __future__ import annotations

import os
from typing import Iterator, List, Optional

import numpy as np
import torch


class TextLineDataset:
    """One document per non-empty line of a UTF-8 text file."""

    def __init__(self, path: str, tokenizer, seq_length: int, max_documents: Optional[int] = None):
        self.tokenizer, self.seq_length = tokenizer, int(seq_length)
        with open(path, encoding="utf-8") as f:
            self.docs = [line.rstrip("\n") for line in f if line.strip()]
        if max_documents is not None:
            self.docs = self.docs[:max_documents]
        if not self.docs:
            raise ValueError(f"{path} holds no documents")

    def __len__(self) -> int:
        return len(self.docs)

    def __getitem__(self, idx: int) -> torch.Tensor:
        tok = self.tokenizer
        ids = tok.encode(self.docs[idx])
        if len(ids) < 2:
            ids = [tok.bos_id, tok.eos_id]
        ids = ids[:self.seq_length]
        ids = ids + [tok.pad_id] * (self.seq_length - len(ids))
        return torch.tensor(ids, dtype=torch.int64)


class PackedTokenDataset:
    """A flat token file (raw little-endian ``uint16`` / ``int32`` / ``int64``, or ``.npy``) cut
    into windows of ``seq_length`` tokens; the trailing partial window is dropped."""

    def __init__(self, path: str, seq_length: int, dtype: Optional[str] = None):
        self.seq_length = int(seq_length)
        if path.endswith(".npy"):
            self.tokens = np.load(path, mmap_mode="r")
        else:
            if dtype is None:
                dtype = {".u16": "uint16", ".i32": "int32", ".i64": "int64"}.get(
                    os.path.splitext(path)[1], "uint16")
            self.tokens = np.memmap(path, dtype=np.dtype(dtype).newbyteorder("<"), mode="r")
        self.windows = len(self.tokens) // self.seq_length
        if self.windows == 0:
            raise ValueError(f"{path} holds fewer than {seq_length} tokens")

    def __len__(self) -> int:
        return self.windows

    def __getitem__(self, idx: int) -> torch.Tensor:
        if not 0 <= idx < self.windows:
            raise IndexError(idx)
        lo = idx * self.seq_length
        return torch.from_numpy(np.asarray(self.tokens[lo:lo + self.seq_length], dtype=np.int64))


def tokenize_to_file(text_path: str, tokenizer, out_path: str, dtype: str = "uint16") -> int:
    """Tokenize a text file line by line into a flat token file; returns the token count."""
    limit = np.iinfo(np.dtype(dtype)).max
    if tokenizer.vocab_size - 1 > limit:
        raise ValueError(f"vocabulary of {tokenizer.vocab_size} does not fit {dtype}")
    total = 0
    with open(text_path, encoding="utf-8") as src, open(out_path, "wb") as dst:
        for line in src:
            if not line.strip():
                continue
            ids = np.asarray(tokenizer.encode(line.rstrip("\n")),
                             dtype=np.dtype(dtype).newbyteorder("<"))
            dst.write(ids.tobytes())
            total += len(ids)
    return total


class DistributedBatchSampler:
    """Index batches for one data-parallel rank.

    The dataset's indices are permuted with a generator seeded by ``seed + epoch`` (identical on
    all ranks), padded by wrapping around to a multiple of ``dp_size * batch_size`` (or cut down
    to one with ``drop_last``), and dealt round-robin: global batch ``g`` goes to rank
    ``g % dp_size``.  ``len()`` is therefore the same on every rank."""

    def __init__(self, num_items: int, batch_size: int, dp_size: int = 1, dp_rank: int = 0,
                 shuffle: bool = True, seed: int = 0, drop_last: bool = True):
        if not 0 <= dp_rank < dp_size:
            raise ValueError("dp_rank out of range")
        if num_items <= 0 or batch_size <= 0:
            raise ValueError("need a non-empty dataset and a positive batch size")
        self.n, self.batch, self.dp, self.rank = num_items, batch_size, dp_size, dp_rank
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch = 0
        stride = dp_size * batch_size
        self.total = (num_items // stride) * stride if drop_last else -(-num_items // stride) * stride
        if self.total == 0:
            raise ValueError(f"{num_items} items cannot fill one batch of {batch_size} on each of "
                             f"{dp_size} ranks")

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    def __len__(self) -> int:
        return self.total // (self.dp * self.batch)

    def __iter__(self) -> Iterator[List[int]]:
        if self.shuffle:
            g = torch.Generator().manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.n, generator=g).tolist()
        else:
            order = list(range(self.n))
        while len(order) < self.total:
            order += order[:self.total - len(order)]
        order = order[:self.total]
        for b in range(len(self)):
            lo = (b * self.dp + self.rank) * self.batch
            yield order[lo:lo + self.batch]
