"""Tokenizers that work offline.

The reference's trainer downloads a Hugging Face tokenizer
(``benchmarks/train_llama7b_dp_pp_lowbit.py:72-88``).  Here ``--tokenizer`` names either
``bytes`` (UTF-8 bytes, no file needed), a SentencePiece ``.model`` file, or a local
directory holding a Hugging Face tokenizer; nothing is fetched from a network.  All of them
expose ``encode``, ``decode``, ``vocab_size`` and the ``pad_id`` / ``bos_id`` / ``eos_id``
the datasets need (``pad_id`` is 0 everywhere, which is the trainer's ``ignore_index``)."""

from __future__ import annotations

import os
from typing import List, Sequence


class ByteTokenizer:
    """UTF-8 bytes shifted by three: 0 = pad, 1 = bos, 2 = eos, byte b -> b + 3."""

    pad_id, bos_id, eos_id = 0, 1, 2
    vocab_size = 259

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        ids = [b + 3 for b in text.encode("utf-8")]
        return ([self.bos_id] if add_bos else []) + ids + ([self.eos_id] if add_eos else [])

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i - 3 for i in ids if i >= 3).decode("utf-8", errors="replace")


class SentencePieceTokenizer:
    """A SentencePiece model file.  Its ids are shifted up by one when the model itself has no
    padding piece, so that id 0 stays free for padding."""

    def __init__(self, model_path: str):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=model_path)
        self.shift = 0 if self.sp.pad_id() == 0 else 1
        self.pad_id = 0
        self.bos_id = self.sp.bos_id() + self.shift if self.sp.bos_id() >= 0 else 0
        self.eos_id = self.sp.eos_id() + self.shift if self.sp.eos_id() >= 0 else 0
        self.vocab_size = self.sp.get_piece_size() + self.shift

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        ids = [i + self.shift for i in self.sp.encode(text)]
        if add_bos and self.sp.bos_id() >= 0:
            ids = [self.bos_id] + ids
        if add_eos and self.sp.eos_id() >= 0:
            ids = ids + [self.eos_id]
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.sp.decode([int(i) - self.shift for i in ids if int(i) != self.pad_id])


class LocalHFTokenizer:
    """A Hugging Face tokenizer loaded from a local directory (``local_files_only``)."""

    def __init__(self, directory: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(directory, local_files_only=True)
        if self.tok.pad_token is None:
            self.tok.pad_token = self.tok.eos_token
        self.pad_id = int(self.tok.pad_token_id)
        self.bos_id = int(self.tok.bos_token_id if self.tok.bos_token_id is not None else 0)
        self.eos_id = int(self.tok.eos_token_id if self.tok.eos_token_id is not None else 0)
        self.vocab_size = len(self.tok)

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True) -> List[int]:
        return list(self.tok(text, add_special_tokens=add_bos)["input_ids"])

    def decode(self, ids: Sequence[int]) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=True)


def load_tokenizer(spec: str):
    """``bytes``, a ``*.model`` SentencePiece file, or a local tokenizer directory."""
    if spec in ("bytes", "byte", ""):
        return ByteTokenizer()
    if os.path.isfile(spec):
        return SentencePieceTokenizer(spec)
    if os.path.isdir(spec):
        return LocalHFTokenizer(spec)
    raise FileNotFoundError(
        f"tokenizer {spec!r}: expected 'bytes', a SentencePiece .model file or a local "
        "directory (no tokenizer is downloaded)")
