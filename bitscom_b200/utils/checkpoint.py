"""Checkpoint / resume: one file per rank holding weights, optimizer moments, the step
counter, error-feedback residuals and the stochastic-rounding call counter.

The reference keeps residuals only in process memory and never writes a checkpoint (its
trainer parses ``--output_dir`` and ignores it,
``benchmarks/train_llama7b_dp_pp_lowbit.py:191``); without the residuals a resumed run
does not continue the same trajectory.
"""

from __future__ import annotations

import os
from typing import Any

import torch


def _to_cpu(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def checkpoint_path(directory: str, rank: int) -> str:
    return os.path.join(directory, f"rank{rank:05d}.pt")


def save_checkpoint(directory: str, state: dict, rank: int = 0) -> str:
    os.makedirs(directory, exist_ok=True)
    path = checkpoint_path(directory, rank)
    tmp = path + ".tmp"
    torch.save(_to_cpu(state), tmp)
    os.replace(tmp, path)
    return path


def load_checkpoint(directory: str, rank: int = 0, map_location="cpu") -> dict:
    return torch.load(checkpoint_path(directory, rank), map_location=map_location,
                      weights_only=False)
