"""Shared helpers for calling the native libraries through ctypes."""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _build

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class NativeError(RuntimeError):
    pass


def cuda_present() -> bool:
    return torch.cuda.is_available()


def load(name: str) -> Optional[ctypes.CDLL]:
    """Load a native library.

    Without a GPU the library is not needed and ``None`` is returned when it cannot be
    loaded.  With a GPU a missing or broken library is an error: falling back to torch
    ops silently would hide that the kernels are not running.
    """
    try:
        return _build.load_library(name)
    except Exception as exc:
        if cuda_present() and os.environ.get("BITSCOM_ALLOW_FALLBACK", "0") != "1":
            raise NativeError(
                f"bitscom_b200: native library '{name}' could not be loaded on a GPU "
                f"machine: {exc}") from exc
        return None


def stream_ptr(device: Optional[torch.device] = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def on_device(device: torch.device):
    """Context that makes ``device`` current for a native launch.  When it already is (one
    process per GPU, the normal case) this is a no-op object: the full ``torch.cuda.device``
    guard costs several microseconds per call, which is visible for small kernels."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_ARG_ERRORS = {
    1001: "a leading dimension or N is not a multiple of 8 elements",
    1002: "an operand is not 16-byte aligned",
    1003: "the tensor map of A could not be encoded",
    1004: "the tensor map of B could not be encoded",
    1005: "the kernel's shared-memory attribute could not be set",
}


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched by this process so far (counted where the launch
    functions of the native libraries are called; library calls that launch nothing pass
    ``launches=0``)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += int(n)


def check(code: int, what: str, launches: int = 1) -> None:
    """Raise on a non-zero return code of a native call; on success count the ``launches``
    kernels the call enqueued."""
    global _launches
    if code == 0:
        _launches += launches
        return
    if code in _ARG_ERRORS:
        raise NativeError(f"{what}: {_ARG_ERRORS[code]}")
    raise NativeError(f"{what} failed with CUDA error {code}")
