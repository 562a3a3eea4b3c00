"""Registration of the ``lowbit`` ``torch.distributed`` backend and its options.

    import bitscom_b200 as bitscom
    bitscom.init(bitwidth=4, error_feedback_mode="ef21_plus")
    torch.distributed.init_process_group(backend="lowbit", ...)

Option resolution matches the reference (``python/bitscom/lowbit_backend.py:70-164``):
one option set per process; ``error_feedback=True`` means mode ``legacy``; mode strings
``auto/none/legacy/ef/ef21/ef21_plus/ef21+``; stage-2 feedback defaults to "on only for
ef21_plus"; registering twice with the same options is a no-op, with different options
an error.  The backend itself is the C++ class ``ProcessGroupLowBit`` in
``csrc/backend.cc`` (module ``bitscom_b200._lowbit_c``).
"""

from __future__ import annotations

from typing import Optional

import torch.distributed as dist

from .quantization import DEFAULT_BLOCK_SIZE, SUPPORTED_BITWIDTHS

try:
    from ._ext import load_backend_extension as _load_ext

    _mod = _load_ext()
    create_backend = _mod.create_backend
    ProcessGroupLowBit = _mod.ProcessGroupLowBit
    LowBitOptions = _mod.LowBitOptions
    _HAS_EXTENSION = True
    _EXTENSION_IMPORT_ERROR = None
except Exception as exc:  # the extension needs a build; see bitscom_b200/_ext.py
    create_backend = None
    ProcessGroupLowBit = None
    LowBitOptions = None
    _HAS_EXTENSION = False
    _EXTENSION_IMPORT_ERROR = exc

_REGISTERED = False
_BACKEND_BITWIDTH = 4
_BACKEND_ERROR_FEEDBACK = False
_BACKEND_ERROR_FEEDBACK_MODE = "none"
_BACKEND_BLOCK_SIZE = DEFAULT_BLOCK_SIZE
_BACKEND_STAGE2_ERROR_FEEDBACK = False

_EF_ALIASES = {
    "auto": "auto", "none": "none", "legacy": "legacy", "ef": "legacy",
    "ef21": "ef21", "ef21_plus": "ef21_plus", "ef21+": "ef21_plus",
}


def _create_lowbit_pg(store, rank, size, timeout):
    """Factory called by ``init_process_group(backend="lowbit")``."""
    if not _HAS_EXTENSION:
        raise RuntimeError(
            "bitscom_b200 C++ extension is not available; run "
            "`python -c 'import __graft_entry__ as g; g.build()'` first."
        ) from _EXTENSION_IMPORT_ERROR
    return create_backend(
        store=store, rank=rank, size=size, timeout=timeout,
        bitwidth=_BACKEND_BITWIDTH,
        error_feedback=_BACKEND_ERROR_FEEDBACK,
        error_feedback_mode=_BACKEND_ERROR_FEEDBACK_MODE,
        block_size=_BACKEND_BLOCK_SIZE,
        stage2_error_feedback=_BACKEND_STAGE2_ERROR_FEEDBACK,
    )


def _normalize_error_feedback_mode(error_feedback_mode: Optional[str]) -> str:
    if error_feedback_mode is None:
        return "none"
    mode = str(error_feedback_mode).strip().lower()
    if mode not in _EF_ALIASES:
        raise ValueError(
            "error_feedback_mode must be one of: " + ", ".join(sorted(_EF_ALIASES)))
    return _EF_ALIASES[mode]


def resolve_options(bitwidth, error_feedback, error_feedback_mode, block_size,
                    stage2_error_feedback):
    """Validated (bitwidth, error_feedback, mode, block_size, stage2) tuple."""
    if bitwidth not in SUPPORTED_BITWIDTHS:
        raise ValueError(f"bitwidth must be one of {SUPPORTED_BITWIDTHS}, got {bitwidth}")
    if block_size <= 0:
        raise ValueError(f"block_size must be > 0, got {block_size}")
    if error_feedback_mode is None:
        mode = "legacy" if error_feedback else "none"
    else:
        mode = _normalize_error_feedback_mode(error_feedback_mode)
        if mode == "auto":
            mode = "legacy" if error_feedback else "none"
        error_feedback = mode != "none"
    stage2 = (mode == "ef21_plus") if stage2_error_feedback is None \
        else bool(stage2_error_feedback)
    return int(bitwidth), bool(error_feedback), mode, int(block_size), stage2


def register_lowbit_backend(
    bitwidth: int = 4,
    error_feedback: bool = False,
    error_feedback_mode: Optional[str] = None,
    block_size: int = DEFAULT_BLOCK_SIZE,
    stage2_error_feedback: Optional[bool] = None,
):
    """Make ``backend="lowbit"`` available to ``init_process_group``."""
    global _REGISTERED, _BACKEND_BITWIDTH, _BACKEND_ERROR_FEEDBACK
    global _BACKEND_ERROR_FEEDBACK_MODE, _BACKEND_BLOCK_SIZE, _BACKEND_STAGE2_ERROR_FEEDBACK

    asked = resolve_options(bitwidth, error_feedback, error_feedback_mode, block_size,
                            stage2_error_feedback)
    current = (_BACKEND_BITWIDTH, _BACKEND_ERROR_FEEDBACK, _BACKEND_ERROR_FEEDBACK_MODE,
               _BACKEND_BLOCK_SIZE, _BACKEND_STAGE2_ERROR_FEEDBACK)
    if _REGISTERED:
        if asked != current:
            names = ("bitwidth", "error_feedback", "error_feedback_mode", "block_size",
                     "stage2_error_feedback")
            diff = ", ".join(f"{n}={c!r} (you specified {a!r})"
                             for n, c, a in zip(names, current, asked))
            raise RuntimeError(
                "lowbit backend is already registered with different options: " + diff)
        return

    (_BACKEND_BITWIDTH, _BACKEND_ERROR_FEEDBACK, _BACKEND_ERROR_FEEDBACK_MODE,
     _BACKEND_BLOCK_SIZE, _BACKEND_STAGE2_ERROR_FEEDBACK) = asked

    if not _HAS_EXTENSION:
        raise RuntimeError(
            "bitscom_b200 C++ extension is not available; build it before registering "
            "the backend (`python -c 'import __graft_entry__ as g; g.build()'`)."
        ) from _EXTENSION_IMPORT_ERROR

    dist.Backend.register_backend(name="lowbit", func=_create_lowbit_pg,
                                  devices=["cpu", "cuda"])
    _REGISTERED = True


def is_extension_available() -> bool:
    return _HAS_EXTENSION
