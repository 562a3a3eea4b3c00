"""bitscom_b200: Blackwell-native low-bit collectives for PyTorch.

The package keeps the public names of Squirrel7ang/bitscom (``python/bitscom/__init__.py:19-51``)
so that ``import bitscom_b200 as bitscom`` is enough to switch:

    bitscom.init(bitwidth=4)                                   # registers the backend
    torch.distributed.init_process_group(backend="lowbit")
    bitscom.LowBitGroup(bitwidth=4).all_reduce(tensor)

What goes beyond the reference (error feedback on every path, seeded stochastic rounding, the
fused kernels, sharded collectives, failure handling) hangs off ``LowBitGroup`` and the
``parallel`` / ``utils`` subpackages.
"""

from typing import Optional

from . import quantization as _q
from .api import LowBitGroup
from .lowbit_backend import is_extension_available, register_lowbit_backend

__version__ = "0.1.0"
SUPPORTED_BITWIDTHS = _q.SUPPORTED_BITWIDTHS
DEFAULT_BLOCK_SIZE = _q.DEFAULT_BLOCK_SIZE

__all__ = ("init", "register_lowbit_backend", "is_extension_available", "LowBitGroup",
           "SUPPORTED_BITWIDTHS", "shutdown")


def init(bitwidth: int = 4, error_feedback: bool = False,
         error_feedback_mode: Optional[str] = None, block_size: int = DEFAULT_BLOCK_SIZE,
         stage2_error_feedback: Optional[bool] = None) -> None:
    """Register the ``lowbit`` torch.distributed backend with these codec options (one option
    set per process; a second call with other options raises).  Call it before
    ``torch.distributed.init_process_group(backend="lowbit")``."""
    options = dict(bitwidth=bitwidth, error_feedback=error_feedback,
                   error_feedback_mode=error_feedback_mode, block_size=block_size,
                   stage2_error_feedback=stage2_error_feedback)
    register_lowbit_backend(**options)


def shutdown() -> None:
    """Collective, orderly release of what this library holds across ranks.  Every rank calls
    it after its last collective and before ``torch.distributed.destroy_process_group()``:

    * the fused communicators' symmetric blocks are released with a handshake (own kernels
      finished -> barrier -> unmap the peers -> barrier -> free), so that no rank frees a block
      a peer still maps and no process exits with CUDA IPC mappings left to the driver;
    * a ``lowbit`` backend releases its own block the same way and shuts down its inner NCCL
      group, which ``destroy_process_group`` does not know about.

    Safe to call when nothing was created; idempotent.  (The reference has no counterpart: its
    backend's destructor destroys a raw NCCL communicator, ``cpp/src/process_group_lowbit.cc:400-415``.)
    """
    import sys

    import torch
    import torch.distributed as dist

    fused = sys.modules.get(__name__ + ".parallel.fused")
    if fused is not None and dist.is_initialized():
        fused.FusedLowBitComm.close_all()
    if not dist.is_initialized() or not torch.cuda.is_available():
        return
    seen = set()
    for pg in list(getattr(dist.distributed_c10d._world, "pg_map", {})):
        try:
            backend = pg._get_backend(torch.device("cuda"))
        except Exception:
            continue
        if id(backend) in seen or not hasattr(backend, "close_symmetric"):
            continue
        seen.add(id(backend))
        backend.shutdown()
