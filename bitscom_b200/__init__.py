"""bitscom_b200: Blackwell-native low-bit collectives for PyTorch.

Drop-in for the public API of Squirrel7ang/bitscom (``python/bitscom/__init__.py:19-51``):

    import bitscom_b200 as bitscom
    bitscom.init(bitwidth=4)
    torch.distributed.init_process_group(backend="lowbit")
    group = bitscom.LowBitGroup(bitwidth=4)
    group.all_reduce(tensor)
"""

from typing import Optional

from .quantization import DEFAULT_BLOCK_SIZE, SUPPORTED_BITWIDTHS
from .lowbit_backend import is_extension_available, register_lowbit_backend
from .api import LowBitGroup

__all__ = [
    "register_lowbit_backend",
    "is_extension_available",
    "LowBitGroup",
    "SUPPORTED_BITWIDTHS",
    "init",
]

__version__ = "0.1.0"


def init(
    bitwidth: int = 4,
    error_feedback: bool = False,
    error_feedback_mode: Optional[str] = None,
    block_size: int = DEFAULT_BLOCK_SIZE,
    stage2_error_feedback: Optional[bool] = None,
):
    """Register the ``lowbit`` backend; call before ``init_process_group``."""
    register_lowbit_backend(
        bitwidth=bitwidth,
        error_feedback=error_feedback,
        error_feedback_mode=error_feedback_mode,
        block_size=block_size,
        stage2_error_feedback=stage2_error_feedback,
    )
