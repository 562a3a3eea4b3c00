"""C++ CPU codec (``csrc/cpu_codec.cc``): blockwise quantize+pack / unpack+dequantize of
fp32 CPU tensors, bit-exact with ``bitscom_b200.quantization`` on CPU."""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _build

_lib = None


def _get():
    global _lib
    if _lib is None:
        try:
            lib = _build.load_library("bcom_cpu")
            vp, ll, ci, cu = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_uint
            lib.bcom_cpu_packed_nbytes.argtypes = [ll, ci]
            lib.bcom_cpu_packed_nbytes.restype = ll
            lib.bcom_cpu_blockwise_quantize_pack_mt.argtypes = [vp, ll, ci, ci, ci, cu, cu, vp,
                                                                vp, ci]
            lib.bcom_cpu_blockwise_unpack_dequantize_mt.argtypes = [vp, vp, ci, ll, ci, vp, ci]
            _lib = lib
        except Exception:
            _lib = False
    return _lib or None


def available() -> bool:
    return _get() is not None


def blockwise_quantize_pack(x: torch.Tensor, bitwidth: int, block_size: int,
                            stochastic: bool = False, sr_seed: Optional[int] = None,
                            sr_offset: int = 0, sr_stream: int = 0
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    from ..quantization import sr_key

    lib = _get()
    flat = x.detach().to(torch.float32).contiguous().view(-1)
    n = flat.numel()
    packed = torch.empty(int(lib.bcom_cpu_packed_nbytes(n, bitwidth)), dtype=torch.uint8)
    scales = torch.empty(-(-n // block_size), dtype=torch.float16)
    if stochastic and sr_seed is None:
        raise ValueError("the C++ CPU codec needs a seed for stochastic rounding")
    key = sr_key(sr_seed, sr_stream) if stochastic else 0
    rc = lib.bcom_cpu_blockwise_quantize_pack_mt(
        flat.data_ptr(), n, bitwidth, block_size, int(bool(stochastic)), key,
        int(sr_offset) & 0xFFFFFFFF, packed.data_ptr(), scales.data_ptr(),
        torch.get_num_threads())
    if rc:
        raise ValueError("bad arguments for the CPU codec")
    return packed, scales


def blockwise_unpack_dequantize(packed: torch.Tensor, scales: torch.Tensor, bitwidth: int,
                                numel: int, block_size: int) -> torch.Tensor:
    lib = _get()
    packed = packed.contiguous().view(-1)
    scales = scales.contiguous().view(-1)
    out = torch.empty(numel, dtype=torch.float32)
    rc = lib.bcom_cpu_blockwise_unpack_dequantize_mt(
        packed.data_ptr(), scales.data_ptr(), bitwidth, numel, block_size, out.data_ptr(),
        torch.get_num_threads())
    if rc:
        raise ValueError("bad arguments for the CPU codec")
    return out
