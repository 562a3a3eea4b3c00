"""Codec kernels: blockwise quantize+pack / unpack+dequantize, per-tensor quantize,
pack / unpack.  Same surface as the reference's ``_lowbit_cuda`` extension
(``cpp/src/lowbit_cuda_bindings.cpp:38-87``) with bf16, 12/16-bit and a seed added."""

from __future__ import annotations

import ctypes
import itertools
import os
import time
from typing import Optional, Tuple

import torch

from . import _native
from ._native import DTYPE_CODE, check, ptr, stream_ptr

_lib = None
_seed_counter = itertools.count(1)


def _get():
    global _lib
    if _lib is None:
        lib = _native.load("bcom_codec")
        if lib is not None:
            lib.bcom_blockwise_quantize_pack.argtypes = [
                ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p,
                ctypes.c_void_p]
            lib.bcom_blockwise_unpack_dequantize.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
            lib.bcom_quantize_per_tensor.argtypes = [
                ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                ctypes.c_uint, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                ctypes.c_void_p]
            lib.bcom_dequantize_per_tensor.argtypes = [
                ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p,
                ctypes.c_void_p]
            lib.bcom_pack.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                      ctypes.c_void_p, ctypes.c_void_p]
            lib.bcom_unpack.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                        ctypes.c_void_p, ctypes.c_void_p]
        _lib = lib if lib is not None else False
    return _lib or None


def available() -> bool:
    return _native.cuda_present() and _get() is not None


def supports_dtype(dtype: torch.dtype) -> bool:
    return dtype in DTYPE_CODE


def supports_blockwise(bitwidth: int, block_size: int) -> bool:
    lib = _get()
    if lib is None:
        return False
    return bool(lib.bcom_codec_fast_block(block_size)) or bool(
        lib.bcom_codec_generic_ok(bitwidth, block_size))


def fresh_seed() -> int:
    """A new seed per call for callers that did not fix one (reference behaviour:
    ``cpp/src/lowbit_cuda_kernels.cu:279-281`` seeds from the clock)."""
    return (time.monotonic_ns() ^ (next(_seed_counter) * 0x9E3779B97F4A7C15) ^ os.getpid()) \
        & 0xFFFFFFFFFFFFFFFF


def _key(sr_seed: Optional[int], stochastic: bool, stream: int) -> int:
    from ..quantization import sr_key

    if not stochastic:
        return 0
    return sr_key(fresh_seed() if sr_seed is None else sr_seed, stream)


def packed_nbytes(numel: int, bitwidth: int) -> int:
    if bitwidth == 12:
        return 3 * ((numel + 1) // 2)
    if bitwidth == 16:
        return 2 * numel
    return -(-numel * bitwidth // 8)


def blockwise_quantize_pack(x: torch.Tensor, bitwidth: int, block_size: int,
                            stochastic: bool = False, sr_seed: Optional[int] = None,
                            sr_offset: int = 0, sr_stream: int = 0
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    lib = _get()
    x = x.detach().contiguous().view(-1)
    n = x.numel()
    packed = torch.empty(packed_nbytes(n, bitwidth), dtype=torch.uint8, device=x.device)
    scales = torch.empty(-(-n // block_size), dtype=torch.float16, device=x.device)
    with _native.on_device(x.device):
        check(lib.bcom_blockwise_quantize_pack(
            ptr(x), DTYPE_CODE[x.dtype], n, bitwidth, block_size, int(bool(stochastic)),
            _key(sr_seed, stochastic, sr_stream), int(sr_offset) & 0xFFFFFFFF,
            ptr(packed), ptr(scales), stream_ptr(x.device)), "blockwise_quantize_pack")
    return packed, scales


def blockwise_unpack_dequantize(packed: torch.Tensor, scales: torch.Tensor, bitwidth: int,
                                numel: int, block_size: int,
                                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    lib = _get()
    packed = packed.contiguous().view(-1)
    scales = scales.contiguous().view(-1)
    if packed.numel() < packed_nbytes(numel, bitwidth):
        raise ValueError("packed buffer is smaller than numel codes")
    if scales.numel() != -(-numel // block_size):
        raise ValueError(
            f"scales length {scales.numel()} does not match expected blocks "
            f"{-(-numel // block_size)}")
    out = torch.empty(numel, dtype=dtype, device=packed.device)
    with _native.on_device(packed.device):
        check(lib.bcom_blockwise_unpack_dequantize(
            ptr(packed), ptr(scales), bitwidth, numel, block_size, ptr(out),
            DTYPE_CODE[dtype], stream_ptr(packed.device)), "blockwise_unpack_dequantize")
    return out


def quantize_per_tensor(x: torch.Tensor, bitwidth: int, stochastic: bool = False,
                        sr_seed: Optional[int] = None, sr_offset: int = 0
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (int16 codes shaped like x, 0-dim fp32 scale on the device)."""
    lib = _get()
    flat = x.detach().contiguous().view(-1)
    q = torch.empty(flat.numel(), dtype=torch.int16, device=x.device)
    scratch = torch.empty(2, dtype=torch.float32, device=x.device)
    with _native.on_device(x.device):
        check(lib.bcom_quantize_per_tensor(
            ptr(flat), DTYPE_CODE[flat.dtype], flat.numel(), bitwidth, int(bool(stochastic)),
            _key(sr_seed, stochastic, 2), int(sr_offset) & 0xFFFFFFFF,
            ptr(scratch[0:1]), ptr(q), ptr(scratch[1:2]), stream_ptr(x.device)),
            "quantize_per_tensor")
    return q.view(x.shape), scratch[1]


def dequantize_per_tensor(q: torch.Tensor, scale: float) -> torch.Tensor:
    lib = _get()
    flat = q.contiguous().view(-1)
    out = torch.empty(flat.numel(), dtype=torch.float32, device=q.device)
    with _native.on_device(q.device):
        check(lib.bcom_dequantize_per_tensor(ptr(flat), flat.numel(), float(scale), ptr(out),
                                             stream_ptr(q.device)), "dequantize_per_tensor")
    return out.view(q.shape)


def pack(q: torch.Tensor, bitwidth: int) -> torch.Tensor:
    lib = _get()
    flat = q.contiguous().view(-1)
    out = torch.empty(packed_nbytes(flat.numel(), bitwidth), dtype=torch.uint8, device=q.device)
    with _native.on_device(q.device):
        check(lib.bcom_pack(ptr(flat), flat.numel(), bitwidth, ptr(out), stream_ptr(q.device)),
              "pack")
    return out


def unpack(packed: torch.Tensor, bitwidth: int, numel: int) -> torch.Tensor:
    lib = _get()
    packed = packed.contiguous().view(-1)
    if packed.numel() < packed_nbytes(numel, bitwidth):
        raise ValueError("packed buffer is smaller than numel codes")
    out = torch.empty(numel, dtype=torch.int16, device=packed.device)
    with _native.on_device(packed.device):
        check(lib.bcom_unpack(ptr(packed), numel, bitwidth, ptr(out),
                              stream_ptr(packed.device)), "unpack")
    return out
