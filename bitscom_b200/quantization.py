"""Symmetric absmax quantizer and bit-packer for low-bit communication.

This is the host-side statement of the codec: pure torch, exact on CPU, and the
numerics contract every CUDA kernel in ``csrc/`` is tested against bit for bit.
It keeps the wire format and public names of the reference quantizer
(``python/bitscom/quantization.py:31-424`` in Squirrel7ang/bitscom):

* codes: 1-bit is the unsigned pair {0, 1}; otherwise two's-complement range
  ``[-2^(b-1), 2^(b-1)-1]``;
* blockwise: per block ``scale = absmax / qmax`` (1.0 for an all-zero block),
  rounded to fp16 for the wire, magnitudes divided by that fp16 value, rounded
  half-to-even or stochastically, sign re-applied (dropped for 1-bit), clamped;
* packing: offset code ``q - qmin``, first element in the least-significant
  bits; 12-bit pairs in 3 bytes; 16-bit as little-endian int16.

Two things are added on top of the reference behaviour:

* ``sr_seed`` / ``sr_offset``: a counter-based random stream (``sr_uniform``)
  shared with the CUDA kernels, so stochastic rounding is reproducible and a
  fused multi-GPU kernel can be checked bit-exactly on CPU.  Without a seed the
  CPU path draws from torch's global generator, as the reference does.
* CUDA tensors of fp32 / fp16 / **bf16** go through the hand-written sm_100a
  codec kernels (``bitscom_b200.ops.codec``) for bitwidths 1/2/4/8/12/16.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

SUPPORTED_BITWIDTHS = (1, 2, 4, 8, 12, 16)
DEFAULT_BLOCK_SIZE = 256

_U32 = 0xFFFFFFFF


def _load_cuda_codec():
    try:
        from .ops import codec as _codec

        return _codec if _codec.available() else None
    except Exception:  # pragma: no cover - depends on the build
        return None


_CUDA = _load_cuda_codec()
_HAS_CUDA_KERNELS = _CUDA is not None

_CPU_NATIVE = None  # False once loading has failed


def _cpu_codec():
    """The C++ CPU codec (bit-equal to the torch-op path below, several times faster), or
    ``None`` when it cannot be built / loaded or ``BITSCOM_CPU_CODEC=0`` asks for torch ops."""
    global _CPU_NATIVE
    if _CPU_NATIVE is None:
        try:
            import os

            from .ops import cpu_codec as _c

            _CPU_NATIVE = _c if (os.environ.get("BITSCOM_CPU_CODEC", "1") != "0"
                                 and _c.available()) else False
        except Exception:  # pragma: no cover - depends on the toolchain
            _CPU_NATIVE = False
    return _CPU_NATIVE or None


def validate_bitwidth(bitwidth: int) -> None:
    if bitwidth not in SUPPORTED_BITWIDTHS:
        raise ValueError(
            f"bitwidth must be one of {SUPPORTED_BITWIDTHS}, got {bitwidth}"
        )


def _quant_bounds(bitwidth: int) -> Tuple[int, int]:
    """(qmin, qmax) of the code range for ``bitwidth``."""
    if bitwidth == 1:
        return 0, 1
    half = 1 << (bitwidth - 1)
    return -half, half - 1


def _check_block_size(block_size: int) -> None:
    if block_size <= 0:
        raise ValueError(f"block_size must be > 0, got {block_size}")


# ----------------------------------------------------------------------------------
# counter-based uniform stream shared with the device codec (csrc/codec.cuh)
# ----------------------------------------------------------------------------------

def sr_key(seed: int, stream: int = 0) -> int:
    """32-bit key of a (seed, stream) pair; ``stream`` separates quantizer stages."""
    z = (int(seed) + 0x9E3779B97F4A7C15 * (int(stream) + 1)) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z ^= z >> 31
    return int((z ^ (z >> 32)) & _U32)


def stage1_stream(rank: int) -> int:
    """Random stream of the FIRST quantizer stage of a collective on ``rank``.  Every rank
    quantizes its own copy of element i, so with one shared stream all ranks would draw the
    same uniform for it and their rounding errors would add up coherently (the error of the
    sum growing with W instead of sqrt(W)); a stream per source rank keeps them independent
    while every engine (fused kernel, host engines, golden model) still derives the same
    bits.  The second stage quantizes each shard on its one owner and keeps stream 1."""
    return 2 * (int(rank) + 1)


def sr_uniform(key: int, index: torch.Tensor) -> torch.Tensor:
    """fp32 uniforms in [0, 1) with 16 random bits, one per element index.

    One 32-bit hash serves two consecutive elements: ``h = (idx >> 1) * 0x9E3779B1 + key``
    followed by two xorshift-multiply rounds; even indices take the low 16 bits, odd
    indices the high 16 bits, scaled by 2^-16.  ``index`` is an int64 tensor and is
    reduced mod 2^32.
    """
    idx = index.to(torch.int64) & _U32
    h = ((idx >> 1) * 0x9E3779B1 + int(key)) & _U32
    h = h ^ (h >> 16)
    h = (h * 0x21F0AAAD) & _U32
    h = h ^ (h >> 15)
    h = (h * 0x735A2D97) & _U32
    h = h ^ (h >> 15)
    bits = torch.where((idx & 1) == 1, h >> 16, h & 0xFFFF)
    return bits.to(torch.float32) * (1.0 / 65536.0)


def _draw_uniform(like: torch.Tensor, sr_seed: Optional[int], sr_offset: int,
                  sr_stream: int) -> torch.Tensor:
    if sr_seed is None:
        return torch.rand_like(like)
    idx = torch.arange(like.numel(), dtype=torch.int64, device=like.device) + int(sr_offset)
    return sr_uniform(sr_key(sr_seed, sr_stream), idx).view_as(like)


def _round(values: torch.Tensor, stochastic: bool, sr_seed: Optional[int],
           sr_offset: int, sr_stream: int) -> torch.Tensor:
    if not stochastic:
        return torch.round(values)  # half to even
    floor = torch.floor(values)
    frac = (values - floor).clamp_(0.0, 1.0)
    bump = _draw_uniform(frac, sr_seed, sr_offset, sr_stream) < frac
    return floor + bump.to(values.dtype)


@dataclass(frozen=True)
class CompressedTensor:
    packed: torch.Tensor
    scale: float
    numel: int
    shape: Tuple[int, ...]
    bitwidth: int
    dtype: torch.dtype

    @property
    def packed_bytes(self) -> int:
        return int(self.packed.numel())


# ----------------------------------------------------------------------------------
# per-tensor quantizer
# ----------------------------------------------------------------------------------

def quantize_tensor(
    tensor: torch.Tensor,
    bitwidth: int,
    *,
    stochastic_rounding: bool = False,
    sr_seed: Optional[int] = None,
    sr_offset: int = 0,
) -> Tuple[torch.Tensor, float]:
    """One scale for the whole tensor; returns (int16 codes shaped like input, scale).

    Rounding acts on the signed ratio ``x / scale`` (reference
    ``quantization.py:65-99``).  The CUDA path finds the absmax on the device
    and reads back only the scalar the API has to return.
    """
    validate_bitwidth(bitwidth)
    if not tensor.is_floating_point():
        raise TypeError("quantize_tensor expects a floating-point tensor")

    if tensor.is_cuda and _CUDA is not None and _CUDA.supports_dtype(tensor.dtype):
        q, scale = _CUDA.quantize_per_tensor(
            tensor, bitwidth, stochastic_rounding, sr_seed, sr_offset)
        return q, float(scale.item())

    qmin, qmax = _quant_bounds(bitwidth)
    x = tensor.detach().to(torch.float32).contiguous()
    peak = float(x.abs().max().item()) if x.numel() else 0.0
    scale = peak / float(qmax) if peak != 0.0 else 1.0
    ratio = x / scale
    q = _round(ratio, stochastic_rounding, sr_seed, sr_offset, 2)
    return q.clamp_(qmin, qmax).to(torch.int16), scale


def dequantize_tensor(
    q_tensor: torch.Tensor,
    scale: float,
    *,
    dtype: torch.dtype = torch.float32,
    device: Optional[torch.device] = None,
    shape: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    if device is None:
        device = q_tensor.device
    if q_tensor.is_cuda and _CUDA is not None and q_tensor.dtype == torch.int16:
        out = _CUDA.dequantize_per_tensor(q_tensor, float(scale))
    else:
        out = q_tensor.to(torch.float32) * float(scale)
    if shape is not None:
        out = out.view(*shape)
    return out.to(device=device, dtype=dtype)


# ----------------------------------------------------------------------------------
# blockwise quantizer
# ----------------------------------------------------------------------------------

def quantize_tensor_blockwise(
    tensor: torch.Tensor,
    bitwidth: int,
    *,
    block_size: int = DEFAULT_BLOCK_SIZE,
    stochastic_rounding: bool = False,
    sr_seed: Optional[int] = None,
    sr_offset: int = 0,
    sr_stream: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (int16 codes [numel], fp16 scales [ceil(numel / block_size)])."""
    validate_bitwidth(bitwidth)
    if not tensor.is_floating_point():
        raise TypeError("quantize_tensor_blockwise expects a floating-point tensor")
    _check_block_size(block_size)

    flat = tensor.detach().to(torch.float32).reshape(-1)
    n = int(flat.numel())
    if n == 0:
        return (flat.to(torch.int16),
                torch.empty(0, dtype=torch.float16, device=flat.device))

    qmin, qmax = _quant_bounds(bitwidth)
    nblocks = -(-n // block_size)
    if nblocks * block_size != n:
        flat = torch.nn.functional.pad(flat, (0, nblocks * block_size - n))
    grid = flat.view(nblocks, block_size)
    mag = grid.abs()
    peak = mag.amax(dim=1)
    scale = peak / float(qmax)
    scale = torch.where(peak > 0, scale, torch.ones_like(scale))
    scale_h = scale.to(torch.float16)

    ratio = mag / scale_h.to(torch.float32).unsqueeze(1)
    level = _round(ratio, stochastic_rounding, sr_seed, sr_offset, sr_stream)
    if bitwidth != 1:
        level = level * grid.sign()
    q = level.clamp_(qmin, qmax).to(torch.int16).view(-1)[:n]
    return q, scale_h


def dequantize_tensor_blockwise(
    q_tensor: torch.Tensor,
    scales: torch.Tensor,
    *,
    block_size: int = DEFAULT_BLOCK_SIZE,
    dtype: torch.dtype = torch.float32,
    device: Optional[torch.device] = None,
    shape: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    if device is None:
        device = q_tensor.device
    _check_block_size(block_size)

    q = q_tensor.to(torch.float32).reshape(-1)
    n = int(q.numel())
    if n:
        nblocks = int(scales.numel())
        want = -(-n // block_size)
        if nblocks != want:
            raise ValueError(
                f"scales length {nblocks} does not match expected blocks {want}"
            )
        per_elem = scales.to(device=q.device, dtype=torch.float32).repeat_interleave(
            block_size)[:n]
        q = q * per_elem
    if shape is not None:
        q = q.view(*shape)
    return q.to(device=device, dtype=dtype)


def _cuda_blockwise_ok(t: torch.Tensor, bitwidth: int, block_size: int,
                       dtype: torch.dtype) -> bool:
    return (
        t.is_cuda
        and _CUDA is not None
        and _CUDA.supports_dtype(dtype)
        and _CUDA.supports_blockwise(bitwidth, block_size)
    )


def quantize_pack_tensor_blockwise(
    tensor: torch.Tensor,
    bitwidth: int,
    *,
    block_size: int = DEFAULT_BLOCK_SIZE,
    stochastic_rounding: bool = False,
    sr_seed: Optional[int] = None,
    sr_offset: int = 0,
    sr_stream: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Blockwise quantize + pack; one fused kernel on CUDA. Returns (packed, scales, numel)."""
    validate_bitwidth(bitwidth)
    if not tensor.is_floating_point():
        raise TypeError("quantize_pack_tensor_blockwise expects a floating-point tensor")
    _check_block_size(block_size)

    if _cuda_blockwise_ok(tensor, bitwidth, block_size, tensor.dtype):
        packed, scales = _CUDA.blockwise_quantize_pack(
            tensor, bitwidth, block_size, stochastic_rounding, sr_seed, sr_offset,
            sr_stream)
        return packed, scales, int(tensor.numel())

    native = _cpu_codec() if tensor.device.type == "cpu" else None
    if native is not None:
        seed = sr_seed
        if stochastic_rounding and seed is None:
            # unseeded: a fresh stream per call, drawn from torch's generator so that
            # torch.manual_seed still makes a run repeatable
            seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item())
        packed, scales = native.blockwise_quantize_pack(
            tensor, bitwidth, block_size, stochastic_rounding, seed, sr_offset, sr_stream)
        return packed, scales, int(tensor.numel())

    q, scales = quantize_tensor_blockwise(
        tensor, bitwidth, block_size=block_size,
        stochastic_rounding=stochastic_rounding,
        sr_seed=sr_seed, sr_offset=sr_offset, sr_stream=sr_stream)
    packed, n = pack_lowbit(q, bitwidth)
    return packed, scales, n


def unpack_dequantize_tensor_blockwise(
    packed: torch.Tensor,
    scales: torch.Tensor,
    bitwidth: int,
    numel: int,
    *,
    block_size: int = DEFAULT_BLOCK_SIZE,
    dtype: torch.dtype = torch.float32,
    device: Optional[torch.device] = None,
    shape: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Unpack + blockwise dequantize; one fused kernel on CUDA."""
    validate_bitwidth(bitwidth)
    if device is None:
        device = packed.device
    _check_block_size(block_size)

    if scales.is_cuda and _cuda_blockwise_ok(packed, bitwidth, block_size, dtype):
        out = _CUDA.blockwise_unpack_dequantize(
            packed, scales, bitwidth, int(numel), block_size, dtype)
        if shape is not None:
            out = out.view(*shape)
        return out.to(device=device, dtype=dtype)

    native = _cpu_codec() if (packed.device.type == "cpu" and scales.device.type == "cpu"
                              and packed.dtype == torch.uint8
                              and scales.dtype == torch.float16) else None
    if native is not None:
        if scales.numel() != -(-int(numel) // block_size):
            raise ValueError("scales length does not match numel and block_size")
        out = native.blockwise_unpack_dequantize(packed, scales, bitwidth, int(numel), block_size)
        if shape is not None:
            out = out.view(*shape)
        return out.to(device=device, dtype=dtype)

    q = unpack_lowbit(packed, bitwidth, numel)
    return dequantize_tensor_blockwise(
        q, scales, block_size=block_size, dtype=dtype, device=device, shape=shape)


# ----------------------------------------------------------------------------------
# bit packing
# ----------------------------------------------------------------------------------

def packed_nbytes(numel: int, bitwidth: int) -> int:
    """Wire bytes for ``numel`` codes (12-bit pairs occupy 3 bytes)."""
    if bitwidth == 12:
        return 3 * ((numel + 1) // 2)
    if bitwidth == 16:
        return 2 * numel
    return -(-numel * bitwidth // 8)


def pack_lowbit(q_tensor: torch.Tensor, bitwidth: int) -> Tuple[torch.Tensor, int]:
    """Pack int codes into contiguous uint8. Returns (packed, numel)."""
    validate_bitwidth(bitwidth)
    n = int(q_tensor.numel())
    if q_tensor.is_cuda and _CUDA is not None and q_tensor.dtype == torch.int16:
        return _CUDA.pack(q_tensor, bitwidth), n

    qmin, _ = _quant_bounds(bitwidth)
    code = q_tensor.reshape(-1).to(torch.int32) - qmin
    dev = code.device

    if bitwidth == 16:
        return code.to(torch.int16).view(torch.uint8).contiguous(), n

    if bitwidth == 12:
        if n & 1:
            code = torch.nn.functional.pad(code, (0, 1))
        lo, hi = code.view(-1, 2).unbind(dim=1)
        out = torch.empty(lo.numel(), 3, dtype=torch.uint8, device=dev)
        out[:, 0] = (lo & 0xFF).to(torch.uint8)
        out[:, 1] = (((lo >> 8) & 0xF) | ((hi & 0xF) << 4)).to(torch.uint8)
        out[:, 2] = ((hi >> 4) & 0xFF).to(torch.uint8)
        return out.view(-1), n

    lanes = 8 // bitwidth
    short = (-n) % lanes
    if short:
        code = torch.nn.functional.pad(code, (0, short))
    code = code.view(-1, lanes)
    byte = torch.zeros(code.shape[0], dtype=torch.int32, device=dev)
    for lane in range(lanes):
        byte |= code[:, lane] << (lane * bitwidth)
    return byte.to(torch.uint8), n


def unpack_lowbit(packed: torch.Tensor, bitwidth: int, numel: int) -> torch.Tensor:
    """Inverse of :func:`pack_lowbit`; returns int16 codes [numel]."""
    validate_bitwidth(bitwidth)
    packed = packed.contiguous().view(-1)
    if packed.is_cuda and _CUDA is not None:
        return _CUDA.unpack(packed, bitwidth, int(numel))

    qmin, _ = _quant_bounds(bitwidth)
    if bitwidth == 16:
        code = packed.view(torch.int16).to(torch.int32)[:numel]
    elif bitwidth == 12:
        b = packed.view(-1, 3).to(torch.int32)
        lo = b[:, 0] | ((b[:, 1] & 0xF) << 8)
        hi = ((b[:, 1] >> 4) & 0xF) | (b[:, 2] << 4)
        code = torch.stack((lo, hi), dim=1).view(-1)[:numel]
    else:
        lanes = 8 // bitwidth
        mask = (1 << bitwidth) - 1
        wide = packed.to(torch.int32)
        code = torch.stack(
            [(wide >> (lane * bitwidth)) & mask for lane in range(lanes)], dim=1
        ).view(-1)[:numel]
    return (code + qmin).to(torch.int16)


# ----------------------------------------------------------------------------------
# per-tensor compress / decompress
# ----------------------------------------------------------------------------------

def compress_tensor(tensor: torch.Tensor, bitwidth: int) -> CompressedTensor:
    q, scale = quantize_tensor(tensor, bitwidth)
    packed, n = pack_lowbit(q, bitwidth)
    return CompressedTensor(
        packed=packed, scale=scale, numel=n, shape=tuple(tensor.shape),
        bitwidth=bitwidth, dtype=tensor.dtype)


def decompress_tensor(
    compressed: CompressedTensor,
    *,
    dtype: Optional[torch.dtype] = None,
    device: Optional[torch.device] = None,
) -> torch.Tensor:
    q = unpack_lowbit(compressed.packed, compressed.bitwidth, compressed.numel)
    return dequantize_tensor(
        q, compressed.scale, dtype=dtype or compressed.dtype, device=device,
        shape=compressed.shape)


def roundtrip_tensor(tensor: torch.Tensor, bitwidth: int) -> torch.Tensor:
    return decompress_tensor(
        compress_tensor(tensor, bitwidth), dtype=tensor.dtype, device=tensor.device)
