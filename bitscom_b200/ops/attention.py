"""Causal flash attention on tcgen05 (``csrc/attention_tcgen05.cu``), head_dim 128 (Llama)
or 64 (GPT-2), consuming the fused ``qkv`` projection in place.  Library baseline: torch
SDPA."""

from __future__ import annotations

import ctypes
import math
import os
from typing import Dict, Tuple

import torch

from . import _native
from ._native import NativeError, check, ptr, stream_ptr

_lib = None
_scratch: Dict[Tuple, torch.Tensor] = {}
# forward kernels: "simple" alternates MMA and softmax inside a CTA; "pipelined" has an issuer
# warp, double-buffered scores in TMEM and the output accumulated in TMEM
_FWD_VARIANTS = {"simple": 0, "pipelined": 1}
# how the backward kernel adds a dQ tile to the fp32 accumulator: float4 atomics from
# registers, or TMA reductions from a shared-memory staging tile
_BWD_DQ_VARIANTS = {"atomic": 0, "tma": 1}


def _get():
    global _lib
    if _lib is None:
        lib = _native.load("bcom_llama")
        if lib is not None and hasattr(lib, "bcom_attention_fwd"):
            vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
            lib.bcom_attention_fwd.argtypes = [vp, vp, vp, ci, ci, ci, ci, cf, vp]
            lib.bcom_attention_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, cf, vp]
            lib.bcom_attention_status.argtypes = [ctypes.POINTER(ctypes.c_uint * 4), ci]
            lib.bcom_attention_set_fwd_variant.argtypes = [ci]
            lib.bcom_attention_set_bwd_dq_variant.argtypes = [ci]
            dq = os.environ.get("BITSCOM_ATTN_BWD_DQ", "").strip().lower()
            if dq in _BWD_DQ_VARIANTS:
                lib.bcom_attention_set_bwd_dq_variant(_BWD_DQ_VARIANTS[dq])
            variant = os.environ.get("BITSCOM_ATTN_FWD", "").strip().lower()
            if variant in _FWD_VARIANTS:
                lib.bcom_attention_set_fwd_variant(_FWD_VARIANTS[variant])
        else:
            lib = None
        _lib = lib if lib is not None else False
    return _lib or None


def available() -> bool:
    return _native.cuda_present() and _get() is not None


def set_forward_variant(name: str) -> str:
    """Select the forward kernel ("simple" or "pipelined", also ``BITSCOM_ATTN_FWD``); returns
    the name that was active before."""
    if name not in _FWD_VARIANTS:
        raise ValueError(f"unknown attention forward variant {name!r}")
    lib = _get()
    if lib is None:
        raise NativeError("attention kernel needs the bcom_llama library and a GPU")
    old = lib.bcom_attention_set_fwd_variant(_FWD_VARIANTS[name])
    return {0: "simple", 1: "pipelined"}[old]


def set_backward_dq_variant(name: str) -> str:
    """Select how dQ tiles are accumulated ("atomic" or "tma", also ``BITSCOM_ATTN_BWD_DQ``);
    returns the name that was active before."""
    if name not in _BWD_DQ_VARIANTS:
        raise ValueError(f"unknown attention backward dQ variant {name!r}")
    lib = _get()
    if lib is None:
        raise NativeError("attention kernel needs the bcom_llama library and a GPU")
    old = lib.bcom_attention_set_bwd_dq_variant(_BWD_DQ_VARIANTS[name])
    return {0: "atomic", 1: "tma"}[old]


def supported(seq: int, head_dim: int) -> bool:
    return head_dim in (64, 128) and seq % 128 == 0


def check_status(clear: bool = True) -> None:
    out = (ctypes.c_uint * 4)()
    check(_get().bcom_attention_status(ctypes.byref(out), int(clear)), "attention_status", launches=0)
    if out[0]:
        raise NativeError(f"attention kernel timed out at wait {out[0]} (cta {out[1]})")


def _zero_scratch(key, shape, device) -> torch.Tensor:
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = torch.zeros(shape, dtype=torch.float32, device=device)
    return buf


class AttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, batch, seq, heads, head_dim):
        lib = _get()
        if lib is None:
            raise NativeError("attention kernel needs the bcom_llama library and a GPU")
        if not supported(seq, head_dim):
            raise ValueError("tcgen05 attention needs head_dim 64 or 128 and seq % 128 == 0")
        H = heads * head_dim
        q2 = qkv.view(batch * seq, 3 * H)
        out = torch.empty(batch * seq, H, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(batch, heads, seq, dtype=torch.float32, device=qkv.device)
        scale = 1.0 / math.sqrt(head_dim)
        check(lib.bcom_attention_fwd(ptr(q2), ptr(out), ptr(lse), batch, seq, heads, head_dim,
                                     scale, stream_ptr(qkv.device)), "attention_fwd")
        ctx.save_for_backward(q2, out, lse)
        ctx.meta = (batch, seq, heads, head_dim, scale)
        return out

    @staticmethod
    def backward(ctx, d_out):
        lib = _get()
        q2, out, lse = ctx.saved_tensors
        batch, seq, heads, head_dim, scale = ctx.meta
        H = heads * head_dim
        d_out = d_out.contiguous()
        dqkv = torch.empty_like(q2)
        dev = q2.device
        dq_acc = _zero_scratch(("dq", batch * seq, H, dev.index), (batch * seq, H), dev)
        delta = torch.empty(batch, heads, seq, dtype=torch.float32, device=dev)
        check(lib.bcom_attention_bwd(ptr(q2), ptr(out), ptr(d_out), ptr(lse), ptr(dqkv),
                                     ptr(dq_acc), ptr(delta), batch, seq, heads, head_dim,
                                     scale, stream_ptr(dev)), "attention_bwd", launches=3)
        return dqkv.view_as(q2), None, None, None, None


def attention(qkv: torch.Tensor, batch: int, seq: int, heads: int, head_dim: int
              ) -> torch.Tensor:
    """``qkv``: ``[batch * seq, 3 * heads * head_dim]`` bf16; returns ``[batch * seq,
    heads * head_dim]``."""
    return AttentionFunction.apply(qkv, batch, seq, heads, head_dim)
