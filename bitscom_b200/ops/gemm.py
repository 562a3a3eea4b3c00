"""bf16 GEMM on tcgen05 tensor cores (``csrc/gemm_tcgen05.cu``) and the linear layer
built from it.  ``torch.matmul`` (cuBLAS) is the library call this replaces; the
reference trainer's model is plain ``nn.Linear``
(``benchmarks/train_llama7b_dp_pp_lowbit.py:222-238``)."""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..parallel.deferred import DeferredWork
from . import _native
from ._native import NativeError, check, ptr, stream_ptr

_lib = None
_lib2 = None      # the CTA-pair kernel's library, loaded when that variant is first selected
_variant = None   # "1cta" | "2cta"; None until the first call reads BITSCOM_GEMM
_VARIANTS = ("1cta", "2cta")


def _get():
    global _lib
    if _lib is None:
        lib = _native.load("bcom_llama")
        if lib is not None:
            vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
            lib.bcom_gemm_bf16.argtypes = [vp, vp, vp, ci, ci, ci, ll, ll, ll, ci, ci, ci, ci,
                                           ci, vp]
            lib.bcom_gemm_bf16_ex.argtypes = [vp, vp, vp, vp, ci, ci, ci, ll, ll, ll, ll, ci, ci,
                                              ci, ci, ci, vp]
            lib.bcom_gemm_status.argtypes = [ctypes.POINTER(ctypes.c_uint * 4), ci]
        _lib = lib if lib is not None else False
    return _lib or None


def _get2():
    """The CTA-pair kernel (``csrc/gemm_tcgen05_2cta.cu``), or ``None`` when its library is
    not part of this installation."""
    global _lib2
    if _lib2 is None:
        try:
            lib = _native.load("bcom_gemm2")
        except Exception:  # sources and binary both absent
            lib = None
        if lib is not None:
            vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
            lib.bcom_gemm2_bf16.argtypes = [vp, vp, vp, ci, ci, ci, ll, ll, ll, ci, ci, ci, ci,
                                            ci, vp]
            lib.bcom_gemm2_bf16_ex.argtypes = [vp, vp, vp, vp, ci, ci, ci, ll, ll, ll, ll, ci,
                                               ci, ci, ci, ci, vp]
            lib.bcom_gemm2_status.argtypes = [ctypes.POINTER(ctypes.c_uint * 4), ci]
            lib.bcom_gemm2_set_profile.argtypes = [vp]
        _lib2 = lib if lib is not None else False
    return _lib2 or None


def pair_available() -> bool:
    """True when the CTA-pair kernel's library is part of this installation (it is a library of
    its own, left out of some deployments) and a GPU is present."""
    return _native.cuda_present() and _get2() is not None


def available() -> bool:
    return _native.cuda_present() and _get() is not None


def variant() -> str:
    """The kernel that ``gemm`` launches: "1cta" (default) or "2cta" (CTA pairs, 256x256 tiles,
    ``tcgen05.mma.cta_group::2``).  Initialised from ``BITSCOM_GEMM``."""
    global _variant
    if _variant is None:
        want = os.environ.get("BITSCOM_GEMM", "1cta").strip().lower()
        _variant = "1cta"
        if want == "2cta":
            set_variant("2cta")
        elif want != "1cta":
            raise ValueError(f"BITSCOM_GEMM={want!r}: expected one of {_VARIANTS}")
    return _variant


def set_variant(name: str) -> str:
    """Select the GEMM kernel; returns the name that was active before.  Raises
    ``NativeError`` if the CTA-pair library is not available."""
    global _variant
    if name not in _VARIANTS:
        raise ValueError(f"unknown GEMM variant {name!r}")
    old = _variant or "1cta"
    if name == "2cta" and _get2() is None:
        raise NativeError("the CTA-pair GEMM needs the bcom_gemm2 library and a GPU")
    _variant = name
    return old


_STATUS = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue", 4: "accumulator hand-off"}


def check_status(clear: bool = True) -> None:
    """Raise if a GEMM kernel gave up on one of its bounded waits (synchronises)."""
    out = (ctypes.c_uint * 4)()
    check(_get().bcom_gemm_status(ctypes.byref(out), int(clear)), "bcom_gemm_status", launches=0)
    which = "tcgen05 GEMM"
    if not out[0] and _lib2:
        check(_lib2.bcom_gemm2_status(ctypes.byref(out), int(clear)), "bcom_gemm2_status", launches=0)
        which = "tcgen05 CTA-pair GEMM"
    if out[0]:
        raise NativeError(f"{which} timed out in the {_STATUS.get(out[0], out[0])} "
                          f"(cta {out[1]}, thread {out[2]})")


_library = False  # True: torch.matmul (cuBLAS) instead of the tcgen05 kernels (comparator only)


def use_library_gemm(on: bool) -> bool:
    """Comparator switch for benchmarks: route ``gemm`` through ``torch.matmul`` (cuBLAS, bf16
    output, accumulation into an existing tensor by a separate add), the way a plain
    ``nn.Linear`` model computes.  Never the default; returns the previous setting."""
    global _library
    old, _library = _library, bool(on)
    return old


def _gemm_library(a, b, a_mn_major, b_mn_major, out, out_dtype, accumulate, residual=None):
    A = a.t() if a_mn_major else a
    B = b if b_mn_major else b.t()
    c = torch.matmul(A, B)
    if residual is not None:
        c = c + residual
    if out is None:
        return c if out_dtype == c.dtype else c.to(out_dtype)
    if accumulate:
        out.add_(c)
    else:
        out.copy_(c)
    return out


def _gemm_host(a, b, a_mn_major, b_mn_major, out, out_dtype, accumulate, residual=None):
    """The kernel's contract for tensors that live on the CPU (fp32 accumulation, result
    rounded once): CPU ranks run the trainers' plumbing with it."""
    A = a.float().t() if a_mn_major else a.float()
    B = b.float() if b_mn_major else b.float().t()
    if A.shape[1] != B.shape[0]:
        raise ValueError(f"reduction dimensions differ: {A.shape[1]} vs {B.shape[0]}")
    c = A @ B
    if residual is not None:
        c = c + residual.float()
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        return c.to(out_dtype)
    if out.shape != c.shape:
        raise ValueError("bad output tensor")
    out.copy_(out.float() + c if accumulate else c)
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False,
         b_mn_major: bool = False, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         max_ctas: int = 0, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C[M, N] (+)= A x B`` with bf16 operands and fp32 accumulation.

    ``a``: ``[M, K]`` (K-major) or, with ``a_mn_major``, stored ``[K, M]``.
    ``b``: ``[N, K]`` (K-major) or, with ``b_mn_major``, stored ``[K, N]``.
    Operands are 2-D with unit stride in the last dimension; row strides are free.
    ``residual`` (bf16 ``[M, N]``, bf16 non-accumulating output only): ``C = residual + A x B``,
    added in the epilogue before the result is rounded.
    """
    if residual is not None and (accumulate or (out is not None and out.dtype != torch.bfloat16)
                                 or (out is None and out_dtype != torch.bfloat16)):
        raise ValueError("residual needs a bf16, non-accumulating output")
    if not a.is_cuda:
        return _gemm_host(a, b, a_mn_major, b_mn_major, out, out_dtype, accumulate, residual)
    if _library:
        return _gemm_library(a, b, a_mn_major, b_mn_major, out, out_dtype, accumulate, residual)
    lib = _get()
    if lib is None:
        raise NativeError("tcgen05 GEMM needs the bcom_llama library and a GPU")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm expects bf16 operands")
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm expects 2-D operands with a contiguous last dimension")
    K, M = (a.shape[0], a.shape[1]) if a_mn_major else (a.shape[1], a.shape[0])
    Kb, N = (b.shape[0], b.shape[1]) if b_mn_major else (b.shape[1], b.shape[0])
    if K != Kb:
        raise ValueError(f"reduction dimensions differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16,
                                                                      torch.float32):
        raise ValueError("bad output tensor")
    if residual is not None and (residual.shape != (M, N) or residual.stride(1) != 1
                                 or residual.dtype != torch.bfloat16):
        raise ValueError("bad residual tensor")
    launch = lib.bcom_gemm_bf16_ex if variant() == "1cta" else _get2().bcom_gemm2_bf16_ex
    with _native.on_device(a.device):
        check(launch(
            ptr(a), ptr(b), ptr(out), ptr(residual), M, N, K, a.stride(0), b.stride(0),
            out.stride(0), 0 if residual is None else residual.stride(0),
            int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32),
            int(accumulate), int(max_ctas), stream_ptr(a.device)), "bcom_gemm_bf16")
    return out


class LinearFunction(torch.autograd.Function):
    """``y = x W^T`` for ``x [tokens, in]`` and ``W [out, in]``, all three GEMMs on tcgen05.

    The weight gradient is accumulated in fp32 into ``weight.main_grad`` when the
    parameter has that attribute (gradient accumulation over micro-batches and the flat
    fp32 bucket the low-bit all-reduce works on); otherwise it is returned in bf16.
    """

    @staticmethod
    def forward(ctx, x, weight, residual=None):
        """``residual`` (same shape as the output): ``y = residual + x W^T`` in the GEMM's
        epilogue; its gradient is the output gradient itself."""
        ctx.save_for_backward(x, weight)
        ctx.has_residual = residual is not None
        x2 = x.reshape(-1, x.shape[-1])
        # allocate with the final shape: the result must not be a view, later kernels
        # (RoPE, cross-entropy) update it in place
        y = torch.empty(*x.shape[:-1], weight.shape[0], dtype=x.dtype, device=x.device)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, weight.shape[0])
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        gemm(x2, weight, out=y.view(-1, weight.shape[0]), residual=res2)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx[T, in] = dy[T, out] x W[out, in]: B is stored [K=out, N=in]
            dx = gemm(dy2, weight, b_mn_major=True).view_as(x)
        if ctx.needs_input_grad[1]:
            # dW[out, in] = dy^T x: both operands stored [K=T, *]
            main = getattr(weight, "main_grad", None)
            if main is not None:
                queue = DeferredWork.active()
                if queue is not None:
                    # pipeline parallelism: the input gradient goes out first, this GEMM runs
                    # while it is on the wire
                    queue.add(lambda: gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=main,
                                           accumulate=True))
                else:
                    gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=main, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn_major=True, b_mn_major=True)
        return dx, dw, (dy if ctx.has_residual and ctx.needs_input_grad[2] else None)


def linear(x: torch.Tensor, weight: torch.Tensor,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x W^T`` (``+ residual``, added inside the GEMM) on the tcgen05 kernels."""
    return LinearFunction.apply(x, weight, residual)
