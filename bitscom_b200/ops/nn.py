"""Autograd wrappers over the bandwidth-bound trainer kernels (``csrc/elementwise.cu``):
RMSNorm, LayerNorm, RoPE, SwiGLU, bias + GELU, fused softmax cross-entropy, embedding, flat
AdamW / SGD."""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _native
from ._native import NativeError, check, ptr, stream_ptr

_lib = None


def _get():
    global _lib
    if _lib is None:
        lib = _native.load("bcom_llama")
        if lib is not None:
            vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
            lib.bcom_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, ci, ci, cf, vp]
            lib.bcom_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, vp]
            lib.bcom_norm_bwd_scratch_elems.argtypes = [ci, ci]
            lib.bcom_norm_bwd_scratch_elems.restype = ll
            lib.bcom_rope.argtypes = [vp, vp, vp, ll, ci, ci, ll, ci, ci, vp]
            lib.bcom_layernorm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, cf, vp]
            lib.bcom_layernorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, vp]
            lib.bcom_bias_gelu_fwd.argtypes = [vp, vp, vp, ll, ci, vp]
            lib.bcom_bias_gelu_bwd.argtypes = [vp, vp, vp, vp, vp, ll, ci, vp]
            lib.bcom_swiglu_fwd.argtypes = [vp, vp, ll, ci, vp]
            lib.bcom_swiglu_bwd.argtypes = [vp, vp, vp, ll, ci, vp]
            lib.bcom_cross_entropy.argtypes = [vp, vp, vp, vp, ci, ci, ll, vp]
            lib.bcom_embedding_fwd.argtypes = [vp, vp, vp, ll, ci, ci, vp]
            lib.bcom_embedding_bwd.argtypes = [vp, vp, vp, ll, ci, ci, vp]
            lib.bcom_adamw.argtypes = [vp, vp, vp, vp, vp, ll, cf, cf, cf, cf, cf, ci, cf, ci, vp]
            lib.bcom_sgd_momentum.argtypes = [vp, vp, vp, ll, cf, cf, cf, cf, ci, vp]
        _lib = lib if lib is not None else False
    return _lib or None


def available() -> bool:
    return _native.cuda_present() and _get() is not None


def _need():
    lib = _get()
    if lib is None:
        raise NativeError("trainer kernels need the bcom_llama library and a GPU")
    return lib


# ----------------------------------------------------------------------------------
class RMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if not x.is_cuda:  # the kernel's arithmetic in torch ops, for CPU ranks
            xf = x2.float()
            rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
            y = (xf * rstd[:, None] * weight.float()).to(x.dtype)
            ctx.save_for_backward(x2, weight, rstd)
            ctx.shape = x.shape
            return y.view(x.shape)
        lib = _need()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        check(lib.bcom_rmsnorm_fwd(ptr(x2), ptr(weight), ptr(y), ptr(rstd), x2.shape[0], H,
                                   float(eps), stream_ptr(x.device)), "rmsnorm_fwd")
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        dx, dw = _rmsnorm_backward(ctx, dy, None)
        return dx, dw, None


def _rmsnorm_backward(ctx, dy, dres):
    """Shared by ``RMSNormFunction`` and ``RMSNormForkFunction``: ``dres`` (or None) is the
    gradient that reaches the same input through the residual connection; it is added to dx
    inside the kernel."""
    x2, weight, rstd = ctx.saved_tensors
    H = x2.shape[1]
    dy2 = dy.reshape(-1, H)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    if dres is not None:
        dres = dres.reshape(-1, H)
        if not dres.is_contiguous():
            dres = dres.contiguous()
    main = getattr(weight, "main_grad", None)
    dw = main if main is not None else torch.zeros(H, dtype=torch.float32, device=dy.device)
    if not dy.is_cuda:  # CPU ranks
        xf, gf, rs = x2.float(), dy2.float(), rstd[:, None]
        gw = gf * weight.float()
        coef = (gw * xf).sum(-1, keepdim=True) * rs.pow(3) / H
        dxf = gw * rs - xf * coef
        if dres is not None:
            dxf = dxf + dres.float()
        dw.add_((gf * xf * rs).sum(0))
        return dxf.to(x2.dtype).view(ctx.shape), (None if main is not None
                                                  else dw.to(weight.dtype))
    lib = _need()
    dx = torch.empty_like(x2)
    # per-CTA weight-gradient partials, folded into dw by a second small kernel
    scratch = torch.empty(int(lib.bcom_norm_bwd_scratch_elems(H, 0)), dtype=torch.float32,
                          device=dy.device)
    check(lib.bcom_rmsnorm_bwd(
        ptr(dy2), ptr(x2), ptr(weight), ptr(rstd), ptr(dres), ptr(dx), ptr(dw), ptr(scratch),
        x2.shape[0], H, stream_ptr(dy.device)), "rmsnorm_bwd", launches=2)
    return dx.view(ctx.shape), (None if main is not None else dw.to(weight.dtype))


class RMSNormForkFunction(torch.autograd.Function):
    """``(rmsnorm(x), x)``: the normalised branch and the residual branch of a pre-norm block
    as ONE node.  Forward is ``RMSNormFunction``'s; the point is backward, where the gradients
    of both branches meet: ``dx = rmsnorm_backward(dh) + dx_residual`` is produced by one kernel
    instead of the norm's backward followed by autograd's own add kernel."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        h = RMSNormFunction.forward(ctx, x, weight, eps)
        return h, x.view_as(x)

    @staticmethod
    def backward(ctx, dh, dres):
        if dh is None:  # only the residual branch was used
            return dres, None, None
        dx, dw = _rmsnorm_backward(ctx, dh, dres)
        return dx, dw, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return RMSNormFunction.apply(x, weight, eps)


def rmsnorm_fork(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(rmsnorm(x), x)`` for a pre-norm residual block: feed the first into the block and
    carry the second as the residual; see ``RMSNormForkFunction``."""
    return RMSNormForkFunction.apply(x, weight, eps)


# ----------------------------------------------------------------------------------
def rope_tables(seq: int, head_dim: int, theta: float = 10000.0, device="cuda"
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of shape [seq, head_dim / 2], fp32 (rotate-half convention)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def _rope_inplace(x2: torch.Tensor, col0: int, heads: int, head_dim: int, cos, sin, seq: int,
                  backward: bool):
    if not x2.is_cuda:  # CPU ranks: rotate-half on every head of this third, in place
        half = head_dim // 2
        t = x2[:, col0:col0 + heads * head_dim].reshape(-1, seq, heads, head_dim).float()
        c = cos[:seq, None, :].float()
        s = sin[:seq, None, :].float() * (-1.0 if backward else 1.0)
        a, b = t[..., :half], t[..., half:]
        rot = torch.cat([a * c - b * s, b * c + a * s], -1)
        x2[:, col0:col0 + heads * head_dim] = rot.reshape(x2.shape[0], -1).to(x2.dtype)
        return
    lib = _need()
    view = x2[:, col0:]
    check(lib.bcom_rope(ptr(view), ptr(cos), ptr(sin), x2.shape[0], heads, head_dim,
                        x2.stride(0), seq, int(backward), stream_ptr(x2.device)), "rope")


class RopeQKFunction(torch.autograd.Function):
    """Rotates the q and k thirds of a fused ``[tokens, 3 * heads * head_dim]`` projection in
    place (the input is consumed: its storage becomes the output)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, heads, head_dim, seq):
        ctx.mark_dirty(qkv)
        q2 = qkv.view(-1, qkv.shape[-1])
        width = heads * head_dim
        _rope_inplace(q2, 0, heads, head_dim, cos, sin, seq, False)
        _rope_inplace(q2, width, heads, head_dim, cos, sin, seq, False)
        ctx.save_for_backward(cos, sin)
        ctx.meta = (heads, head_dim, seq)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        cos, sin = ctx.saved_tensors
        heads, head_dim, seq = ctx.meta
        d = dqkv.contiguous()
        if d.data_ptr() == dqkv.data_ptr():
            d = d.clone()
        d2 = d.view(-1, d.shape[-1])
        width = heads * head_dim
        _rope_inplace(d2, 0, heads, head_dim, cos, sin, seq, True)
        _rope_inplace(d2, width, heads, head_dim, cos, sin, seq, True)
        return d, None, None, None, None, None


def rope_qk_(qkv, cos, sin, heads: int, head_dim: int, seq: int):
    return RopeQKFunction.apply(qkv, cos, sin, heads, head_dim, seq)


# ----------------------------------------------------------------------------------
def _grad_target(param: torch.Tensor, n: int, device):
    """fp32 buffer a parameter gradient is accumulated into: the flat ``main_grad`` view when
    the parameter has one (then autograd gets ``None``), else a fresh zero vector."""
    main = getattr(param, "main_grad", None)
    if main is not None:
        return main, True
    return torch.zeros(n, dtype=torch.float32, device=device), False


class LayerNormFunction(torch.autograd.Function):
    """LayerNorm over the last dimension (bf16, H <= 1024, H % 8 == 0)."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        lib = _need()
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        check(lib.bcom_layernorm_fwd(ptr(x2), ptr(weight), ptr(bias), ptr(y), ptr(mean),
                                     ptr(rstd), rows, H, float(eps), stream_ptr(x.device)),
              "layernorm_fwd")
        ctx.save_for_backward(x2, weight, bias, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _need()
        x2, weight, bias, mean, rstd = ctx.saved_tensors
        H = x2.shape[1]
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        dw, w_main = _grad_target(weight, H, dy.device)
        db, b_main = _grad_target(bias, H, dy.device)
        scratch = torch.empty(int(lib.bcom_norm_bwd_scratch_elems(H, 1)), dtype=torch.float32,
                              device=dy.device)
        check(lib.bcom_layernorm_bwd(
            ptr(dy2), ptr(x2), ptr(weight), ptr(mean), ptr(rstd), ptr(dx), ptr(dw), ptr(db),
            ptr(scratch), x2.shape[0], H, stream_ptr(dy.device)), "layernorm_bwd", launches=2)
        return (dx.view(ctx.shape), None if w_main else dw.to(weight.dtype),
                None if b_main else db.to(bias.dtype), None)


def layernorm_supported(x: torch.Tensor) -> bool:
    H = x.shape[-1]
    return x.is_cuda and x.dtype == torch.bfloat16 and H % 8 == 0 and H <= 1024


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5
              ) -> torch.Tensor:
    return LayerNormFunction.apply(x, weight, bias, eps)


class BiasGeluFunction(torch.autograd.Function):
    """``gelu(x + bias)`` with the tanh approximation; the backward pass recomputes the
    activation from ``x`` and ``bias`` and accumulates the bias gradient in fp32."""

    @staticmethod
    def forward(ctx, x, bias):
        lib = _need()
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = torch.empty_like(x2)
        check(lib.bcom_bias_gelu_fwd(ptr(x2), ptr(bias), ptr(y), x2.shape[0], C,
                                     stream_ptr(x.device)), "bias_gelu_fwd")
        ctx.save_for_backward(x2, bias)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _need()
        x2, bias = ctx.saved_tensors
        C = x2.shape[1]
        dy2 = dy.reshape(-1, C)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        db, b_main = _grad_target(bias, C, dy.device)
        check(lib.bcom_bias_gelu_bwd(ptr(dy2), ptr(x2), ptr(bias), ptr(dx), ptr(db),
                                     x2.shape[0], C, stream_ptr(dy.device)), "bias_gelu_bwd")
        return dx.view(ctx.shape), None if b_main else db.to(bias.dtype)


def bias_gelu(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    return BiasGeluFunction.apply(x, bias)


# ----------------------------------------------------------------------------------
class SwiGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        F = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * F)
        if not gu.is_contiguous():
            gu = gu.contiguous()
        if not gate_up.is_cuda:  # CPU ranks
            g, u = gu[:, :F].float(), gu[:, F:].float()
            ctx.save_for_backward(gu)
            ctx.shape = gate_up.shape
            return (g * torch.sigmoid(g) * u).to(gu.dtype).view(*gate_up.shape[:-1], F)
        lib = _need()
        h = torch.empty(gu.shape[0], F, dtype=gu.dtype, device=gu.device)
        check(lib.bcom_swiglu_fwd(ptr(gu), ptr(h), gu.shape[0], F, stream_ptr(gu.device)),
              "swiglu_fwd")
        ctx.save_for_backward(gu)
        ctx.shape = gate_up.shape
        return h.view(*gate_up.shape[:-1], F)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        F = gu.shape[1] // 2
        d = dh.reshape(-1, F)
        if not d.is_contiguous():
            d = d.contiguous()
        if not dh.is_cuda:  # CPU ranks
            g, u, df = gu[:, :F].float(), gu[:, F:].float(), d.float()
            sg = torch.sigmoid(g)
            silu = g * sg
            dgu = torch.cat([df * u * (sg + silu * (1.0 - sg)), df * silu], 1).to(gu.dtype)
            return dgu.view(ctx.shape)
        lib = _need()
        dgu = torch.empty_like(gu)
        check(lib.bcom_swiglu_bwd(ptr(gu), ptr(d), ptr(dgu), gu.shape[0], F,
                                  stream_ptr(gu.device)), "swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    return SwiGLUFunction.apply(gate_up)


# ----------------------------------------------------------------------------------
class CrossEntropyFunction(torch.autograd.Function):
    """Mean token cross-entropy over non-ignored targets.  The logits buffer is consumed:
    the kernel writes d(loss)/d(logits) into it during the forward pass, so the backward
    pass is a multiply by the incoming scalar."""

    @staticmethod
    def forward(ctx, logits, targets, ignore_index, loss_scale):
        V = logits.shape[-1]
        l2 = logits.view(-1, V)
        t = targets.reshape(-1).to(torch.int64).contiguous()
        valid = (t != ignore_index).sum().clamp_(min=1).to(torch.float32)
        scale = (loss_scale / valid).reshape(1).contiguous()
        if not logits.is_cuda:  # the kernel's arithmetic in torch ops, for CPU ranks
            keep = t != ignore_index
            z = l2.float()
            lse = torch.logsumexp(z, dim=-1)
            safe = t.clamp(min=0, max=V - 1)
            per_row = torch.where(keep, lse - z.gather(1, safe[:, None])[:, 0],
                                  torch.zeros_like(lse))
            d = torch.softmax(z, dim=-1)
            d[torch.arange(d.shape[0]), safe] -= 1.0
            d.mul_(keep[:, None].to(d.dtype) * scale[0])
            l2.copy_(d)
            ctx.save_for_backward(logits)
            ctx.mark_non_differentiable(valid)
            return per_row.sum() * scale[0], valid
        lib = _need()
        per_row = torch.empty(l2.shape[0], dtype=torch.float32, device=logits.device)
        check(lib.bcom_cross_entropy(ptr(l2), ptr(t), ptr(per_row), ptr(scale), l2.shape[0], V,
                                     int(ignore_index), stream_ptr(logits.device)),
              "cross_entropy")
        ctx.save_for_backward(logits)
        ctx.mark_non_differentiable(valid)
        return per_row.sum() * scale[0], valid

    @staticmethod
    def backward(ctx, dloss, _dvalid):
        (dlogits,) = ctx.saved_tensors
        # the buffer already holds d(loss)/d(logits); scale it by the incoming gradient
        return dlogits.mul_(dloss.to(dlogits.dtype)), None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100,
                  loss_scale: float = 1.0) -> torch.Tensor:
    loss, _ = CrossEntropyFunction.apply(logits, targets, ignore_index, loss_scale)
    return loss


# ----------------------------------------------------------------------------------
class EmbeddingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        H = table.shape[1]
        if not table.is_cuda:  # CPU ranks
            ctx.save_for_backward(flat, table)
            return table.detach().index_select(0, flat).view(*ids.shape, H)
        lib = _need()
        out = torch.empty(flat.numel(), H, dtype=table.dtype, device=table.device)
        check(lib.bcom_embedding_fwd(ptr(flat), ptr(table), ptr(out), flat.numel(), H,
                                     table.shape[0], stream_ptr(table.device)), "embedding_fwd")
        ctx.save_for_backward(flat, table)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        flat, table = ctx.saved_tensors
        H = table.shape[1]
        d = dout.reshape(-1, H)
        if not d.is_contiguous():
            d = d.contiguous()
        main = getattr(table, "main_grad", None)
        dt = main if main is not None else torch.zeros(table.shape, dtype=torch.float32,
                                                        device=table.device)
        if not table.is_cuda:  # CPU ranks
            dt.index_add_(0, flat, d.float())
            return None, (None if main is not None else dt.to(table.dtype))
        lib = _need()
        check(lib.bcom_embedding_bwd(ptr(flat), ptr(d), ptr(dt), flat.numel(), H, table.shape[0],
                                     stream_ptr(table.device)), "embedding_bwd")
        return None, (None if main is not None else dt.to(table.dtype))


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return EmbeddingFunction.apply(ids, table)


# ----------------------------------------------------------------------------------
class FlatAdamW:
    """AdamW over ONE flat fp32 master buffer with a bf16 working copy.

    ``master``, ``grad`` are fp32 ``[n]``; ``params_bf16`` is the bf16 ``[n]`` buffer the
    model's parameters are views of.  One kernel per step updates moments and master,
    refreshes the bf16 copy, applies ``grad_scale`` (e.g. 1 / data-parallel size) and
    zeroes the gradient for the next accumulation."""

    def __init__(self, master: torch.Tensor, grad: torch.Tensor,
                 params_bf16: Optional[torch.Tensor], lr: float = 1e-4,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        n = master.numel()
        if n % 4:
            raise ValueError("flat buffers must be padded to a multiple of 4 elements")
        self.master, self.grad, self.params_bf16 = master, grad, params_bf16
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.exp_avg = torch.zeros_like(master)
        self.exp_avg_sq = torch.zeros_like(master)
        self.step_count = 0

    def _step_host(self, grad_scale: float, zero_grad: bool) -> None:
        """The kernel's arithmetic in torch ops, for buffers that live on the CPU (CPU ranks
        exercise the sharded optimizer's collectives with it)."""
        b1, b2 = self.betas
        g = self.grad * grad_scale
        self.exp_avg.mul_(b1).add_(g, alpha=1.0 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1.0 - b2)
        mhat = self.exp_avg / (1.0 - b1 ** self.step_count)
        vhat = self.exp_avg_sq / (1.0 - b2 ** self.step_count)
        self.master.mul_(1.0 - self.lr * self.weight_decay)
        self.master.addcdiv_(mhat, vhat.sqrt_().add_(self.eps), value=-self.lr)
        if zero_grad:
            self.grad.zero_()
        if self.params_bf16 is not None:
            self.params_bf16.copy_(self.master)

    def step(self, grad_scale: float = 1.0, zero_grad: bool = True) -> None:
        if not self.master.is_cuda:
            self.step_count += 1
            self._step_host(grad_scale, zero_grad)
            return
        lib = _need()
        self.step_count += 1
        check(lib.bcom_adamw(ptr(self.master), ptr(self.params_bf16), ptr(self.grad),
                             ptr(self.exp_avg), ptr(self.exp_avg_sq), self.master.numel(),
                             float(self.lr), float(self.betas[0]), float(self.betas[1]),
                             float(self.eps), float(self.weight_decay), self.step_count,
                             float(grad_scale), int(zero_grad), stream_ptr(self.master.device)),
              "adamw")

    def state_dict(self):
        return {"step": self.step_count, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "master": self.master}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.master.copy_(sd["master"])
        if self.params_bf16 is not None:
            self.params_bf16.copy_(self.master)


class FlatSGD:
    """SGD with momentum over flat fp32 buffers."""

    def __init__(self, param: torch.Tensor, grad: torch.Tensor, lr: float = 0.1,
                 momentum: float = 0.9, weight_decay: float = 0.0):
        self.param, self.grad = param, grad
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.buf = torch.zeros_like(param)

    def step(self, grad_scale: float = 1.0, zero_grad: bool = True) -> None:
        if not self.param.is_cuda:  # the kernel's arithmetic in torch ops, for CPU buffers
            g = self.grad * grad_scale + self.weight_decay * self.param
            self.buf.mul_(self.momentum).add_(g)
            self.param.add_(self.buf, alpha=-self.lr)
            if zero_grad:
                self.grad.zero_()
            return
        lib = _need()
        check(lib.bcom_sgd_momentum(ptr(self.param), ptr(self.grad), ptr(self.buf),
                                    self.param.numel(), float(self.lr), float(self.momentum),
                                    float(self.weight_decay), float(grad_scale), int(zero_grad),
                                    stream_ptr(self.param.device)), "sgd_momentum")
