"""tcgen05 causal attention (forward + backward) against fp32 SDPA on the same inputs."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.ops import attention as A


def _ref(qkv, B, S, nh, hd):
    H = nh * hd
    q, k, v = (qkv[:, i * H:(i + 1) * H].view(B, S, nh, hd).transpose(1, 2) for i in range(3))
    o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.transpose(1, 2).reshape(B * S, H)


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("B,S,nh", [(1, 128, 1), (2, 256, 2), (1, 512, 4), (1, 2048, 2)])
def test_attention_forward_backward(B, S, nh, hd):
    assert A.available() and A.supported(S, hd)
    H = nh * hd
    g = torch.Generator(device="cuda").manual_seed(S + nh)
    qkv = (torch.randn(B * S, 3 * H, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    d_out = (torch.randn(B * S, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)

    x = qkv.clone().requires_grad_()
    out = A.attention(x, B, S, nh, hd)
    out.backward(d_out)
    torch.cuda.synchronize()
    A.check_status()

    xr = qkv.float().requires_grad_()
    ref = _ref(xr, B, S, nh, hd)
    ref.backward(d_out.float())

    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, f"forward max err {err}"
    for name, lo in (("dq", 0), ("dk", H), ("dv", 2 * H)):
        got, want = x.grad[:, lo:lo + H].float(), xr.grad[:, lo:lo + H]
        e = (got - want).abs().max().item()
        tol = 3e-2 * max(1.0, want.abs().max().item())
        assert e < tol, f"{name} max err {e} (tol {tol})"


@pytest.mark.parametrize("variant", ["pipelined", "simple"])
@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("B,S,nh", [(1, 128, 1), (2, 384, 2), (1, 2048, 2)])
def test_forward_variants_match_reference(B, S, nh, hd, variant):
    """Both forward kernels against fp32 SDPA: the software-pipelined one (issuer warp, scores
    double-buffered in TMEM, output accumulated in TMEM with rescaling on demand; the default)
    and the simple one whose MMA and softmax take turns.  The log-sum-exp each writes is
    checked through the backward pass of the same call."""
    H = nh * hd
    g = torch.Generator(device="cuda").manual_seed(S + nh + hd)
    qkv = (torch.randn(B * S, 3 * H, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    d_out = (torch.randn(B * S, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    before = A.set_forward_variant(variant)
    try:
        x = qkv.clone().requires_grad_()
        out = A.attention(x, B, S, nh, hd)
        out.backward(d_out)
        torch.cuda.synchronize()
        A.check_status()
    finally:
        A.set_forward_variant(before)
    xr = qkv.float().requires_grad_()
    ref = _ref(xr, B, S, nh, hd)
    ref.backward(d_out.float())
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, f"forward max err {err}"
    e = (x.grad.float() - xr.grad).abs().max().item()
    assert e < 3e-2 * max(1.0, xr.grad.abs().max().item()), f"grad max err {e}"


@pytest.mark.parametrize("dq", ["tma", "atomic"])
@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("B,S,nh", [(1, 128, 1), (2, 384, 2), (1, 1024, 3)])
def test_backward_dq_variants_match_reference(B, S, nh, hd, dq):
    """dQ accumulated by TMA reductions from a swizzled staging tile, and by float4 atomics,
    against fp32 autograd; two calls in a row (the accumulator must be left zeroed)."""
    H = nh * hd
    g = torch.Generator(device="cuda").manual_seed(7 * S + nh + hd)
    qkv = (torch.randn(B * S, 3 * H, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    d_out = (torch.randn(B * S, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    xr = qkv.float().requires_grad_()
    _ref(xr, B, S, nh, hd).backward(d_out.float())
    before = A.set_backward_dq_variant(dq)
    try:
        for _ in range(2):
            x = qkv.clone().requires_grad_()
            A.attention(x, B, S, nh, hd).backward(d_out)
            torch.cuda.synchronize()
            A.check_status()
            for name, lo in (("dq", 0), ("dk", H), ("dv", 2 * H)):
                got, want = x.grad[:, lo:lo + H].float(), xr.grad[:, lo:lo + H]
                e = (got - want).abs().max().item()
                tol = 3e-2 * max(1.0, want.abs().max().item())
                assert e < tol, f"{name} max err {e} (tol {tol})"
    finally:
        A.set_backward_dq_variant(before)


def test_attention_second_call_reuses_zeroed_scratch():
    B, S, nh, hd = 1, 256, 2, 128
    H = nh * hd
    qkv = (torch.randn(B * S, 3 * H, device="cuda") * 0.5).to(torch.bfloat16)
    d_out = (torch.randn(B * S, H, device="cuda") * 0.5).to(torch.bfloat16)
    grads = []
    for _ in range(2):
        x = qkv.clone().requires_grad_()
        A.attention(x, B, S, nh, hd).backward(d_out)
        grads.append(x.grad.clone())
    assert torch.equal(grads[0], grads[1])


@pytest.mark.performance
def test_attention_throughput_report():
    B, S, nh, hd = 2, 2048, 32, 128
    H = nh * hd
    qkv = (torch.randn(B * S, 3 * H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    d_out = (torch.randn(B * S, H, device="cuda") * 0.5).to(torch.bfloat16)
    flops_fwd = 4 * B * nh * S * S * hd / 2
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for _ in range(2):
        A.attention(qkv, B, S, nh, hd).backward(d_out)
    ev[0].record()
    out = A.attention(qkv, B, S, nh, hd)
    ev[1].record()
    out.backward(d_out)
    ev[2].record()
    torch.cuda.synchronize()
    A.check_status()
    f, b = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
    print(f"attention fwd {f:.3f} ms = {flops_fwd / f / 1e9:.0f} TFLOP/s; "
          f"bwd {b:.3f} ms = {2.5 * flops_fwd / b / 1e9:.0f} TFLOP/s")
