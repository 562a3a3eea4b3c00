"""tcgen05 GEMM against a plain fp32 matmul of the same bf16 inputs."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.ops import gemm as G


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


def _mk(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(rows, cols, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


def _check(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    tol = 0.02 * (K ** 0.5) * 0.25 + 0.02 * ref.abs().max().item()
    assert err <= tol, f"max err {err} > {tol}"


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 256, 1024),
                                   (200, 264, 136), (1024, 1024, 4096), (77, 8, 40)])
def test_gemm_matches_fp32_reference(a_mn, b_mn, M, N, K):
    a = _mk(K, M, 1) if a_mn else _mk(M, K, 1)
    b = _mk(K, N, 2) if b_mn else _mk(N, K, 2)
    if (a.shape[1] % 8) or (b.shape[1] % 8):
        pytest.skip("row stride must stay 16-byte aligned")
    out = G.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    G.check_status()
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    _check(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_exact_on_small_integers():
    a = torch.randint(-3, 4, (256, 192), device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (512, 192), device="cuda").to(torch.bfloat16)
    out = G.gemm(a, b, out_dtype=torch.float32)
    assert torch.equal(out, a.float() @ b.float().t())


def test_fp32_output_and_accumulate():
    a, b = _mk(300, 512, 3), _mk(520, 512, 4)
    ref = a.float() @ b.float().t()
    out = G.gemm(a, b, out_dtype=torch.float32)
    _check(out, ref, 512)
    G.gemm(a, b, out=out, accumulate=True)
    _check(out, 2 * ref, 512)
    ob = G.gemm(a, b)
    G.gemm(a, b, out=ob, accumulate=True)
    _check(ob, 2 * ref, 2048)
    G.check_status()


def test_strided_operands():
    big = _mk(512, 1024, 5)
    a = big[:, 256:768]          # row stride 1024, 512 columns
    b = _mk(256, 512, 6)
    out = G.gemm(a, b)
    _check(out, a.float() @ b.float().t(), 512)


def test_gemm_from_a_worker_thread():
    import threading

    a, b = _mk(512, 768, 11), _mk(768, 1024, 12)
    box = {}

    def work():
        try:
            box["out"] = G.gemm(a, b, b_mn_major=True)
        except Exception as exc:  # surfaced in the main thread
            box["err"] = exc

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "err" not in box, box.get("err")
    _check(box["out"], a.float() @ b.float(), 768)


def test_linear_autograd_matches_torch():
    x = _mk(512, 1024, 7).requires_grad_()
    w = _mk(768, 1024, 8).requires_grad_()
    y = G.linear(x.view(4, 128, 1024), w)
    dy = _mk(512, 768, 9).view(4, 128, 768)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = (xr @ wr.t()).view(4, 128, 768)
    yr.backward(dy.float())
    _check(y, yr.detach(), 1024)
    _check(x.grad, xr.grad, 768)
    _check(w.grad, wr.grad, 512)
    # fp32 main_grad accumulation
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(768, 1024, device="cuda")
    for _ in range(2):
        G.linear(x.detach().view(4, 128, 1024), w2).backward(dy)
    _check(w2.main_grad, 2 * wr.grad, 1024)
    assert w2.grad is None
    G.check_status()


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 256), (512, 256, 1024),
                                   (200, 264, 136), (1024, 1024, 4096), (77, 8, 40),
                                   (4096, 4096, 512)])
def test_cta_pair_gemm(a_mn, b_mn, M, N, K):
    """The CTA-pair kernel (256x256 tiles, tcgen05 cta_group::2) against fp32 matmul, bf16 and
    accumulating fp32 outputs; exact on small integers, so a swapped half tile cannot hide in
    the tolerance."""
    if not G.pair_available():
        pytest.skip("the CTA-pair library is not part of this installation")
    a = _mk(K, M, 1) if a_mn else _mk(M, K, 1)
    b = _mk(K, N, 2) if b_mn else _mk(N, K, 2)
    if (a.shape[1] % 8) or (b.shape[1] % 8):
        pytest.skip("row stride must stay 16-byte aligned")
    ai = torch.randint(-3, 4, a.shape, device="cuda").to(torch.bfloat16)
    bi = torch.randint(-3, 4, b.shape, device="cuda").to(torch.bfloat16)
    before = G.set_variant("2cta")
    try:
        out = G.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
        acc = G.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
        G.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=acc, accumulate=True)
        exact = G.gemm(ai, bi, a_mn_major=a_mn, b_mn_major=b_mn, out_dtype=torch.float32)
        torch.cuda.synchronize()
        G.check_status()
    finally:
        G.set_variant(before)
    ref = _ref(a, b, a_mn, b_mn)
    _check(out, ref, K)
    _check(acc, 2 * ref, K)
    assert torch.equal(exact, _ref(ai, bi, a_mn, b_mn))


def test_gemm_throughput_report():
    M = N = K = 8192
    a, b = _mk(M, K, 1), _mk(N, K, 2)
    for _ in range(3):
        G.gemm(a, b)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        out = G.gemm(a, b)
    e.record()
    torch.cuda.synchronize()
    G.check_status()
    ms = s.elapsed_time(e) / 10
    tf = 2 * M * N * K / ms / 1e9
    s.record()
    for _ in range(10):
        ref = a @ b.t()
    e.record()
    torch.cuda.synchronize()
    ms_ref = s.elapsed_time(e) / 10
    print(f"tcgen05 gemm 8192^3: {ms:.3f} ms = {tf:.0f} TFLOP/s; "
          f"torch.matmul {ms_ref:.3f} ms = {2 * M * N * K / ms_ref / 1e9:.0f} TFLOP/s")
    _check(out, ref.float(), K)
    assert tf > 300
