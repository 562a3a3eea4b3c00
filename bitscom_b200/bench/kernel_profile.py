"""Small single-GPU workloads for profiling one kernel at a time (ncu-sized).

    python -m bitscom_b200.bench.kernel_profile fused   --elems 33554432 --bits 4 --world 2
    python -m bitscom_b200.bench.kernel_profile codec   --elems 67108864 --bits 4
    python -m bitscom_b200.bench.kernel_profile gemm    --m 4096 --n 4096 --k 4096

Each case warms up, then times a few launches with CUDA events (inputs larger than L2,
or rotated so that L2 does not hold them) and prints one JSON line with the achieved
bandwidth / throughput and its fraction of the measured peaks.
"""

from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "of measured"
    return 6650.0, 1590.0, "of fallback"


def _timed(fn, iters, reps=3):
    """Mean time of ``iters`` back-to-back launches, median over ``reps`` repetitions (one
    slow launch on a cold box would otherwise dominate a five-launch mean)."""
    means = []
    for r in range(reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for i in range(iters):
            fn(r * iters + i)  # a running index: a case may consume one item per call
        e.record()
        torch.cuda.synchronize()
        means.append(s.elapsed_time(e) / iters)
    return sorted(means)[len(means) // 2]


def fused(args):
    from bitscom_b200.parallel import fused as F

    hbm, _, tag = _peaks()
    W, n = args.world, args.elems
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    world = F.EmulatedWorld(W, "cuda:0", region_bytes=args.region_mb << 20)
    S = -(-n // W)
    bufs = [(torch.randn(n, device="cuda") * 1e-3).to(dtype) for _ in range(W)]
    ef = not args.no_ef
    res1 = [torch.zeros(S * W, device="cuda") for _ in range(W)] if ef else None
    res2 = [torch.zeros(S, device="cuda") for _ in range(W)] if ef else None

    shards = [torch.empty(S, dtype=dtype, device="cuda") for _ in range(W)]
    if args.mode != "allreduce":
        bufs = [b[:S * W] if b.numel() >= S * W else torch.cat(
            [b, b.new_zeros(S * W - b.numel())]) for b in bufs]

    def run(i):
        kw = dict(bitwidth=args.bits, block_size=256, stochastic=not args.nearest, seed=i)
        if args.mode == "reduce_scatter":     # phases 1 and 2 without the re-quantize
            world.reduce_scatter(shards, bufs, res1=res1, **kw)
        elif args.mode == "all_gather":       # phase 2 fed from the input, and phase 3
            world.all_gather(bufs, shards, res2=res2, **kw)
        else:
            world.all_reduce(bufs, res1=res1, res2=res2, **kw)

    for i in range(args.warmup):
        run(i)
    ms = _timed(run, args.iters)
    assert all(s[0] == 0 for s in world.status())
    torch.cuda.synchronize()
    phases = world.phase_times_us()[0]   # rank 0's first CTA, last launch
    esize = 4 if dtype == torch.float32 else 2
    pk = args.bits / 8 + 2 / 256
    phase1 = n * (esize + (8 if ef else 0) + pk)
    phase2_in, requant = W * S * pk, W * S * pk + (S * 8 if ef else 0)
    phase3 = n * (pk + esize)
    if args.mode == "reduce_scatter":
        per_rank = phase1 + phase2_in + S * esize
    elif args.mode == "all_gather":
        per_rank = S * esize + requant + phase3
    else:
        per_rank = phase1 + phase2_in + requant + phase3
    total = per_rank * W  # all emulated ranks share one GPU's HBM
    print(json.dumps({"case": f"fused_{args.mode}_emulated", "world": W, "elems": n,
                      "rounding": "nearest" if args.nearest else "stochastic",
                      "dtype": args.dtype, "bits": args.bits, "ef": ef, "ms": ms,
                      "hbm_bytes": total, "gbs": total / ms / 1e6,
                      "frac_hbm": total / ms / 1e6 / hbm, "peaks": tag,
                      "phases_us_rank0": phases}))
    world.close()


def codec(args):
    from bitscom_b200.ops import codec as C

    hbm, _, tag = _peaks()
    n = args.elems
    x = torch.randn(n, device="cuda") * 1e-3
    if args.dtype == "bf16":
        x = x.to(torch.bfloat16)
    p, s = C.blockwise_quantize_pack(x, args.bits, 256)
    for _ in range(args.warmup):
        C.blockwise_quantize_pack(x, args.bits, 256)
    ms_q = _timed(lambda i: C.blockwise_quantize_pack(x, args.bits, 256), args.iters)
    ms_d = _timed(lambda i: C.blockwise_unpack_dequantize(p, s, args.bits, n, 256, x.dtype),
                  args.iters)
    nbytes = n * x.element_size() + p.numel() + s.numel() * 2
    print(json.dumps({"case": "codec", "elems": n, "dtype": args.dtype, "bits": args.bits,
                      "quantize_ms": ms_q, "quantize_gbs": nbytes / ms_q / 1e6,
                      "quantize_frac_hbm": nbytes / ms_q / 1e6 / hbm,
                      "dequantize_ms": ms_d, "dequantize_gbs": nbytes / ms_d / 1e6,
                      "dequantize_frac_hbm": nbytes / ms_d / 1e6 / hbm, "peaks": tag}))


def gemm(args):
    from bitscom_b200.ops import gemm as G

    _, tflops, tag = _peaks()
    G.set_variant(args.gemm_variant)
    M, N, K = args.m, args.n, args.k
    copies = max(1, min(8, (256 << 20) // max(1, (M * K + N * K) * 2)))
    As = [(torch.randn(M, K, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(copies)]
    Bs = [(torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(copies)]
    if args.wgrad:
        # weight-gradient form: dW[M, N] += dY^T X with dY stored [K, M], X stored [K, N]
        As = [(torch.randn(K, M, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(copies)]
        Bs = [(torch.randn(K, N, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(copies)]
        acc = torch.zeros(M, N, device="cuda")

        def run(i):
            G.gemm(As[i % copies], Bs[i % copies], a_mn_major=True, b_mn_major=True, out=acc,
                   accumulate=True)
    else:
        def run(i):
            G.gemm(As[i % copies], Bs[i % copies])
    for i in range(args.warmup):
        run(i)
    ms = _timed(run, args.iters)
    G.check_status()
    if args.wgrad:
        tf = 2 * M * N * K / ms / 1e9
        print(json.dumps({"case": "gemm_tcgen05_wgrad_fp32_accumulate",
                          "variant": args.gemm_variant, "M": M, "N": N, "K": K, "ms": ms,
                          "tflops": tf, "frac_bf16_peak": tf / tflops, "peaks": tag}))
        return
    ms_ref = _timed(lambda i: torch.matmul(As[i % copies], Bs[i % copies].t()), args.iters)
    tf = 2 * M * N * K / ms / 1e9
    print(json.dumps({"case": "gemm_tcgen05", "variant": args.gemm_variant, "M": M, "N": N,
                      "K": K, "ms": ms, "tflops": tf,
                      "frac_bf16_peak": tf / tflops, "torch_matmul_ms": ms_ref,
                      "torch_tflops": 2 * M * N * K / ms_ref / 1e9, "peaks": tag}))


def attention(args):
    from bitscom_b200.ops import attention as A

    _, tflops, tag = _peaks()
    B, S, nh, hd = args.batch, args.seq, args.heads, args.head_dim
    A.set_forward_variant(args.fwd_variant)
    A.set_backward_dq_variant(args.bwd_dq)
    H = nh * hd
    qkv = (torch.randn(B * S, 3 * H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    d_out = (torch.randn(B * S, H, device="cuda") * 0.5).to(torch.bfloat16)
    for _ in range(args.warmup):
        A.attention(qkv, B, S, nh, hd).backward(d_out)
    ms_f = _timed(lambda i: A.attention(qkv, B, S, nh, hd), args.iters)
    # the backward pass consumes one forward graph per call: build them outside the timing
    outs = [A.attention(qkv, B, S, nh, hd) for _ in range(3 * args.iters)]
    ms_b = _timed(lambda i: outs[i].backward(d_out), args.iters)
    A.check_status()
    flops = 4.0 * B * nh * S * S * hd / 2
    q, k, v = (qkv.detach()[:, i * H:(i + 1) * H].view(B, S, nh, hd).transpose(1, 2)
               for i in range(3))
    ms_ref = _timed(lambda i: torch.nn.functional.scaled_dot_product_attention(
        q, k, v, is_causal=True), args.iters)
    print(json.dumps({"case": "attention_tcgen05", "batch": B, "seq": S, "heads": nh,
                      "head_dim": hd, "fwd_variant": args.fwd_variant, "bwd_dq": args.bwd_dq,
                      "fwd_ms": ms_f, "fwd_tflops": flops / ms_f / 1e9,
                      "fwd_frac_bf16_peak": flops / ms_f / 1e9 / tflops,
                      "bwd_ms": ms_b, "bwd_tflops": 2.5 * flops / ms_b / 1e9,
                      "bwd_frac_bf16_peak": 2.5 * flops / ms_b / 1e9 / tflops,
                      "sdpa_fwd_ms": ms_ref, "peaks": tag}))


def elementwise(args):
    from bitscom_b200.ops import nn as K


    hbm, _, tag = _peaks()
    T, H, F, V = args.tokens, 4096, 11008, 32000
    rows = []

    def bf(*shape):
        return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)

    x, w = bf(T, H).requires_grad_(), bf(H).requires_grad_()
    w.main_grad = torch.zeros(H, device="cuda")
    dy = bf(T, H)
    for _ in range(args.warmup):  # first launches load the kernels and grow the allocator
        K.rmsnorm(x, w).backward(dy)
    ms = _timed(lambda i: K.rmsnorm(x, w), args.iters)
    rows.append(("rmsnorm_fwd", ms, 2 * T * H * 2))
    ms = _timed(lambda i: K.rmsnorm(x, w).backward(dy), args.iters) - ms
    rows.append(("rmsnorm_bwd", ms, 3 * T * H * 2))
    gu, dh = bf(T, 2 * F).requires_grad_(), bf(T, F)
    for _ in range(args.warmup):
        K.swiglu(gu).backward(dh)
    ms_f = _timed(lambda i: K.swiglu(gu), args.iters)
    rows.append(("swiglu_fwd", ms_f, 3 * T * F * 2))
    ms = _timed(lambda i: K.swiglu(gu).backward(dh), args.iters) - ms_f
    rows.append(("swiglu_bwd", ms, 5 * T * F * 2))
    # GPT-2 medium shapes: LayerNorm over 1024, bias + GELU over 4096
    xl, wl, bl = bf(T, 1024).requires_grad_(), bf(1024).requires_grad_(), bf(1024).requires_grad_()
    wl.main_grad, bl.main_grad = torch.zeros(1024, device="cuda"), torch.zeros(1024, device="cuda")
    dyl = bf(T, 1024)
    for _ in range(args.warmup):
        K.layernorm(xl, wl, bl).backward(dyl)
    ms_f = _timed(lambda i: K.layernorm(xl, wl, bl), args.iters)
    rows.append(("layernorm_fwd", ms_f, 2 * T * 1024 * 2))
    ms = _timed(lambda i: K.layernorm(xl, wl, bl).backward(dyl), args.iters) - ms_f
    rows.append(("layernorm_bwd", ms, 3 * T * 1024 * 2))
    xg, bg = bf(T, 4096).requires_grad_(), bf(4096).requires_grad_()
    bg.main_grad = torch.zeros(4096, device="cuda")
    dyg = bf(T, 4096)
    for _ in range(args.warmup):
        K.bias_gelu(xg, bg).backward(dyg)
    ms_f = _timed(lambda i: K.bias_gelu(xg, bg), args.iters)
    rows.append(("bias_gelu_fwd", ms_f, 2 * T * 4096 * 2))
    ms = _timed(lambda i: K.bias_gelu(xg, bg).backward(dyg), args.iters) - ms_f
    rows.append(("bias_gelu_bwd", ms, 3 * T * 4096 * 2))
    logits = bf(T, V)
    tgt = torch.randint(1, V, (T,), device="cuda")
    for _ in range(args.warmup):
        K.cross_entropy(logits, tgt, 0)
    ms = _timed(lambda i: K.cross_entropy(logits, tgt, 0), args.iters)
    rows.append(("cross_entropy_fwd_bwd", ms, 4 * T * V * 2))
    n = 1 << 28
    master, grad = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    opt = K.FlatAdamW(master, grad, torch.empty(n, device="cuda", dtype=torch.bfloat16))
    opt.step()
    ms = _timed(lambda i: opt.step(), args.iters)
    rows.append(("adamw_flat", ms, n * 34))
    print(json.dumps({"case": "elementwise", "tokens": T, "peaks": tag, "kernels": [
        {"name": nm, "ms": ms, "gbs": b / ms / 1e6, "frac_hbm": b / ms / 1e6 / hbm}
        for nm, ms, b in rows]}))


def norms_raw(args):
    """Device time of the normalisation / activation backward kernels themselves: the native
    entry points are called directly on preallocated buffers, back to back, so that neither
    autograd nor the allocator sits between two launches (at these sizes a Python-level
    forward + backward costs more host time than the kernels take on the device)."""
    from bitscom_b200.ops import nn as K
    from bitscom_b200.ops._native import ptr, stream_ptr

    lib = K._need()
    hbm, _, tag = _peaks()
    T = args.tokens
    dev = torch.device("cuda")
    st = stream_ptr(dev)

    def bf(*shape):
        return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)

    rows = []
    copies = 4  # rotate over buffers larger than L2 in total

    def rms(H):
        xs, dys = [bf(T, H) for _ in range(copies)], [bf(T, H) for _ in range(copies)]
        w, rstd = bf(H), torch.rand(T, device="cuda") + 0.5
        dx, dw = torch.empty_like(xs[0]), torch.zeros(H, device="cuda")
        scratch = torch.empty(int(lib.bcom_norm_bwd_scratch_elems(H, 0)), device="cuda")
        res = bf(T, H)
        plain = lambda i: lib.bcom_rmsnorm_bwd(  # noqa: E731
            ptr(dys[i % copies]), ptr(xs[i % copies]), ptr(w), ptr(rstd), None, ptr(dx), ptr(dw),
            ptr(scratch), T, H, st)
        fused = lambda i: lib.bcom_rmsnorm_bwd(  # noqa: E731
            ptr(dys[i % copies]), ptr(xs[i % copies]), ptr(w), ptr(rstd), ptr(res), ptr(dx),
            ptr(dw), ptr(scratch), T, H, st)
        for name, fn, nb in (("rmsnorm_bwd", plain, 3), ("rmsnorm_bwd_plus_residual", fused, 4)):
            for i in range(3):
                fn(i)
            rows.append((f"{name}_H{H}", _timed(fn, 20), nb * T * H * 2))

    def ln(H):
        xs, dys = [bf(T, H) for _ in range(copies)], [bf(T, H) for _ in range(copies)]
        w = bf(H)
        mean, rstd = torch.randn(T, device="cuda") * 0.1, torch.rand(T, device="cuda") + 0.5
        dx = torch.empty_like(xs[0])
        dw, db = torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda")
        scratch = torch.empty(int(lib.bcom_norm_bwd_scratch_elems(H, 1)), device="cuda")
        bwd = lambda i: lib.bcom_layernorm_bwd(  # noqa: E731
            ptr(dys[i % copies]), ptr(xs[i % copies]), ptr(w), ptr(mean), ptr(rstd), ptr(dx),
            ptr(dw), ptr(db), ptr(scratch), T, H, st)
        for i in range(3):
            bwd(i)
        rows.append((f"layernorm_bwd_H{H}", _timed(bwd, 20), 3 * T * H * 2))
        y, mo, ro, b = torch.empty_like(xs[0]), torch.empty(T, device="cuda"), \
            torch.empty(T, device="cuda"), bf(H)
        fwd = lambda i: lib.bcom_layernorm_fwd(  # noqa: E731
            ptr(xs[i % copies]), ptr(w), ptr(b), ptr(y), ptr(mo), ptr(ro), T, H, 1e-5, st)
        for i in range(3):
            fwd(i)
        rows.append((f"layernorm_fwd_H{H}", _timed(fwd, 20), 2 * T * H * 2))

    def swiglu(F):
        gus, dhs = [bf(T, 2 * F) for _ in range(2)], [bf(T, F) for _ in range(2)]
        h, dgu = torch.empty(T, F, device="cuda", dtype=torch.bfloat16), torch.empty_like(gus[0])
        fwd = lambda i: lib.bcom_swiglu_fwd(ptr(gus[i % 2]), ptr(h), T, F, st)  # noqa: E731
        bwd = lambda i: lib.bcom_swiglu_bwd(ptr(gus[i % 2]), ptr(dhs[i % 2]), ptr(dgu), T, F,  # noqa: E731
                                            st)
        for name, fn, nb in (("swiglu_fwd", fwd, 3), ("swiglu_bwd", bwd, 5)):
            for i in range(3):
                fn(i)
            rows.append((name, _timed(fn, 20), nb * T * F * 2))

    def gelu(C):
        xs, dys = [bf(T, C) for _ in range(copies)], [bf(T, C) for _ in range(copies)]
        b, dx, db = bf(C), torch.empty_like(xs[0]), torch.zeros(C, device="cuda")
        bwd = lambda i: lib.bcom_bias_gelu_bwd(  # noqa: E731
            ptr(dys[i % copies]), ptr(xs[i % copies]), ptr(b), ptr(dx), ptr(db), T, C, st)
        for i in range(3):
            bwd(i)
        rows.append((f"bias_gelu_bwd_C{C}", _timed(bwd, 20), 3 * T * C * 2))

    rms(4096)
    ln(1024)
    swiglu(11008)
    gelu(4096)
    print(json.dumps({"case": "norms_raw", "tokens": T, "peaks": tag, "kernels": [
        {"name": nm, "ms": ms, "gbs": b / ms / 1e6, "frac_hbm": b / ms / 1e6 / hbm}
        for nm, ms, b in rows]}))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["fused", "codec", "gemm", "attention", "elementwise",
                                     "norms_raw"])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128])
    ap.add_argument("--fwd-variant", default="pipelined",
                    choices=["simple", "pipelined"])
    ap.add_argument("--bwd-dq", default="tma", choices=["atomic", "tma"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--elems", type=int, default=1 << 25)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--region-mb", type=int, default=64)
    ap.add_argument("--no-ef", action="store_true")
    ap.add_argument("--mode", default="allreduce",
                    choices=["allreduce", "reduce_scatter", "all_gather"])
    ap.add_argument("--nearest", action="store_true")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--wgrad", action="store_true")
    ap.add_argument("--gemm-variant", default="1cta", choices=["1cta", "2cta"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    {"fused": fused, "codec": codec, "gemm": gemm, "attention": attention,
     "elementwise": elementwise, "norms_raw": norms_raw}[args.case](args)


if __name__ == "__main__":
    main()
