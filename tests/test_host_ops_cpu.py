"""Host paths of the trainer ops (GEMM, cross-entropy, embedding: what CPU ranks run instead of
the kernels) against plain torch, and the GPT-2 sharded trainer (the fourth benchmark
configuration) on two CPU ranks over gloo."""

import json
import os
import subprocess
import sys

import torch
import torch.nn.functional as F

from bitscom_b200.ops import gemm as G
from bitscom_b200.ops import nn as K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bf(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * 0.5).to(torch.bfloat16)


def test_host_gemm_layouts_and_accumulation():
    a, b = _bf(24, 40, seed=1), _bf(16, 40, seed=2)
    ref = a.float() @ b.float().t()
    assert torch.equal(G.gemm(a, b), ref.to(torch.bfloat16))
    assert torch.equal(G.gemm(a.t().contiguous(), b.t().contiguous(), a_mn_major=True,
                              b_mn_major=True, out_dtype=torch.float32), ref)
    acc = torch.ones(24, 16)
    G.gemm(a, b, out=acc, accumulate=True)
    assert torch.equal(acc, ref + 1)


def test_host_linear_autograd_and_main_grad():
    x = _bf(6, 5, 32, seed=3).requires_grad_()
    w = _bf(8, 32, seed=4).requires_grad_()
    dy = _bf(6, 5, 8, seed=5)
    G.linear(x, w).backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(dy.float())
    assert torch.allclose(x.grad.float(), xr.grad, atol=2e-2, rtol=2e-2)
    assert torch.allclose(w.grad.float(), wr.grad, atol=5e-2, rtol=2e-2)
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(8, 32)
    for _ in range(2):
        G.linear(x.detach(), w2).backward(dy)
    assert w2.grad is None and torch.allclose(w2.main_grad, 2 * wr.grad, atol=1e-4)


def test_host_cross_entropy_matches_torch_and_consumes_logits():
    logits = _bf(10, 64, seed=6).float().mul(4).to(torch.bfloat16)
    targets = torch.tensor([3, 0, 63, -100, 7, 7, -100, 1, 2, 9])
    ref_in = logits.float().requires_grad_()
    ref = F.cross_entropy(ref_in, targets, ignore_index=-100)
    ref.backward()
    x = logits.clone().requires_grad_()
    work = x * 1.0            # the op overwrites its input buffer with the gradient
    loss = K.cross_entropy(work, targets, ignore_index=-100, loss_scale=1.0)
    assert abs(float(loss) - float(ref)) < 1e-5
    (loss * 3.0).backward()
    assert torch.allclose(x.grad.float(), 3.0 * ref_in.grad, atol=2e-3)
    assert x.grad[3].abs().sum() == 0 and x.grad[6].abs().sum() == 0


def test_host_embedding_forward_and_scatter_add():
    table = _bf(20, 8, seed=7).requires_grad_()
    ids = torch.tensor([[1, 5, 5], [19, 0, 5]])
    out = K.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    d = _bf(2, 3, 8, seed=8)
    out.backward(d)
    want = torch.zeros(20, 8).index_add_(0, ids.reshape(-1), d.reshape(-1, 8).float())
    assert torch.allclose(table.grad.float(), want, atol=1e-2)
    t2 = table.detach().clone().requires_grad_()
    t2.main_grad = torch.zeros(20, 8)
    K.embedding(ids, t2).backward(d)
    assert t2.grad is None and torch.equal(t2.main_grad, want)


def test_host_rmsnorm_swiglu_rope_match_fp32_autograd():
    x = _bf(6, 32, seed=11).requires_grad_()
    w = (1 + 0.1 * _bf(32, seed=12).float()).to(torch.bfloat16).requires_grad_()
    dy = _bf(6, 32, seed=13)
    K.rmsnorm(x, w, 1e-5).backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dy.float())
    assert torch.allclose(x.grad.float(), xr.grad, atol=2e-2)
    assert torch.allclose(w.grad.float(), wr.grad, atol=3e-2)

    gu = _bf(5, 16, seed=14).float().mul(2).to(torch.bfloat16).requires_grad_()
    dh = _bf(5, 8, seed=15)
    K.swiglu(gu).backward(dh)
    gr = gu.detach().float().requires_grad_()
    (F.silu(gr[:, :8]) * gr[:, 8:]).backward(dh.float())
    assert torch.allclose(gu.grad.float(), gr.grad, atol=2e-2)

    B, S, nh, hd = 2, 8, 2, 8
    W = nh * hd
    cos, sin = K.rope_tables(S, hd, 1e4, "cpu")
    q = _bf(B * S, 3 * W, seed=16)

    def rotate(t):
        t = t.view(B, S, nh, hd).float()
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        c, s_ = cos[None, :, None, :], sin[None, :, None, :]
        return torch.cat([a * c - b * s_, b * c + a * s_], -1).reshape(B * S, W)

    def reference(t):
        return torch.cat([rotate(t[:, :W]), rotate(t[:, W:2 * W]), t[:, 2 * W:].float()], 1)

    q0 = q.clone().requires_grad_()
    out = K.rope_qk_(q0 * 1.0, cos, sin, nh, hd, S)
    assert torch.allclose(out.float(), reference(q), atol=2e-2)
    g = _bf(B * S, 3 * W, seed=17)
    out.backward(g)
    qr = q.float().requires_grad_()
    reference(qr).backward(g.float())
    assert torch.allclose(q0.grad.float(), qr.grad, atol=2e-2)


def _free_port() -> int:
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _train(tmp_path, mode):
    out = tmp_path / f"{mode}.jsonl"
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         "-m", "bitscom_b200.trainer.gpt2_sharded", "--device", "cpu", "--model", "tiny",
         "--mode", mode, "--steps", "12", "--warmup", "0", "--micro-batch", "2",
         "--out", str(out)],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    return json.loads(out.read_text().strip().splitlines()[-1])


def test_gpt2_sharded_trainer_on_two_cpu_ranks(tmp_path):
    """Tiny GPT-2, ZeRO-1 optimizer on 4-bit reduce-scatter + 8-bit all-gather, and the same
    program with dense collectives ("nccl" mode, gloo here): both run the sharded step on CPU
    ranks, the loss falls, and the two stay close."""
    low, dense = _train(tmp_path, "lowbit"), _train(tmp_path, "nccl")
    for row in (low, dense):
        assert row["device"] == "cpu" and row["world"] == 2 and not row["fused_ops"]
        assert row["loss_last"] < row["loss_first"]
    assert abs(low["loss_last"] - dense["loss_last"]) < 0.05


def _gpt2(nproc, tmp_path, *extra):
    env = dict(os.environ, TORCH_DISTRIBUTED_DEBUG="OFF", OMP_NUM_THREADS="1")
    out = tmp_path / "rows.jsonl"
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(nproc),
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         "-m", "bitscom_b200.trainer.gpt2_sharded", "--device", "cpu", "--model", "tiny",
         "--micro-batch", "2", "--warmup", "0", "--out", str(out), *extra],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    return json.loads(out.read_text().strip().splitlines()[-1])


def test_monolithic_sharded_run_resumes_on_another_number_of_ranks(tmp_path):
    """The same with one bucket (``--zero-buckets one``)."""
    ckpt = str(tmp_path / "ckpt")
    four = _gpt2(4, tmp_path, "--steps", "2", "--output_dir", ckpt)
    assert four["zero_buckets"] == "one"
    again = _gpt2(2, tmp_path, "--steps", "1", "--resume", ckpt)
    assert again["steps_done_before"] == 2
    assert abs(again["master_sum_start"] - four["master_sum_end"]) < 1e-9 * max(
        1.0, abs(four["master_sum_end"]))


def test_sharded_run_resumes_on_another_number_of_ranks(tmp_path):
    """Four ranks train and checkpoint their optimizer shards; two ranks (and then three, whose
    padding differs) pick the state up: the fp32 master weights they start from are the ones
    the four-rank run ended with, and the step counter carries over."""
    ckpt = str(tmp_path / "ckpt")
    four = _gpt2(4, tmp_path, "--steps", "3", "--output_dir", ckpt, "--zero-buckets", "layer")
    assert four["steps_done_before"] == 0 and "overlapped" in four["zero_buckets"]
    assert abs(four["master_sum_end"] - four["master_sum_start"]) > 1e-6   # it did train
    for world in (2, 3):
        again = _gpt2(world, tmp_path, "--steps", "1", "--resume", ckpt, "--zero-buckets",
                      "layer")
        assert again["world"] == world and again["steps_done_before"] == 3
        assert abs(again["master_sum_start"] - four["master_sum_end"]) < 1e-9 * max(
            1.0, abs(four["master_sum_end"]))
