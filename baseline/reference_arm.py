"""Reference arm of bench.py: the UNMODIFIED reference library installed under
``baseline/_ref`` (``pip install --target baseline/_ref`` of Squirrel7ang/bitscom), driven
the way its own trainer drives it (``benchmarks/train_llama7b_dp_pp_lowbit.py``): fp32
parameters, ``torch.optim.AdamW``, one synchronous ``LowBitGroup.all_reduce`` per
parameter gradient followed by ``div_(dp_size)``.

Two substitutions are unavoidable and are reported in the JSON line:
  * the model class: the reference imports ``MyLlamaForCausalLM`` from a package
    (``psgd``) that is not part of its tree; ``transformers.LlamaForCausalLM`` with the
    same config (vocab 32000, hidden 4096, ffn 11008, 32 layers, 32 heads, rope 1e4, tied
    embeddings), randomly initialised, stands in;
  * the data: the reference downloads a tokenizer and a dataset; synthetic uniform token
    ids of the same shape are used.
Pipeline parallelism of the reference goes through ``torch.distributed.pipelining`` on
the external model class's attribute names and cannot be reproduced without rewriting
it, so this arm runs data parallelism only (pp = 1) at every N.
"""

from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args) -> None:
    if not os.path.isdir(os.path.join(REF, "bitscom")):
        _unavailable("baseline/_ref/bitscom is not installed on this machine")
        return
    try:
        _run(args)
    except SystemExit:
        raise
    except BaseException as exc:  # report instead of failing the driver
        _unavailable(f"{type(exc).__name__}: {str(exc)[:200]}")


def _allreduce_block(bitscom, torch, dist, dev, world, sizes_mb) -> dict:
    """The reference's ``LowBitGroup(...).all_reduce`` (its Python pipeline over NCCL with its
    own CUDA quantize kernels: 4-bit, block 256, stochastic rounding; it has no error feedback
    on this path) against NCCL bf16 / fp32 on the same buckets as the other arm's block.
    CUDA events, rotating buffers larger than L2 in total, max over ranks."""
    group = bitscom.LowBitGroup(bitwidth=4, process_group=dist.group.WORLD,
                                stochastic_rounding=True, block_size=256)

    def time_ms(fn, bufs, iters=5, warmup=3):
        for i in range(warmup):
            fn(bufs[i % len(bufs)])
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(bufs[i % len(bufs)])
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rows = []
    for mb in sizes_mb:
        size = int(mb * (1 << 20))
        for dname, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
            n = size // (4 if dtype == torch.float32 else 2)
            copies = max(2, min(8, -(-(252 << 20) // size)))
            row = {"bytes": size, "bucket_dtype": dname, "numel": n, "world": world, "bits": 4,
                   "stochastic_rounding": True, "error_feedback": False}
            try:
                bufs = [(torch.randn(n, device=dev) * 1e-3).to(dtype) for _ in range(copies)]
                other = torch.bfloat16 if dtype == torch.float32 else torch.float32
                obufs = [torch.zeros(n, device=dev, dtype=other) for _ in range(copies)]
                same = time_ms(lambda t: dist.all_reduce(t), bufs)
                oth = time_ms(lambda t: dist.all_reduce(t), obufs)
                del obufs
                ms = time_ms(lambda t: group.all_reduce(t), bufs)
                bf16_ms = oth if dtype == torch.float32 else same
                fp32_ms = same if dtype == torch.float32 else oth
                row.update(lowbit_ms=ms, nccl_bf16_ms=bf16_ms, nccl_fp32_ms=fp32_ms,
                           lowbit_effective_gbs=n * 4 / ms / 1e6, vs_nccl_bf16=bf16_ms / ms,
                           vs_nccl_fp32=fp32_ms / ms)
                del bufs
            except BaseException as exc:  # e.g. out of memory in the reference's temporaries
                row["error"] = f"{type(exc).__name__}: {str(exc)[:160]}"
            torch.cuda.empty_cache()
            rows.append(row)
    return {"setting": "reference LowBitGroup Python pipeline over NCCL: 4-bit, block 256, "
                       "stochastic rounding, no error feedback (its C++ backend, the path with "
                       "error feedback, crashes in its constructor under torch 2.11)",
            "world": world, "rows": rows,
            "timing": "CUDA events, 5 calls after 3 warm-ups on rotating buffers, max over ranks"}


def _run(args) -> None:
    sys.path.insert(0, REF)
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    import bitscom  # the reference package
    from transformers import LlamaConfig, LlamaForCausalLM

    assert os.path.realpath(bitscom.__file__).startswith(os.path.realpath(REF))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # a short collective timeout: if one rank fails, the others report instead of waiting
        from datetime import timedelta

        dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=240))

    allreduce = None
    if world > 1 and not getattr(args, "no_allreduce_block", False):
        allreduce = _allreduce_block(bitscom, torch, dist, dev, world,
                                     getattr(args, "allreduce_mb", [64, 1024]))

    seq, micro_batches = 2048, 4
    cfg = LlamaConfig(vocab_size=32000, hidden_size=4096, intermediate_size=11008,
                      num_hidden_layers=32, num_attention_heads=32, rope_theta=10000.0,
                      pad_token_id=0, tie_word_embeddings=True,
                      max_position_embeddings=seq)
    if args.model != "llama7b":
        cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512,
                          num_hidden_layers=2, num_attention_heads=2, pad_token_id=0,
                          tie_word_embeddings=True, max_position_embeddings=256)
        seq = 256
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg)   # fp32 parameters, as in the reference trainer
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    group = bitscom.LowBitGroup(bitwidth=4, process_group=dist.group.WORLD) if world > 1 \
        else None

    def loss_fn(logits, target):
        return F.cross_entropy(logits[..., :-1, :].reshape(-1, logits.size(-1)),
                               target[..., 1:].reshape(-1), ignore_index=0)

    def batch(step):
        g = torch.Generator().manual_seed(1000003 * (step + 1) + rank)
        return torch.randint(1, cfg.vocab_size, (micro_batches, 1, seq),
                             generator=g).pin_memory()

    def train_step(ids_host):
        ids = ids_host.to(dev, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        total = 0.0
        for mb in range(micro_batches):
            out = model(input_ids=ids[mb]).logits
            loss = loss_fn(out, ids[mb]) / micro_batches
            loss.backward()
            total = total + loss.detach()
        if group is not None:
            for p in model.parameters():
                if p.grad is None:
                    continue
                group.all_reduce(p.grad, op=dist.ReduceOp.SUM, async_op=False)
                p.grad.div_(world)
        opt.step()
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        train_step(batch(i))
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    last = None
    for i in range(args.steps):
        last = float(train_step(batch(args.warmup + i)).item())
    end.record()
    barrier()
    ms = torch.tensor([start.elapsed_time(end)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    tokens = world * micro_batches * seq
    value = tokens * args.steps / (float(ms.item()) / 1e3)
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": "llama7b_dp_pp_train_tokens_per_s",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": float(ms.item()) / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32 (the reference trainer's default dtype)",
            "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": "llama-7b" if args.model == "llama7b" else "tiny",
                       "global_batch": world * micro_batches, "seq_len": seq,
                       "parallelism": f"dp{world}xpp1",
                       "grad_sync": "reference LowBitGroup.all_reduce per parameter, 4-bit"},
            "substitutions": ["transformers.LlamaForCausalLM for psgd.MyLlamaForCausalLM",
                              "synthetic token ids for the downloaded dataset",
                              "pp=1 (reference PP path depends on the missing model class)"],
            "e2e": {"value": value, "unit": "tokens/s",
                    "h2d_bytes_per_step": micro_batches * seq * 8, "d2h_bytes_per_step": 4},
            "loss": last, **({"allreduce": allreduce} if allreduce is not None else {})}),
            flush=True)
    if world > 1:
        dist.destroy_process_group()
