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
            "loss": last}), flush=True)
    if world > 1:
        dist.destroy_process_group()
