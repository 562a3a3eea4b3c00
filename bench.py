"""Headline benchmark: Llama-7B DP x PP training tokens/s (synthetic data, random init).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Config: 32 layers, hidden 4096, 32 heads, FFN 11008 SwiGLU, RMSNorm, RoPE, vocab 32000,
sequence 2048, bf16 compute with fp32 master weights, AdamW.  N = 1 runs one stage; N >= 2
runs PP = 2 with 1F1B over NCCL p2p and DP = N / 2 with the 4-bit low-bit gradient
all-reduce (error feedback on).  Per-GPU work is fixed as N grows (weak scaling): each
data-parallel replica processes 4 * PP micro-batches of two sequences per step (16384
tokens per GPU per step).

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed
with CUDA events (max over ranks):
  * `value`: inputs already on the device, loss read once at the end;
  * `e2e`: every step copies its token ids from pinned host memory and reads the loss
    back to the host.
At N >= 2 the line also carries an `allreduce` block: the fused low-bit all-reduce against
NCCL bf16 / fp32 on 64 MB and 1 GB buckets over all N GPUs, with a bit-exact check against the
golden model (bitscom_b200/bench/allreduce_block.py), measured before the model is built.
`--impl reference` runs the reference's library from baseline/_ref (see
baseline/reference_arm.py) or prints why it cannot.  `--impl torch` runs this repo's model code
with torch.matmul (cuBLAS) and SDPA in place of the tcgen05 GEMM and attention kernels: the
library bar the hand-written kernels are measured against.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


from bitscom_b200.utils.clocks import ClockSampler  # noqa: E402


def run_ours(args):
    import torch
    import torch.distributed as dist

    from bitscom_b200.models.llama import LlamaConfig
    from bitscom_b200.trainer.llama_dp_pp import LlamaTrainer, TrainerConfig, _default_attention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun")
    pp = args.pp if args.pp else (2 if args.gpus >= 2 else 1)
    mcfg = LlamaConfig.llama7b() if args.model == "llama7b" else LlamaConfig.tiny(max_seq=256)
    cuda = args.device == "cuda"
    mcfg.attention = args.attention or (_default_attention() if cuda else "sdpa")
    seq = 2048 if args.model == "llama7b" else 256
    chunks = max(1, min(args.pp_chunks, mcfg.num_layers // pp)) if pp > 1 else 1
    tcfg = TrainerConfig(pp_size=pp, pp_chunks=chunks,
                         micro_batches=args.micro_batches or 4 * pp,
                         micro_batch_size=args.micro_batch_size, seq_length=seq, bitwidth=4,
                         error_feedback=True, dp_sync=args.dp_sync, local_size=args.local_size,
                         defer_wgrad=args.defer_wgrad, device=args.device,
                         sync_max_ctas=args.sync_ctas)
    if args.impl == "torch":
        from bitscom_b200.ops import gemm as G

        G.use_library_gemm(True)
        mcfg.attention = "sdpa"

    # the collective half of the metric, over all N GPUs, before the model takes the memory
    allreduce = None
    if world > 1 and cuda and args.impl == "ours" and not args.no_allreduce_block:
        try:
            allreduce = allreduce_block(args)
        except Exception as exc:  # the training half of the line is still worth reporting
            allreduce = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}
            import torch.distributed as _dist

            if _dist.is_initialized():
                _dist.barrier()

    trainer = LlamaTrainer(mcfg, tcfg)
    rank, dev = trainer.rank, trainer.device

    from bitscom_b200.ops import _native
    from bitscom_b200.utils import timing

    def barrier():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(steps, e2e: bool, first_step: int):
        host_batches = [trainer.synthetic_batch(first_step + i) for i in range(steps)]
        dev_batches = None if e2e else [b.to(dev) for b in host_batches]
        last = None
        barrier()
        if cuda:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        t0 = time.perf_counter()
        for i in range(steps):
            loss = trainer.train_step(host_batches[i] if e2e else dev_batches[i])
            if loss is not None:
                last = float(loss.item()) if e2e else loss
        if cuda:
            end.record()
        barrier()
        # --device cpu (contract tests without a GPU) has only the host clock
        ms = torch.tensor([start.elapsed_time(end) if cuda else (time.perf_counter() - t0) * 1e3],
                          device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if last is not None and not isinstance(last, float):
            last = float(last.item())
        if world > 1:  # the loss lives on the last pipeline stage; rank 0 reports it
            box = torch.tensor([last if (last is not None and trainer.dp_rank == 0) else 0.0],
                               device=dev)
            dist.all_reduce(box)
            last = float(box.item())
        return float(ms.item()), last

    for i in range(args.warmup):
        trainer.train_step(trainer.synthetic_batch(i))
    barrier()
    timing.reset_counters()
    sampler = ClockSampler(trainer.local)
    if rank == 0:
        sampler.start()
    launches_before = _native.launch_count()
    ms_dev, loss_dev = timed(args.steps, False, args.warmup)
    # kernels of this library launched by THIS rank inside the device-timed region, counted
    # where the native launch functions are called (ops/_native.py)
    launches = _native.launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else None
    # where the device-timed steps went, per rank, then the slowest rank's figure of each phase
    breakdown = trainer.step_breakdown(last=args.steps) if cuda else None
    if breakdown is not None and world > 1:
        box = torch.tensor([breakdown[k] for k in sorted(breakdown)], device=dev)
        dist.all_reduce(box, op=dist.ReduceOp.MAX)
        breakdown = {k: float(v) for k, v in zip(sorted(breakdown), box.tolist())}
    ms_e2e, loss_e2e = timed(args.steps, True, args.warmup + args.steps)
    trainer.check_kernels()  # a kernel that gave up on a bounded wait must not yield a number

    tokens = trainer.tokens_per_step()
    value = tokens * args.steps / (ms_dev / 1e3)
    e2e_value = tokens * args.steps / (ms_e2e / 1e3)
    c = trainer.cfg
    # whole-job bytes per step: every rank copies its replica's token ids from pinned host
    # memory (first stage: inputs, last stage: targets); every last-stage rank reads its loss
    h2d = c.micro_batches * c.micro_batch_size * c.seq_length * 8 * max(world, 1)
    d2h = 4 * trainer.dp
    out = {
        "metric": "llama7b_dp_pp_train_tokens_per_s" if args.model == "llama7b"
        else "tiny_llama_train_tokens_per_s",
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,  # the reference publishes no tokens/s figure
        "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
        "impl": "bitscom_b200" if args.impl == "ours"
        else "torch (this repo's model code on torch.matmul / cuBLAS and SDPA)",
        "device": args.device,
        "config": {"model": "llama-7b (32L, 4096h, 32 heads, ffn 11008, vocab 32000)"
                   if args.model == "llama7b" else "tiny",
                   "global_batch": trainer.dp * c.micro_batches * c.micro_batch_size,
                   "seq_len": c.seq_length, "parallelism": f"dp{trainer.dp}xpp{trainer.pp}",
                   "micro_batches": c.micro_batches, "pp_chunks": trainer.chunks,
                   "schedule": ("interleaved 1F1B" if trainer.chunks > 1 else "1F1B")
                   + (" + deferred weight gradients" if c.defer_wgrad else ""),
                   "grad_sync": trainer.grad_sync_description(),
                   "attention": mcfg.attention, "optimizer": "AdamW fp32 master",
                   "l2": ("per-step working set (>100 GB weights+activations) exceeds the "
                          "126 MB L2; no flush needed") if args.model == "llama7b"
                   else "tiny model: a functional check, not a measurement"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "loss": loss_e2e},
        "gpu_launches": launches,
        "gpu_launches_note": "own kernels launched by rank 0 in the device-timed region",
        "clocks": clocks,
        "loss": loss_dev,
    }
    if breakdown is not None:
        out["step_breakdown_ms"] = dict(breakdown, note="max over ranks of each phase, device "
                                        "time on the compute stream; exposed_grad_sync = wait "
                                        "for gradient buckets after backward had ended")
    if allreduce is not None:
        out["allreduce"] = allreduce
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        import bitscom_b200

        bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
        dist.destroy_process_group()


def allreduce_block(args) -> dict:
    """Fused low-bit all-reduce vs NCCL bf16 / fp32 over all ranks of the job (see
    bitscom_b200/bench/allreduce_block.py); returns the record on every rank."""
    import torch
    import torch.distributed as dist

    from bitscom_b200.bench import allreduce_block as AB
    from bitscom_b200.parallel.fused import FusedLowBitComm
    from bitscom_b200.trainer.llama_dp_pp import _init_distributed

    rank, world, local = _init_distributed("cuda")
    # The block's own communicator sends the all-gather half through NVLink multicast stores
    # when the fabric offers them (validated bit-exact at 2 and 8 GPUs, 5-7 % faster between
    # 32 and 256 MB); it falls back to peer stores on every rank alike when one rank cannot
    # map the multicast object.  The trainer's gradient sync below keeps plain peer stores.
    nvls = "BITSCOM_NVLS" not in os.environ and not args.no_nvls_block
    if nvls:
        os.environ["BITSCOM_NVLS"] = "1"
    try:
        comm = FusedLowBitComm.for_group(dist.group.WORLD, torch.device("cuda", local))
    finally:
        if nvls:
            del os.environ["BITSCOM_NVLS"]
    exact = AB.bit_exact_check(comm, world, rank)
    # the same check on an aligned bucket, which takes the small-bucket form of the kernel
    exact_small = AB.bit_exact_check(comm, world, rank, n=1 << 18)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    rows = AB.measure(comm, sizes_mb=args.allreduce_mb, iters=10, warmup=3)
    clocks = sampler.stop() if rank == 0 else None
    comm_multicast = getattr(comm, "multicast", False)
    comm.close()  # collective: the symmetric blocks go before the model is built
    torch.cuda.empty_cache()
    return {"setting": "4-bit, block 256, stochastic rounding, error feedback + stage 2",
            "world": world, "bit_exact_vs_golden_model": exact,
            "bit_exact_small_bucket_form": exact_small, "multicast": bool(comm_multicast),
            "rows": rows, "clocks": clocks,
            "timing": "CUDA events, 10 calls after 3 warm-ups on rotating buffers (> L2 in "
                      "total), max over ranks"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="llama7b", choices=["llama7b", "tiny"])
    ap.add_argument("--pp", type=int, default=0)
    ap.add_argument("--pp-chunks", type=int, default=4,
                    help="model chunks per pipeline rank (2 or more: interleaved 1F1B; measured "
                         "on 2 GPUs: 40.1k / 41.3k / 41.9k tokens/s with 1 / 2 / 4 chunks)")
    ap.add_argument("--micro-batches", type=int, default=0)
    ap.add_argument("--micro-batch-size", type=int, default=2, help="sequences per micro-batch")
    ap.add_argument("--attention", default=None, choices=[None, "tcgen05", "sdpa"])
    ap.add_argument("--dp-sync", default="pipeline_a", choices=["pipeline_a", "flat", "dense"])
    ap.add_argument("--local-size", type=int, default=1)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="'cpu' (with --model tiny) runs the same program on CPU ranks: a check "
                         "of this script's output contract, not a benchmark")
    ap.add_argument("--allreduce-mb", type=float, nargs="+", default=[64, 1024],
                    help="bucket sizes (MB) of the all-reduce block reported at N >= 2")
    ap.add_argument("--no-allreduce-block", action="store_true")
    ap.add_argument("--no-nvls-block", action="store_true",
                    help="keep the all-reduce block on plain peer stores")
    ap.add_argument("--sync-ctas", type=int, default=148,
                    help="grid cap of gradient buckets launched while backward is still "
                         "running (0 = no cap)")
    ap.add_argument("--defer-wgrad", action="store_true", default=True,
                    help="pipeline stages send the input gradient before running the "
                         "weight-gradient GEMMs (the default; measured faster at dp2 x pp2)")
    ap.add_argument("--no-defer-wgrad", dest="defer_wgrad", action="store_false")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
