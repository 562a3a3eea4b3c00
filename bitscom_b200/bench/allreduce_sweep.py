"""Low-bit all-reduce sweep against NCCL (one process per GPU, launch with torchrun).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m bitscom_b200.bench.allreduce_sweep --min-mb 1 --max-mb 1024 --bits 1 2 4 8

For every size (bytes of the gradient buffer, powers of two), dtype and bitwidth it times

  * the fused low-bit all-reduce (block 256, stochastic rounding, error feedback and
    stage-2 error feedback on, like the reference's heaviest setting),
  * NCCL all-reduce of the same buffer in fp32 and in bf16,

with CUDA events on the launching stream, after warm-up, rotating over enough distinct
buffers that consecutive iterations never find their input in L2, and reports the MAX
over ranks.  "effective GB/s" is the fp32-equivalent payload (4 bytes per element)
divided by the time, the figure the reference's collective benchmark would quote
(``benchmarks/collective_compare.py:41-46,117-119`` times the same call on the host).
The roofline column is time >= max(HBM bytes / measured copy bandwidth,
wire bytes / NVLink bandwidth).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

L2_BYTES = 126 << 20


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    hbm, src = 6650.0, "fallback"
    if os.path.exists(path):
        with open(path) as f:
            hbm, src = float(json.load(f).get("hbm_gbs", hbm)), "measured"
    return hbm, 770.0, src


def _time_ms(fn, bufs, iters, warmup):
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
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-mb", type=float, default=1)
    ap.add_argument("--max-mb", type=float, default=256)
    ap.add_argument("--bits", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "bf16"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-ef", action="store_true")
    ap.add_argument("--nearest", action="store_true")
    ap.add_argument("--out", default="bench_outputs/allreduce_sweep.jsonl")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()

    from bitscom_b200.api import ErrorFeedbackState, ShardPlan
    from bitscom_b200.parallel.fused import FusedLowBitComm

    comm = FusedLowBitComm.for_group(dist.group.WORLD, torch.device("cuda", local))
    hbm_gbs, link_gbs, peak_src = _peaks()
    rows = []
    size = int(args.min_mb * (1 << 20))
    while size <= int(args.max_mb * (1 << 20)):
        for dname in args.dtypes:
            dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dname]
            esize = 4 if dtype == torch.float32 else 2
            n = size // esize
            copies = max(2, min(64, -(-2 * L2_BYTES // size)))
            bufs = [torch.randn(n, device="cuda", dtype=torch.float32).mul_(1e-3).to(dtype)
                    for _ in range(copies)]
            nccl_ms = _time_ms(lambda t: dist.all_reduce(t), bufs, args.iters, args.warmup)
            base = {"bytes": size, "dtype": dname, "numel": n, "world": world,
                    "nccl_ms": nccl_ms, "nccl_algbw_gbs": size / nccl_ms / 1e6,
                    "nccl_fp32eq_gbs": n * 4 / nccl_ms / 1e6}
            for bits in args.bits:
                efs = [None if args.no_ef else ErrorFeedbackState() for _ in bufs]
                for e in efs:  # residuals exist before anything is timed
                    if e is not None:
                        e.ensure(ShardPlan(world, n), bufs[0].device, True)
                index = {b.data_ptr(): e for b, e in zip(bufs, efs)}

                def run(t, bits=bits, index=index):
                    comm.all_reduce(t, bitwidth=bits, block_size=256,
                                    stochastic=not args.nearest, seed=1,
                                    ef=index[t.data_ptr()], stage2=not args.no_ef)

                ms = _time_ms(run, bufs, args.iters, args.warmup)
                comm.check_status()
                S = -(-n // world)
                per_elem_packed = bits / 8 + 2 / 256
                wire = (world - 1) * S * per_elem_packed  # per direction, per phase
                ef_b = 0 if args.no_ef else 8
                hbm = (n * (esize + ef_b + per_elem_packed)               # phase 1
                       + world * S * per_elem_packed * 2 + S * ef_b       # phase 2
                       + n * (per_elem_packed + esize))                   # phase 3
                floor_ms = max(hbm / (hbm_gbs * 1e6), 2 * wire / (link_gbs * 1e6))
                rows.append(dict(base, bits=bits, lowbit_ms=ms,
                                 lowbit_fp32eq_gbs=n * 4 / ms / 1e6,
                                 speedup_vs_nccl=nccl_ms / ms,
                                 roofline_ms=floor_ms, roofline_frac=floor_ms / ms,
                                 peaks=peak_src))
                if rank == 0:
                    print(json.dumps(rows[-1]), flush=True)
            del bufs
            torch.cuda.empty_cache()
        size *= 2
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    import bitscom_b200

    bitscom_b200.shutdown()  # release symmetric blocks in order, before the group goes
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
