"""Low-bit all-reduce sweep against NCCL (one process per GPU, launch with torchrun).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m bitscom_b200.bench.allreduce_sweep --min-mb 1 --max-mb 1024 --bits 1 2 4 8

For every size (bytes of the gradient buffer, powers of two), dtype and bitwidth it times

  * the fused low-bit all-reduce (block 256, stochastic rounding, error feedback and
    stage-2 error feedback on, like the reference's heaviest setting),
  * NCCL all-reduce of the same buffer in fp32 and in bf16,

with CUDA events on the launching stream, after warm-up, rotating over enough distinct
buffers that consecutive iterations never find their input in L2, and reports the MAX
over ranks; every row carries the SM clocks and throttle reasons sampled while it was timed
(the measurement itself lives in ``bench/allreduce_block.py``).  "effective GB/s" is the fp32-equivalent payload (4 bytes per element)
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

from ..utils.clocks import ClockSampler
from . import allreduce_block as AB


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

    from bitscom_b200.parallel.fused import FusedLowBitComm

    comm = FusedLowBitComm.for_group(dist.group.WORLD, torch.device("cuda", local))
    rows = []
    size = args.min_mb
    while size <= args.max_mb:
        for bits in args.bits:
            # every row carries the SM clocks and throttle reasons seen while it was timed
            sampler = ClockSampler(local, period_ms=100)
            if rank == 0:
                sampler.start()
            got = AB.measure(comm, sizes_mb=[size], dtypes=args.dtypes, bits=bits,
                             iters=args.iters, warmup=args.warmup, ef=not args.no_ef,
                             stochastic=not args.nearest)
            clocks = sampler.stop() if rank == 0 else None
            for r in got:
                r["clocks"] = clocks
                r["multicast"] = bool(comm.multicast)
                rows.append(r)
                if rank == 0:
                    print(json.dumps(r), flush=True)
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
