"""All-reduce timing of the UNMODIFIED reference library (``baseline/_ref/bitscom``) with
CUDA events, max over ranks, on the same sizes as ``bitscom_b200.bench.allreduce_sweep``.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        baseline/reference_collective.py --bits 4 --min-mb 1 --max-mb 256

``--path python`` (default) times ``bitscom.LowBitGroup(...).all_reduce`` over an NCCL
process group: the reference's Python pipeline with its own CUDA quantize kernels, two
``all_to_all`` and two ``all_gather`` per call — the path every trainer in the reference's
tree uses (``python/bitscom/api.py:703-875``); it has stochastic rounding but no error
feedback.

``--path backend`` would time ``dist.all_reduce`` on the reference's C++ ``lowbit`` backend
(``benchmarks/collective_compare.py:117-119``).  On this machine (torch 2.11) that backend
dies with SIGSEGV inside its constructor, right after its creation banner, before any
collective runs; it is therefore not run and the script reports it as unavailable.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--min-mb", type=float, default=1)
    ap.add_argument("--max-mb", type=float, default=256)
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "bf16"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--path", default="python", choices=["python", "backend"])
    ap.add_argument("--out", default="bench_outputs/reference_allreduce.jsonl")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if args.path == "backend":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "reference C++ lowbit backend crashes with SIGSEGV in its "
                              "constructor under torch 2.11; not run again"}))
        return
    try:
        import bitscom

        assert os.path.realpath(bitscom.__file__).startswith(os.path.realpath(HERE))
        dist.init_process_group(backend="nccl", init_method="env://",
                                device_id=torch.device("cuda", local))
        group = bitscom.LowBitGroup(bitwidth=args.bits, process_group=dist.group.WORLD,
                                    stochastic_rounding=True, block_size=256)
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}))
        return
    world = dist.get_world_size()
    rows = []
    size = int(args.min_mb * (1 << 20))
    while size <= int(args.max_mb * (1 << 20)):
        for dname in args.dtypes:
            dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dname]
            n = size // (4 if dtype == torch.float32 else 2)
            copies = max(2, min(8, -(-(252 << 20) // size)))
            bufs = [(torch.randn(n, device="cuda") * 1e-3).to(dtype) for _ in range(copies)]
            try:
                for i in range(args.warmup * copies):
                    group.all_reduce(bufs[i % copies])
                torch.cuda.synchronize()
                dist.barrier()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for i in range(args.iters):
                    group.all_reduce(bufs[i % copies])
                e.record()
                torch.cuda.synchronize()
                ms = torch.tensor([s.elapsed_time(e) / args.iters], device="cuda")
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                row = {"impl": "reference", "bytes": size, "dtype": dname, "numel": n,
                       "world": world, "bits": args.bits, "lowbit_ms": float(ms.item()),
                       "lowbit_fp32eq_gbs": n * 4 / float(ms.item()) / 1e6,
                       "note": "LowBitGroup Python pipeline over NCCL, stochastic rounding, no EF"}
            except Exception as exc:
                row = {"impl": "reference", "bytes": size, "dtype": dname, "bits": args.bits,
                       "world": world, "error": f"{type(exc).__name__}: {str(exc)[:160]}"}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            del bufs
            torch.cuda.empty_cache()
        size *= 2
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
