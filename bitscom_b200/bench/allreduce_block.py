"""The all-reduce half of the headline metric, as one record: the fused low-bit all-reduce
against NCCL bf16 and NCCL fp32 on the same buckets, plus a bit-exact check against the golden
model (``parallel/simulate.py``) in the same process.

Setting (the reference's heaviest, ``benchmarks/collective_compare.py:117-119`` is its timing
loop): 4-bit codes, block 256, stochastic rounding, error feedback and second-stage error
feedback on.  Buckets of 64 MB and 1 GB, as fp32 and as bf16 gradients.  Times are CUDA
events on the launching stream after warm-up, rotating over distinct buffers larger than L2
in total, MAX over ranks.  "effective GB/s" counts the fp32-equivalent payload (4 bytes per
element).  Roofline: time >= max(HBM bytes / measured copy bandwidth, bytes that cross
NVLink per direction / 770 GB/s).

Used by ``bench.py`` (N >= 2) and by ``bench/allreduce_sweep.py``.
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch
import torch.distributed as dist

L2_BYTES = 126 << 20
LINK_GBS = 770.0  # measured peer copy, per direction


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    hbm, src = 6650.0, "of fallback"
    if os.path.exists(path):
        with open(path) as f:
            hbm, src = float(json.load(f).get("hbm_gbs", hbm)), "of measured"
    return hbm, LINK_GBS, src


def time_ms(fn, bufs, iters: int, warmup: int, group=None) -> float:
    """Mean time per call over ``iters`` back-to-back calls on rotating buffers; device-timed,
    MAX over the ranks of ``group``."""
    for i in range(max(warmup, 3)):
        fn(bufs[i % len(bufs)])
    torch.cuda.synchronize()
    dist.barrier(group=group)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(bufs[i % len(bufs)])
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def roofline_ms(n: int, esize: int, bits: int, world: int, ef: bool, hbm_gbs: float,
                link_gbs: float) -> float:
    S = -(-n // world)
    packed = bits / 8 + 2 / 256
    wire = (world - 1) * S * packed                      # per direction, per phase
    ef_b = 8 if ef else 0
    hbm = (n * (esize + ef_b + packed)                   # phase 1
           + world * S * packed * 2 + S * ef_b           # phase 2
           + n * (packed + esize))                       # phase 3
    return max(hbm / (hbm_gbs * 1e6), 2 * wire / (link_gbs * 1e6))


def bit_exact_check(comm, world: int, rank: int, n: int = 100003, bits: int = 4,
                    iters: int = 2) -> bool:
    """A small bucket through the fused kernel (stochastic rounding with a fixed seed, both
    error-feedback stages, ``iters`` calls so that residuals are used) against the golden
    model, bit for bit; True only if every rank agrees."""
    from ..api import ErrorFeedbackState
    from ..parallel.simulate import SimState, simulate_all_reduce

    def inp(r, it):
        g = torch.Generator().manual_seed(4242 + r + 1000 * it)
        return torch.randn(n, generator=g) * 1e-3

    state, ef, ok = SimState(), ErrorFeedbackState(), True
    threads = torch.get_num_threads()
    torch.set_num_threads(1)  # every rank replays the model: do not oversubscribe the host
    try:
        for it in range(iters):
            everyone = [inp(r, it) for r in range(world)]
            want = simulate_all_reduce(everyone, bits, 256, stochastic=True, seed=77 + it,
                                       state=state, stage2=True)[rank]
            x = everyone[rank].cuda()
            comm.all_reduce(x, bitwidth=bits, block_size=256, stochastic=True, seed=77 + it,
                            ef=ef, stage2=True)
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(x.cpu(), want))
    finally:
        torch.set_num_threads(threads)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=comm.group)
    return bool(flag.item())


def measure(comm, sizes_mb: Sequence[float] = (64, 1024), dtypes: Sequence[str] = ("fp32", "bf16"),
            bits: int = 4, iters: int = 10, warmup: int = 3, ef: bool = True,
            stochastic: bool = True) -> List[Dict]:
    """One row per (bucket bytes, bucket dtype); see the module docstring."""
    from ..api import ErrorFeedbackState, ShardPlan

    group = comm.group
    world = dist.get_world_size(group)
    hbm_gbs, link_gbs, tag = peaks()
    rows = []
    for mb in sizes_mb:
        size = int(mb * (1 << 20))
        for dname in dtypes:
            dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dname]
            esize = 4 if dtype == torch.float32 else 2
            n = size // esize
            copies = max(2, min(64, -(-2 * L2_BYTES // size)))
            bufs = [torch.randn(n, device="cuda", dtype=torch.float32).mul_(1e-3).to(dtype)
                    for _ in range(copies)]
            nccl_same = time_ms(lambda t: dist.all_reduce(t, group=group), bufs, iters, warmup,
                                group)
            # the other NCCL arm on the same ELEMENT count
            other = torch.bfloat16 if dtype == torch.float32 else torch.float32
            obufs = [torch.zeros(n, device="cuda", dtype=other) for _ in range(copies)]
            nccl_other = time_ms(lambda t: dist.all_reduce(t, group=group), obufs, iters, warmup,
                                 group)
            del obufs
            nccl_bf16 = nccl_other if dtype == torch.float32 else nccl_same
            nccl_fp32 = nccl_same if dtype == torch.float32 else nccl_other
            efs = [ErrorFeedbackState() if ef else None for _ in bufs]
            for e in efs:  # residuals exist before anything is timed
                if e is not None:
                    e.ensure(ShardPlan(world, n), bufs[0].device, True)
            index = {b.data_ptr(): e for b, e in zip(bufs, efs)}

            def run(t, index=index):
                comm.all_reduce(t, bitwidth=bits, block_size=256, stochastic=stochastic, seed=1,
                                ef=index[t.data_ptr()], stage2=ef)

            ms = time_ms(run, bufs, iters, warmup, group)
            comm.check_status()
            phases = comm.phase_times_us() if hasattr(comm, "phase_times_us") else None
            floor = roofline_ms(n, esize, bits, world, ef, hbm_gbs, link_gbs)
            rows.append({
                "bytes": size, "bucket_dtype": dname, "numel": n, "world": world, "bits": bits,
                "stochastic_rounding": stochastic, "error_feedback": ef, "stage2": ef,
                "lowbit_ms": ms, "nccl_bf16_ms": nccl_bf16, "nccl_fp32_ms": nccl_fp32,
                "lowbit_effective_gbs": n * 4 / ms / 1e6,
                "nccl_bf16_effective_gbs": n * 4 / nccl_bf16 / 1e6,
                "nccl_fp32_effective_gbs": n * 4 / nccl_fp32 / 1e6,
                "vs_nccl_bf16": nccl_bf16 / ms, "vs_nccl_fp32": nccl_fp32 / ms,
                "roofline_ms": floor, "roofline_frac": floor / ms, "peaks": tag,
                # this rank's last launch, from time stamps its first CTA took on the device
                "phases_us_rank0": phases})
            del bufs, efs, index
            torch.cuda.empty_cache()
    return rows
