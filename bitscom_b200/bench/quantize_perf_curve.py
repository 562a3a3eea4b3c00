"""Latency of one quantize call against tensor size, host path against device path.

For each power-of-two size it times, after warm-up, the median of

* ``cpu_torch``   the torch-op oracle on a CPU tensor (what the reference calls the
  original path, ``benchmarks/quantize_perf_curve.py:13-24``),
* ``cpu_native``  this package's C++ CPU codec (blockwise mode only),
* ``gpu``         the CUDA kernel path on a device tensor, host-timed with a synchronize on
  both sides because the figure of interest is the latency of the *call*
  (``:27-41`` of the same file), and ``gpu_device_ms`` from CUDA events for the kernel time
  alone,

in ``--mode per_tensor`` (``quantize_tensor``, the reference's curve) or ``--mode
blockwise`` (``quantize_pack_tensor_blockwise``, the call the collectives use).  Without a
GPU only the host columns are filled.  Writes ``quantize_curve_<mode>_bw<b>.csv`` to
``--out-dir`` and prints one JSON line per size.

    python -m bitscom_b200.bench.quantize_perf_curve --bitwidth 4 --max-pow2 23
"""

from __future__ import annotations

import argparse
import csv
import json
import os
import statistics
import time
from typing import Callable, Dict, List, Optional

import torch

from .. import quantization as Q
from ..ops import cpu_codec


def iters_for(n: int) -> int:
    if n <= 1 << 14:
        return 200
    if n <= 1 << 18:
        return 120
    if n <= 1 << 21:
        return 60
    return 30


def median_host_ms(fn: Callable[[], object], warmup: int, iters: int,
                   sync: Optional[Callable[[], None]] = None) -> float:
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iters):
        if sync:
            sync()
        t0 = time.perf_counter()
        fn()
        if sync:
            sync()
        samples.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(samples)


def median_device_ms(fn: Callable[[], object], iters: int) -> float:
    samples = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        samples.append(a.elapsed_time(b))
    return statistics.median(samples)


def torch_oracle_blockwise(x: torch.Tensor, bitwidth: int, block: int):
    q, scales = Q.quantize_tensor_blockwise(x, bitwidth, block_size=block)
    return Q.pack_lowbit(q, bitwidth)[0], scales


def measure(n: int, args, device: Optional[torch.device]) -> Dict[str, float]:
    x_cpu = torch.linspace(-1.0, 1.0, steps=n)
    iters = min(iters_for(n), args.max_iters)
    warmup = min(args.warmup, max(5, iters // 4))
    row: Dict[str, float] = {"numel": n}
    if args.mode == "per_tensor":
        row["cpu_torch_ms"] = median_host_ms(
            lambda: Q.quantize_tensor(x_cpu, args.bitwidth), warmup, iters)
    else:
        row["cpu_torch_ms"] = median_host_ms(
            lambda: torch_oracle_blockwise(x_cpu, args.bitwidth, args.block_size), warmup,
            iters)
        if cpu_codec.available() and args.bitwidth in (1, 2, 4, 8):
            row["cpu_native_ms"] = median_host_ms(
                lambda: cpu_codec.blockwise_quantize_pack(x_cpu, args.bitwidth,
                                                          args.block_size), warmup, iters)
    if device is not None:
        x_gpu = x_cpu.to(device)
        if args.mode == "per_tensor":
            call = lambda: Q.quantize_tensor(x_gpu, args.bitwidth)  # noqa: E731
        else:
            call = lambda: Q.quantize_pack_tensor_blockwise(  # noqa: E731
                x_gpu, args.bitwidth, block_size=args.block_size)
        sync = lambda: torch.cuda.synchronize(device)  # noqa: E731
        row["gpu_ms"] = median_host_ms(call, warmup, iters, sync)
        row["gpu_device_ms"] = median_device_ms(call, iters)
        row["speedup_gpu_vs_cpu"] = row["cpu_torch_ms"] / row["gpu_ms"]
        row["gpu_melems_per_s"] = n / 1e6 / (row["gpu_ms"] / 1e3)
    row["cpu_melems_per_s"] = n / 1e6 / (row["cpu_torch_ms"] / 1e3)
    return row


def main(argv=None) -> List[Dict[str, float]]:
    ap = argparse.ArgumentParser(description="quantize call latency, CPU path vs CUDA path")
    ap.add_argument("--bitwidth", type=int, default=4)
    ap.add_argument("--mode", default="per_tensor", choices=["per_tensor", "blockwise"])
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--min-pow2", type=int, default=10)
    ap.add_argument("--max-pow2", type=int, default=23)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--max-iters", type=int, default=200)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out-dir", default=None)
    args = ap.parse_args(argv)

    device = torch.device(args.device) if args.device.startswith("cuda") else None
    if device is not None and not torch.cuda.is_available():
        raise RuntimeError("a CUDA device was asked for but none is available")
    rows = []
    for k in range(args.min_pow2, args.max_pow2 + 1):
        row = measure(1 << k, args, device)
        rows.append(row)
        print(json.dumps(row))
    if args.out_dir:
        os.makedirs(args.out_dir, exist_ok=True)
        fields = ["numel", "cpu_torch_ms", "cpu_native_ms", "gpu_ms", "gpu_device_ms",
                  "speedup_gpu_vs_cpu", "cpu_melems_per_s", "gpu_melems_per_s"]
        path = os.path.join(args.out_dir, f"quantize_curve_{args.mode}_bw{args.bitwidth}.csv")
        with open(path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=fields, restval="")
            w.writeheader()
            w.writerows(rows)
        print(f"saved {path}")
        from ..utils.plot import save_line_plot

        xs = [r["numel"] for r in rows]
        series = {k: (xs, [r[k] for r in rows]) for k in
                  ("cpu_torch_ms", "cpu_native_ms", "gpu_ms", "gpu_device_ms")
                  if all(isinstance(r.get(k), (int, float)) for r in rows)}
        save_line_plot(path[:-4] + ".png", series,
                       title=f"quantize latency, {args.mode}, {args.bitwidth}-bit",
                       xlabel="elements", ylabel="ms", logx=True, logy=True)
    return rows


if __name__ == "__main__":
    main()
