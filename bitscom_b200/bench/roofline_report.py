"""Turn the JSON lines printed by ``bench.kernel_profile`` and ``bench.allreduce_sweep`` into
one roofline table (markdown): achieved rate, the peak it is measured against and the
fraction, per kernel and workload.

    python -m bitscom_b200.bench.kernel_profile gemm --m 8192 --n 8192 --k 8192 >> runs.jsonl
    python -m bitscom_b200.bench.kernel_profile attention >> runs.jsonl
    python -m bitscom_b200.bench.roofline_report runs.jsonl

The peaks are the measured ones when the peak file is present (a STREAM-style copy for
bandwidth, a cuBLAS bf16 GEMM for the tensor rate), else the fallback figures the profile
programs use; the column says which.  A fraction a little above 1.0 is possible (the
denominators are themselves kernels); far above it means the timed kernel did not do the
work.  The reference has no such report: its benchmarks print milliseconds only
(``benchmarks/collective_compare.py:117-119``).
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, Iterable, List


def _rows_of(rec: Dict) -> List[Dict]:
    tag = rec.get("peaks", "")
    case = rec.get("case", rec.get("workload", "?"))
    out = []
    if case in ("elementwise", "norms_raw"):
        for k in rec.get("kernels", []):
            out.append({"kernel": k["name"], "workload": f"{rec.get('tokens')} tokens",
                        "time_ms": k["ms"], "achieved": f"{k['gbs']:.0f} GB/s",
                        "fraction": k["frac_hbm"], "of": f"HBM copy, {tag}"})
    elif case.startswith("gemm"):
        name = case + (f" ({rec['variant']})" if rec.get("variant") else "")
        out.append({"kernel": name, "workload": " x ".join(str(rec.get(d)) for d in "MNK"),
                    "time_ms": rec.get("ms"), "achieved": f"{rec.get('tflops', 0):.0f} TFLOP/s",
                    "fraction": rec.get("frac_bf16_peak"), "of": f"cuBLAS bf16, {tag}"})
    elif case.startswith("attention"):
        shape = f"B{rec.get('batch')} S{rec.get('seq')} H{rec.get('heads')} D{rec.get('head_dim')}"
        variant = {"fwd": rec.get("fwd_variant", "simple"), "bwd": "dQ " + rec.get("bwd_dq", "atomic")}
        for d in ("fwd", "bwd"):
            out.append({"kernel": f"{case} {d} ({variant[d]})",
                        "workload": shape, "time_ms": rec.get(d + "_ms"),
                        "achieved": f"{rec.get(d + '_tflops', 0):.0f} TFLOP/s",
                        "fraction": rec.get(d + "_frac_bf16_peak"), "of": f"cuBLAS bf16, {tag}"})
    elif case == "codec":
        for d in ("quantize", "dequantize"):
            out.append({"kernel": f"codec {d}", "workload": f"{rec.get('elems')} x {rec.get('dtype')}"
                        f" {rec.get('bits')}-bit", "time_ms": rec.get(d + "_ms"),
                        "achieved": f"{rec.get(d + '_gbs', 0):.0f} GB/s",
                        "fraction": rec.get(d + "_frac_hbm"), "of": f"HBM copy, {tag}"})
    elif case.startswith("fused"):
        setting = (f", {rec['rounding']}" if rec.get("rounding") else "") + (
            ", EF" if rec.get("ef") else ", no EF")
        out.append({"kernel": case, "workload": f"W{rec.get('world')} x {rec.get('elems')} "
                    f"{rec.get('dtype')} {rec.get('bits')}-bit{setting}", "time_ms": rec.get("ms"),
                    "achieved": f"{rec.get('gbs', 0):.0f} GB/s", "fraction": rec.get("frac_hbm"),
                    "of": f"HBM copy, {tag}"})
    elif "roofline_frac" in rec:  # allreduce_sweep rows
        size = rec.get("bytes", 0) / (1 << 20)
        out.append({"kernel": f"low-bit all-reduce {rec.get('bits')}-bit",
                    "workload": f"{rec.get('world')} GPUs, {size:g} MB "
                    f"{rec.get('bucket_dtype', rec.get('dtype'))}",
                    "time_ms": rec.get("lowbit_ms"),
                    "achieved": f"{rec.get('lowbit_effective_gbs', rec.get('lowbit_fp32eq_gbs', 0)):.0f}"
                    " GB/s fp32-equivalent",
                    "fraction": rec.get("roofline_frac"),
                    "of": f"max(HBM, NVLink) bound, {rec.get('peaks', tag)}"})
    return out


def collect(lines: Iterable[str]) -> List[Dict]:
    rows: List[Dict] = []
    for line in lines:
        line = line.strip()
        if not line.startswith("{"):
            continue
        try:
            rows += _rows_of(json.loads(line))
        except (ValueError, KeyError, TypeError):
            continue  # not one of ours
    return rows


def to_markdown(rows: List[Dict]) -> str:
    out = ["| kernel | workload | time | achieved | fraction | of |", "|---|---|---|---|---|---|"]
    for r in rows:
        t = "—" if r["time_ms"] is None else f"{r['time_ms']:.3f} ms"
        f = "—" if r["fraction"] is None else f"{r['fraction']:.2f}"
        out.append(f"| {r['kernel']} | {r['workload']} | {t} | {r['achieved']} | {f} | {r['of']} |")
    return "\n".join(out)


def main(argv=None) -> str:
    ap = argparse.ArgumentParser(description="roofline table from profile JSON lines")
    ap.add_argument("files", nargs="*", help="JSONL files (default: standard input)")
    args = ap.parse_args(argv)
    lines: List[str] = []
    if args.files:
        for path in args.files:
            with open(path, encoding="utf-8") as f:
                lines += f.readlines()
    else:
        lines = sys.stdin.readlines()
    table = to_markdown(collect(lines))
    print(table)
    return table


if __name__ == "__main__":
    main()
