"""Error-feedback benefit: relative error of the accumulated (quantized) gradient with and
without error feedback, single process, no communication.

Same experiment as the reference's ``benchmarks/error_feedback_comparison.py:40-70``
(``run_ef_benefit_curve``): each step draws g ~ N(0, 0.05^2), quantizes it per tensor
(``--blockwise`` switches to the blockwise quantizer the collectives use), accumulates the
dequantized value with and without carrying the residual, and reports
``||sum q(g) - sum g|| / ||sum g||``.  The reference publishes the value after 160 steps
(``benchmarks/outputs/ef_benefit_curve_bw{2,4,8}.csv:161``: 0.9739 -> 0.1808 at 2-bit,
0.2016 -> 0.0158 at 4-bit, 0.0111 -> 0.00081 at 8-bit).

    python -m bitscom_b200.bench.error_feedback_benefit --bits 2 4 8 --steps 160
"""

from __future__ import annotations

import argparse
import csv
import json
import os
from typing import List, Tuple

import torch

from ..quantization import (dequantize_tensor, dequantize_tensor_blockwise, quantize_tensor,
                            quantize_tensor_blockwise)


def _roundtrip(x: torch.Tensor, bits: int, blockwise: bool) -> torch.Tensor:
    if blockwise:
        q, s = quantize_tensor_blockwise(x, bits)
        return dequantize_tensor_blockwise(q, s, device=x.device)
    q, scale = quantize_tensor(x, bits)
    return dequantize_tensor(q, scale, dtype=torch.float32, device=x.device)


def ef_benefit_curve(bits: int, steps: int = 160, vec_size: int = 1 << 20, seed: int = 2026,
                     device: str = "cpu", blockwise: bool = False
                     ) -> List[Tuple[int, float, float]]:
    torch.manual_seed(seed)
    true_cum = torch.zeros(vec_size, device=device)
    plain_cum, ef_cum, residual = (torch.zeros_like(true_cum) for _ in range(3))
    rows = []
    for step in range(1, steps + 1):
        g = torch.randn(vec_size, device=device) * 0.05
        true_cum += g
        plain_cum += _roundtrip(g, bits, blockwise)
        corrected = g + residual
        sent = _roundtrip(corrected, bits, blockwise)
        residual = corrected - sent
        ef_cum += sent
        denom = true_cum.norm().item() + 1e-12
        rows.append((step, (plain_cum - true_cum).norm().item() / denom,
                     (ef_cum - true_cum).norm().item() / denom))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--bits", type=int, nargs="+", default=[2, 4, 8])
    ap.add_argument("--steps", type=int, default=160)
    ap.add_argument("--vec-size", type=int, default=1 << 20)
    ap.add_argument("--seed", type=int, default=2026)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--blockwise", action="store_true")
    ap.add_argument("--out-dir", default=None, help="write ef_benefit_curve_bw{b}.csv here")
    args = ap.parse_args(argv)
    for b in args.bits:
        rows = ef_benefit_curve(b, args.steps, args.vec_size, args.seed, args.device,
                                args.blockwise)
        step, no_ef, ef = rows[-1]
        print(json.dumps({"bitwidth": b, "steps": step, "no_ef_rel_error": no_ef,
                          "ef_rel_error": ef, "blockwise": args.blockwise}))
        if args.out_dir:
            os.makedirs(args.out_dir, exist_ok=True)
            with open(os.path.join(args.out_dir, f"ef_benefit_curve_bw{b}.csv"), "w",
                      newline="") as f:
                w = csv.writer(f)
                w.writerow(["step", "no_ef_rel_error", "ef_rel_error"])
                w.writerows(rows)
            from ..utils.plot import save_line_plot

            steps = [r[0] for r in rows]
            save_line_plot(os.path.join(args.out_dir, f"ef_comparison_bw{b}.png"),
                           {"no error feedback": (steps, [r[1] for r in rows]),
                            "error feedback": (steps, [r[2] for r in rows])},
                           title=f"relative cumulative error, {b}-bit", xlabel="step",
                           ylabel="rel err", logy=True)


if __name__ == "__main__":
    main()
