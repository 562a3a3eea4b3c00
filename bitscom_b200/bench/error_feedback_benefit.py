"""Error-feedback benefit: relative error of the accumulated (quantized) gradient with and
without error feedback, single process, no communication.

Same experiment as the reference's ``benchmarks/error_feedback_comparison.py:40-70``
(``run_ef_benefit_curve``): each step draws g ~ N(0, 0.05^2), quantizes it per tensor
(``--blockwise`` switches to the blockwise quantizer the collectives use), accumulates the
dequantized value with and without carrying the residual, and reports
``||sum q(g) - sum g|| / ||sum g||``.  The reference publishes the value after 160 steps
(``benchmarks/outputs/ef_benefit_curve_bw{2,4,8}.csv:161``: 0.9739 -> 0.1808 at 2-bit,
0.2016 -> 0.0158 at 4-bit, 0.0111 -> 0.00081 at 8-bit).

The second half of that benchmark (``run_training``, ``:97-137``) is here too: a three-layer MLP
(64 -> 128 -> 128 -> 10) trained with plain SGD on batches whose label is the arg-max of a fixed
linear map of the input, every parameter's gradient passed through the quantizer before the
step, with and without a per-parameter residual.  The reference publishes the loss at step 120
(``benchmarks/outputs/ef_training_curve_bw{2,4,8}.csv:121``: 0.004924 / 0.005398 at 2-bit,
0.005385 / 0.005326 at 4-bit, 0.005325 / 0.005325 at 8-bit).

    python -m bitscom_b200.bench.error_feedback_benefit --bits 2 4 8 --steps 160 --train-steps 160
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


def ef_training_curve(bits: int, steps: int = 160, lr: float = 0.05, batch_size: int = 256,
                      seed: int = 2026, use_ef: bool = True, device: str = "cpu",
                      blockwise: bool = False) -> List[float]:
    """Loss per step of the MLP whose gradients go through the quantizer (see the module
    docstring).  Same seed, same data and same initial weights for both settings of ``use_ef``."""
    gen = torch.Generator(device="cpu").manual_seed(seed)

    def draw(*shape, scale=1.0):
        return (torch.randn(*shape, generator=gen) * scale).to(device)

    dims = [(64, 128), (128, 128), (128, 10)]
    params = []
    for fan_in, fan_out in dims:   # the uniform(-1/sqrt(fan_in), +) start of a linear layer
        bound = fan_in ** -0.5
        w = ((torch.rand(fan_out, fan_in, generator=gen) * 2 - 1) * bound).to(device)
        b = ((torch.rand(fan_out, generator=gen) * 2 - 1) * bound).to(device)
        params += [w.requires_grad_(), b.requires_grad_()]
    teacher = torch.linspace(-1.0, 1.0, 64, device=device).unsqueeze(1).repeat(1, 10)
    residuals = [torch.zeros_like(p) for p in params]
    losses: List[float] = []
    for _ in range(steps):
        x = draw(batch_size, 64)
        y = (x @ teacher).argmax(dim=1)
        h = x
        for i in range(0, len(params), 2):
            h = torch.nn.functional.linear(h, params[i], params[i + 1])
            if i + 2 < len(params):
                h = torch.relu(h)
        loss = torch.nn.functional.cross_entropy(h, y)
        grads = torch.autograd.grad(loss, params)
        with torch.no_grad():
            for p, g, r in zip(params, grads, residuals):
                corrected = g + r if use_ef else g
                sent = _roundtrip(corrected.reshape(-1), bits, blockwise).view_as(g)
                if use_ef:
                    r.copy_(corrected - sent)
                p.sub_(lr * sent)
        losses.append(float(loss.detach()))
    return losses


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--bits", type=int, nargs="+", default=[2, 4, 8])
    ap.add_argument("--steps", type=int, default=160)
    ap.add_argument("--vec-size", type=int, default=1 << 20)
    ap.add_argument("--seed", type=int, default=2026)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--blockwise", action="store_true")
    ap.add_argument("--out-dir", default=None,
                    help="write ef_benefit_curve_bw{b}.csv (and ef_training_curve_bw{b}.csv) here")
    ap.add_argument("--train-steps", type=int, default=0,
                    help="also train the small MLP for this many steps with and without error "
                         "feedback (the reference's default is 160)")
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--batch-size", type=int, default=256)
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
        if args.train_steps > 0:
            kw = dict(steps=args.train_steps, lr=args.lr, batch_size=args.batch_size,
                      seed=args.seed, device=args.device, blockwise=args.blockwise)
            plain = ef_training_curve(b, use_ef=False, **kw)
            with_ef = ef_training_curve(b, use_ef=True, **kw)
            at = min(120, args.train_steps) - 1
            print(json.dumps({"bitwidth": b, "train_steps": args.train_steps,
                              "loss_no_ef_first": plain[0], "loss_ef_first": with_ef[0],
                              f"loss_no_ef_step{at + 1}": plain[at],
                              f"loss_ef_step{at + 1}": with_ef[at],
                              "loss_no_ef_last": plain[-1], "loss_ef_last": with_ef[-1]}))
            if args.out_dir:
                with open(os.path.join(args.out_dir, f"ef_training_curve_bw{b}.csv"), "w",
                          newline="") as f:
                    w = csv.writer(f)
                    w.writerow(["step", "loss_noef", "loss_ef"])
                    w.writerows((i + 1, plain[i], with_ef[i]) for i in range(len(plain)))
                from ..utils.plot import save_line_plot

                xs = list(range(1, len(plain) + 1))
                save_line_plot(os.path.join(args.out_dir, f"ef_training_curve_bw{b}.png"),
                               {"no error feedback": (xs, plain), "error feedback": (xs, with_ef)},
                               title=f"training loss, gradients at {b} bit", xlabel="step",
                               ylabel="loss", logy=True)


if __name__ == "__main__":
    main()
