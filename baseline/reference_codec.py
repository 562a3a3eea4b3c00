"""Codec kernels of the UNMODIFIED reference library (``baseline/_ref/bitscom`` with its own
``_lowbit_cuda`` extension) timed next to this library's, same tensors, same method (CUDA
events around back-to-back calls after warm-up, inputs larger than L2):

    python baseline/reference_codec.py --elems 67108864

Rows: blockwise quantize + pack and unpack + dequantize (4-bit, block 256; the reference's
fused CUDA path, ``python/bitscom/quantization.py:153-192,238-287`` over
``cpp/src/lowbit_cuda_kernels.cu:144-250``), per-tensor quantize (``:65-100``, device kernels
``.cu:29-81``) and pack / unpack of int16 codes (``:311-391``, ``.cu:83-133``).  Both sides
are called through their public Python functions, so both pay their own allocation of the
outputs.  If the reference cannot be imported one ``unavailable`` line is printed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _timed(fn, iters: int, warmup: int) -> float:
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", type=int, default=1 << 26)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--block", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()

    import torch

    sys.path.insert(0, ROOT)
    from bitscom_b200 import quantization as ours

    sys.path.insert(0, os.path.join(HERE, "_ref"))
    try:
        import bitscom.quantization as ref

        assert os.path.realpath(ref.__file__).startswith(os.path.realpath(HERE))
        if not getattr(ref, "_HAS_CUDA_KERNELS", False):
            raise RuntimeError("the reference's _lowbit_cuda extension did not load")
    except BaseException as exc:
        print(json.dumps({"impl": "reference", "unavailable":
                          f"{type(exc).__name__}: {str(exc)[:200]}"}))
        return

    n, bits, block = args.elems, args.bits, args.block
    x = torch.randn(n, device="cuda") * 1e-3
    rows = []

    def row(name, t_ref, t_ours, nbytes):
        rows.append({"kernel": name, "elems": n, "bits": bits, "reference_ms": t_ref,
                     "this_repo_ms": t_ours, "speedup": t_ref / t_ours,
                     "this_repo_gbs": nbytes / t_ours / 1e6})

    # blockwise quantize + pack / unpack + dequantize
    rp, rs, _ = ref.quantize_pack_tensor_blockwise(x, bits, block_size=block)
    op, os_, _ = ours.quantize_pack_tensor_blockwise(x, bits, block_size=block)
    same_codes = bool(torch.equal(rp.view(torch.uint8).reshape(-1), op.view(torch.uint8).reshape(-1)))
    packed_bytes = n * bits // 8 + 2 * (n // block)
    row("blockwise quantize + pack",
        _timed(lambda: ref.quantize_pack_tensor_blockwise(x, bits, block_size=block),
               args.iters, args.warmup),
        _timed(lambda: ours.quantize_pack_tensor_blockwise(x, bits, block_size=block),
               args.iters, args.warmup), 4 * n + packed_bytes)
    rows[-1]["same_packed_bytes"] = same_codes
    row("blockwise unpack + dequantize",
        _timed(lambda: ref.unpack_dequantize_tensor_blockwise(rp, rs, bits, n, block_size=block),
               args.iters, args.warmup),
        _timed(lambda: ours.unpack_dequantize_tensor_blockwise(op, os_, bits, n,
                                                               block_size=block),
               args.iters, args.warmup), 4 * n + packed_bytes)
    # per-tensor quantize (int16 codes + scale)
    row("per-tensor quantize",
        _timed(lambda: ref.quantize_tensor(x, bits), args.iters, args.warmup),
        _timed(lambda: ours.quantize_tensor(x, bits), args.iters, args.warmup), 6 * n)
    rq, _ = ref.quantize_tensor(x, bits)[:2]
    oq, _ = ours.quantize_tensor(x, bits)[:2]
    row("pack int16 codes",
        _timed(lambda: ref.pack_lowbit(rq, bits), args.iters, args.warmup),
        _timed(lambda: ours.pack_lowbit(oq, bits), args.iters, args.warmup),
        2 * n + n * bits // 8)
    rpk, _ = ref.pack_lowbit(rq, bits)
    opk, _ = ours.pack_lowbit(oq, bits)
    row("unpack int16 codes",
        _timed(lambda: ref.unpack_lowbit(rpk, bits, n), args.iters, args.warmup),
        _timed(lambda: ours.unpack_lowbit(opk, bits, n), args.iters, args.warmup),
        2 * n + n * bits // 8)
    for r in rows:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
