"""Low-bit gradient all-reduce in a dozen lines; runs on CPU ranks (gloo) or GPUs (nccl).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/allreduce_quickstart.py
"""

import os

import torch
import torch.distributed as dist

import bitscom_b200 as bitscom


def main():
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    # 4-bit blockwise quantization with fp16 block scales; once with error feedback on both
    # stages, once without, on the same gradients
    with_ef = bitscom.LowBitGroup(bitwidth=4, block_size=256, error_feedback=True,
                                  stage2_error_feedback=True)
    without = bitscom.LowBitGroup(bitwidth=4, block_size=256)
    exact = torch.zeros(1 << 20, device=device)
    sum_ef, sum_plain = torch.zeros_like(exact), torch.zeros_like(exact)
    for step in range(8):
        g = torch.Generator().manual_seed(100 * step + rank)
        grad = (torch.randn(1 << 20, generator=g) * 1e-3).to(device)
        dense, a, b = grad.clone(), grad.clone(), grad.clone()
        dist.all_reduce(dense)                     # what a dense all-reduce would give
        with_ef.all_reduce(a, ef_key="bucket0")    # in place; the caller divides by world
        without.all_reduce(b)
        exact += dense
        sum_ef += a
        sum_plain += b
    # error feedback carries each step's quantization error into the next step, so the error
    # of the running sum stays at ONE step's error instead of growing with the step count
    rel_ef = float((sum_ef - exact).norm() / exact.norm())
    rel_plain = float((sum_plain - exact).norm() / exact.norm())
    if rank == 0:
        print(f"world {world}, 8 steps, relative error of the accumulated sum: "
              f"with error feedback {rel_ef:.4f} without {rel_plain:.4f}")
        print("residual norms:", with_ef.residual_norms())
    dist.destroy_process_group()
    return rel_ef, rel_plain


if __name__ == "__main__":
    main()
