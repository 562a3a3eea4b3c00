"""ZeRO-1 style training on low-bit collectives: every rank keeps the bf16 model but only 1 / W of
the fp32 master weights and AdamW moments; gradients arrive by a 4-bit reduce-scatter, updated
parameters leave by an 8-bit all-gather (error feedback on both).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/sharded_optimizer.py
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bitscom_b200 as bitscom  # noqa: E402
from bitscom_b200.parallel.flat import FlatParameters  # noqa: E402
from bitscom_b200.parallel.zero import ShardedAdamW  # noqa: E402


def main(steps: int = 60):
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    # parameters live in ONE flat bf16 buffer (padded so that every rank owns an equal shard);
    # the model's tensors are views of it, their gradients views of one flat fp32 buffer
    shapes = {"w1": (128, 32), "b1": (128,), "w2": (1, 128)}
    flat = FlatParameters(shapes, device, pad_to=256 * world)
    init = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for name, view in flat.named_views():
            view.copy_(torch.randn(view.shape, generator=init) * (0.0 if name == "b1" else 0.1))
    flat.sync_master_from_params()
    params = {name: flat.make_parameter(name) for name in shapes}

    grads_group = bitscom.LowBitGroup(bitwidth=4, error_feedback=True)
    params_group = bitscom.LowBitGroup(bitwidth=8, error_feedback=True)
    opt = ShardedAdamW(flat, grads_group, lr=2e-2, weight_decay=0.0,
                       param_bits_group=params_group)

    data = torch.Generator().manual_seed(1 + rank)
    teacher = torch.randn(32, 1, generator=torch.Generator().manual_seed(99))
    losses = []
    for _ in range(steps):
        x = torch.randn(256, 32, generator=data)
        y = torch.tanh(x @ teacher)
        x, y = x.to(device, flat.dtype), y.to(device)
        h = torch.tanh(x @ params["w1"].t() + params["b1"])
        loss = torch.nn.functional.mse_loss((h @ params["w2"].t()).float(), y)
        for p in params.values():
            p.grad = None
        loss.backward()
        for name, p in params.items():          # into the flat fp32 gradient buffer
            flat.grad_view(name).add_(p.grad.float())
        opt.step()                               # reduce-scatter, AdamW on the shard, all-gather
        losses.append(float(loss.detach()))
    params_group.check_agreement(flat.params)    # every rank holds the same bf16 model
    if rank == 0:
        shard = flat.numel // world
        print(f"each of {world} ranks keeps {shard} of {flat.numel} fp32 master weights")
        print(f"loss {losses[0]:.4f} -> {losses[-1]:.4f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
