"""torch DistributedDataParallel with the low-bit communication hook (2-bit + error feedback).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/ddp_comm_hook.py
"""

import os

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

import bitscom_b200 as bitscom
from bitscom_b200.parallel.hooks import lowbit_ddp_comm_hook, make_ddp_hook_state


def main(steps: int = 30):
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank = dist.get_rank()
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(),
                                torch.nn.Linear(256, 10)).to(device)
    ddp = DDP(model, device_ids=[device.index] if use_cuda else None)
    group = bitscom.LowBitGroup(bitwidth=2, error_feedback=True)
    ddp.register_comm_hook(make_ddp_hook_state(group, average=True), lowbit_ddp_comm_hook)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1, momentum=0.9)

    g = torch.Generator().manual_seed(1 + rank)
    teacher = torch.randn(64, 10, generator=torch.Generator().manual_seed(99))
    losses = []
    for _ in range(steps):
        x = torch.randn(128, 64, generator=g)
        y = (x @ teacher).argmax(1)
        loss = torch.nn.functional.cross_entropy(ddp(x.to(device)), y.to(device))
        opt.zero_grad(set_to_none=True)
        loss.backward()                    # buckets are all-reduced in 2 bits as they fill
        opt.step()
        losses.append(float(loss.item()))
    if rank == 0:
        print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
