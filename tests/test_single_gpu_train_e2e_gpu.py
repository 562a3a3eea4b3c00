"""Single-GPU integration: a world-size-1 ``lowbit`` process group over a file store, a small
ResNet trained for a few synthetic steps with per-parameter ``LowBitGroup.all_reduce`` (the
plumbing exercised by the reference's ``tests/test_single_gpu_train_e2e.py:58-126``: with one
rank the dense path is taken through the backend)."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist

pytestmark = [pytest.mark.gpu, pytest.mark.integration]


def test_tiny_resnet_trains_through_lowbit_backend_world1():
    import bitscom_b200
    from bitscom_b200 import LowBitGroup
    from bitscom_b200.models.resnet import ResNet18

    if not bitscom_b200.is_extension_available():
        pytest.skip("backend extension not built")
    assert not dist.is_initialized()
    bitscom_b200.init(bitwidth=4)
    with tempfile.TemporaryDirectory() as tmp:
        dist.init_process_group("lowbit", init_method=f"file://{os.path.join(tmp, 'store')}",
                                rank=0, world_size=1)
        try:
            torch.manual_seed(0)
            model = ResNet18().cuda()
            before = [p.detach().clone() for p in model.parameters()]
            opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
            group = LowBitGroup(bitwidth=4)
            assert group.world_size == 1 and group.rank == 0
            x = torch.randn(32, 3, 32, 32, device="cuda")
            y = torch.randint(0, 10, (32,), device="cuda")
            losses = []
            for _ in range(5):
                opt.zero_grad(set_to_none=True)
                loss = torch.nn.functional.cross_entropy(model(x), y)
                loss.backward()
                for p in model.parameters():
                    if p.grad is not None:
                        group.all_reduce(p.grad)
                        p.grad.div_(group.world_size)
                opt.step()
                losses.append(loss.item())
            torch.cuda.synchronize()
            assert any(not torch.equal(a, b.detach()) for a, b in zip(before, model.parameters()))
            assert losses[-1] < losses[0]
        finally:
            dist.destroy_process_group()
