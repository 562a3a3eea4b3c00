"""Single-GPU integration: a world-size-1 ``lowbit`` process group over a file store, a small
ResNet trained for a few synthetic steps with per-parameter ``LowBitGroup.all_reduce`` (the
plumbing exercised by the reference's ``tests/test_single_gpu_train_e2e.py:58-126``: with one
rank the dense path is taken through the backend's inner NCCL group).

Each case runs in a child process with a time limit: the teardown of a process group joins
helper threads, and a teardown that never returns must fail this one test, not stop the run.
"""

import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.integration]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = textwrap.dedent("""
    import json, os, sys, tempfile, time
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    import bitscom_b200
    from bitscom_b200 import LowBitGroup
    from bitscom_b200.models.resnet import ResNet18

    explicit_shutdown = {explicit!r}
    assert bitscom_b200.is_extension_available()
    bitscom_b200.init(bitwidth=4)
    with tempfile.TemporaryDirectory() as tmp:
        dist.init_process_group("lowbit", init_method="file://" + os.path.join(tmp, "store"),
                                rank=0, world_size=1)
        torch.manual_seed(0)
        model = ResNet18().cuda()
        before = [p.detach().clone() for p in model.parameters()]
        opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
        group = LowBitGroup(bitwidth=4)
        assert group.world_size == 1 and group.rank == 0
        x = torch.randn(32, 3, 32, 32, device="cuda")
        y = torch.randint(0, 10, (32,), device="cuda")
        losses = []
        t0 = time.time()
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
        step_ms = (time.time() - t0) / 5 * 1e3
        changed = any(not torch.equal(a, b.detach()) for a, b in zip(before, model.parameters()))
        t1 = time.time()
        if explicit_shutdown:
            bitscom_b200.shutdown()
        dist.destroy_process_group()
        teardown_s = time.time() - t1
    # the process keeps running after the teardown: the interpreter is still usable
    z = (torch.ones(4, device="cuda") * 2).sum().item()
    print(json.dumps(dict(losses=losses, changed=changed, avg_step_time_ms=step_ms,
                          teardown_s=teardown_s, after=z)))
""")


@pytest.mark.parametrize("explicit_shutdown", [True, False])
def test_tiny_resnet_trains_through_lowbit_backend_world1(explicit_shutdown):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    code = _CHILD.format(root=ROOT, explicit=explicit_shutdown)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                          timeout=240, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    out = json.loads(proc.stdout.strip().splitlines()[-1])
    assert out["changed"] and out["after"] == 8.0
    assert out["losses"][-1] < out["losses"][0]
    assert out["teardown_s"] < 60
