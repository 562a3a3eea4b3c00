"""Public-API round trip on two CPU ranks (gloo): the calls of the reference's integration
script (``tests/test_e2e.py:18-62``: all_reduce of rank-valued ones, broadcast from rank 0)
plus the pass-through collectives and the simulate-quantization switch; and the loose
host-side performance checks of ``tests/test_perf_quantization.py:27-54``."""

import os
import time

import pytest
import torch
import torch.distributed as dist

import bitscom_b200 as bitscom
from bitscom_b200.quantization import compress_tensor, decompress_tensor, roundtrip_tensor

from _dist import run_ranks


def _api_round_trip(rank, world):
    # a constant tensor sits on the top code, so the only error is the fp16 rounding of the
    # two scales (the reference's script checks 1e-3 absolute against a dense placeholder)
    t = torch.ones(1024) * (rank + 1)
    group = bitscom.LowBitGroup(bitwidth=4)
    assert group.rank == rank and group.world_size == world
    assert group.all_reduce(t) is None
    want = float(sum(range(1, world + 1)))
    assert abs(t.sum().item() - want * 1024) < 2e-3 * want * 1024
    assert (t - t[0]).abs().max().item() == 0.0

    b = torch.arange(100, dtype=torch.float32) if rank == 0 else torch.zeros(100)
    group.broadcast(b, src=0)
    assert torch.equal(b, torch.arange(100, dtype=torch.float32))

    parts = [torch.empty(8) for _ in range(world)]
    group.all_gather(parts, torch.full((8,), float(rank)))
    assert [p[0].item() for p in parts] == [float(r) for r in range(world)]

    work = group.all_reduce(torch.ones(64), async_op=True)
    work.wait()

    # simulate_quantization on a dense (8-bit) group: values take a quantize round trip first
    sim = bitscom.LowBitGroup(bitwidth=8, simulate_quantization=True)
    x = torch.linspace(-1, 1, 257) * (rank + 1)
    y = x.clone()
    sim.all_reduce(y)
    exact = torch.linspace(-1, 1, 257) * sum(range(1, world + 1))
    err = (y - exact).abs().max().item()
    assert 0 < err < 0.02 * world

    # SUM is the only low-bit reduction: MAX goes through the dense path untouched
    m = torch.full((16,), float(rank))
    group.all_reduce(m, op=dist.ReduceOp.MAX)
    assert torch.equal(m, torch.full((16,), float(world - 1)))


def test_public_api_round_trip_two_ranks():
    run_ranks(_api_round_trip, 2)


def _bench(fn, warmup=2, iters=10):
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) / iters


@pytest.mark.performance
@pytest.mark.skipif(os.getenv("BITSCOM_RUN_PERF", "0") != "1",
                    reason="set BITSCOM_RUN_PERF=1 to run performance tests")
def test_roundtrip_cost_is_bounded():
    x = torch.randn(1_000_000)
    rt, clone = _bench(lambda: roundtrip_tensor(x, 4)), _bench(lambda: x.clone())
    assert 0 < rt < clone * 200


def test_compression_ratio():
    x = torch.randn(500_000)
    for bits in (1, 2, 4, 8, 12, 16):
        c = compress_tensor(x, bits)
        assert decompress_tensor(c).shape == x.shape
        assert c.packed_bytes == -(-x.numel() * bits // 8) if bits != 12 \
            else c.packed_bytes == 3 * ((x.numel() + 1) // 2)
        assert c.packed_bytes < x.numel() * 4
