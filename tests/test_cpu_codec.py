"""C++ CPU codec against the host quantizer: bit-exact, and faster."""

import time

import pytest
import torch

from bitscom_b200 import quantization as Q
from bitscom_b200.ops import cpu_codec as C

pytestmark = pytest.mark.skipif(not C.available(), reason="no C++ compiler for the CPU codec")


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 12, 16])
@pytest.mark.parametrize("block,n", [(256, 4097), (64, 1000), (100, 1234), (7, 50), (256, 1)])
def test_bit_exact_nearest_and_seeded_sr(bits, block, n):
    g = torch.Generator().manual_seed(n + bits)
    x = torch.randn(n, generator=g) * 1e-2
    x[::13] = 0
    if n > 600:
        x[512:768] = 0          # an all-zero block
        x[300] = 1e-9           # tiny values next to large ones
    for sr in (False, True):
        kw = dict(stochastic_rounding=sr, sr_seed=7 if sr else None, sr_offset=33, sr_stream=1)
        q, s = Q.quantize_tensor_blockwise(x, bits, block_size=block, **kw)
        want_p, _ = Q.pack_lowbit(q, bits)
        p, sc = C.blockwise_quantize_pack(x, bits, block, sr, 7 if sr else None, 33, 1)
        assert torch.equal(sc, s)
        assert torch.equal(p, want_p)
        d = C.blockwise_unpack_dequantize(p, sc, bits, n, block)
        assert torch.equal(d, Q.dequantize_tensor_blockwise(q, s, block_size=block))


def test_half_conversion_matches_torch_on_edge_values():
    vals = torch.tensor([0.0, 1e-8, 5.96e-8, 6.1e-5, 6.0e-5, 1.0, 1.0009765625, 65504.0,
                         65519.9, 65520.0, 1e6, 3.3e-8, 2.98e-8, 2.9802322e-8])
    for v in vals.tolist():
        x = torch.tensor([v, 0.0])          # absmax = v, qmax = 1 for 2-bit
        _, sc = C.blockwise_quantize_pack(x, 2, 2)
        want = Q.quantize_tensor_blockwise(x, 2, block_size=2)[1]
        assert torch.equal(sc, want), v


@pytest.mark.performance
def test_faster_than_torch_ops_on_cpu():
    x = torch.randn(1 << 20)
    t0 = time.perf_counter()
    for _ in range(3):
        Q.quantize_pack_tensor_blockwise(x, 4)
    t_torch = (time.perf_counter() - t0) / 3
    t0 = time.perf_counter()
    for _ in range(3):
        C.blockwise_quantize_pack(x, 4, 256)
    t_cpp = (time.perf_counter() - t0) / 3
    print(f"CPU 1 Mi elements 4-bit: torch ops {t_torch * 1e3:.2f} ms, C++ {t_cpp * 1e3:.2f} ms")
    assert t_cpp < t_torch * 2


@pytest.mark.parametrize("bits", [1, 4, 12])
@pytest.mark.parametrize("block", [8, 256, 1000])
def test_threaded_path_and_special_values_are_bit_exact(bits, block):
    """Large tensors are split over threads; infinities, zero blocks, tiny blocks and NaN
    (which selects scale 1.0 for its block, as in the host quantizer) stay bit-exact."""
    old = torch.get_num_threads()
    torch.set_num_threads(4)
    try:
        n = (1 << 19) + 37
        g = torch.Generator().manual_seed(bits * 1000 + block)
        x = torch.randn(n, generator=g) * torch.rand(n, generator=g).pow(4)
        x[5], x[4000], x[300000] = float("inf"), float("-inf"), 0.0
        x[100 * block:101 * block] = 0.0
        x[200 * block:201 * block] = 1e-9
        x[7 * block + 3] = float("nan")
        for sr in (False, True):
            q, s = Q.quantize_tensor_blockwise(x, bits, block_size=block, stochastic_rounding=sr,
                                               sr_seed=7, sr_offset=11)
            want_p, _ = Q.pack_lowbit(q, bits)
            p, sc = C.blockwise_quantize_pack(x, bits, block, sr, 7, 11)
            assert torch.equal(sc.view(torch.int16), s.view(torch.int16))
            assert torch.equal(p, want_p)
            d = C.blockwise_unpack_dequantize(p, sc, bits, n, block)
            want_d = Q.dequantize_tensor_blockwise(q, s, block_size=block).view(-1)
            assert torch.equal(torch.nan_to_num(d, nan=7.0), torch.nan_to_num(want_d, nan=7.0))
    finally:
        torch.set_num_threads(old)
