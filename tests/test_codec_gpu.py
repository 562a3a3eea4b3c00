"""CUDA codec kernels against the host quantizer (the bit-exact oracle)."""

import pytest
import torch

from bitscom_b200 import quantization as Q

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from bitscom_b200.ops import codec


def _cpu(fn, x, *a, **k):
    return fn(x.cpu(), *a, **k)


@pytest.fixture(autouse=True)
def _need_native():
    assert codec.available(), "native codec library must load on a GPU machine"
    assert Q._HAS_CUDA_KERNELS


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [1, 2, 4, 8, 12, 16])
@pytest.mark.parametrize("block,n", [(256, 4097), (256, 1 << 16), (64, 1000), (8, 77),
                                     (100, 1234), (6, 50), (512, 5000)])
def test_blockwise_bit_exact(dtype, bits, block, n):
    if not codec.supports_blockwise(bits, block):
        pytest.skip("block size not byte aligned for this bitwidth")
    g = torch.Generator().manual_seed(n + bits)
    x = (torch.randn(n, generator=g) * 1e-2).to(dtype)
    x[::97] = 0
    xd = x.cuda()
    p, s, m = Q.quantize_pack_tensor_blockwise(xd, bits, block_size=block)
    pc, sc, mc = Q.quantize_pack_tensor_blockwise(x, bits, block_size=block)
    assert m == mc and torch.equal(s.cpu(), sc)
    assert torch.equal(p.cpu(), pc)
    for out_dtype in (torch.float32, dtype):
        d = Q.unpack_dequantize_tensor_blockwise(p, s, bits, n, block_size=block, dtype=out_dtype)
        dc = Q.unpack_dequantize_tensor_blockwise(pc, sc, bits, n, block_size=block,
                                                  dtype=out_dtype)
        assert d.dtype == out_dtype and torch.equal(d.cpu(), dc)


def test_blockwise_unaligned_view_and_zero_blocks():
    x = torch.randn(5003)
    x[256:512] = 0
    xd = x.cuda()
    for start in (1, 3, 4):
        p, s, n = Q.quantize_pack_tensor_blockwise(xd[start:], 4, block_size=256)
        pc, sc, _ = Q.quantize_pack_tensor_blockwise(x[start:], 4, block_size=256)
        assert torch.equal(p.cpu(), pc) and torch.equal(s.cpu(), sc)


@pytest.mark.parametrize("block,n", [(256, 4096), (100, 1234)])
def test_nan_and_inf_blocks_match_the_host_quantizer(block, n):
    """A NaN makes its block's absmax NaN, which selects the scale 1.0; an infinity makes the
    scale infinite.  Both must come out as on the host (fast and generic kernels)."""
    x = torch.randn(n)
    x[3], x[block + 5], x[n - 2] = float("nan"), float("inf"), float("nan")
    for bits in (2, 4, 8):
        if not codec.supports_blockwise(bits, block):
            continue
        for sr in (False, True):
            kw = dict(block_size=block, stochastic_rounding=sr, sr_seed=5 if sr else None)
            p, s, _ = Q.quantize_pack_tensor_blockwise(x.cuda(), bits, **kw)
            pc, sc, _ = Q.quantize_pack_tensor_blockwise(x, bits, **kw)
            assert torch.equal(s.cpu().view(torch.int16), sc.view(torch.int16))
            assert torch.equal(p.cpu(), pc)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_seeded_stochastic_rounding_bit_exact(bits):
    x = torch.randn(10000) * 0.1
    kw = dict(block_size=256, stochastic_rounding=True, sr_seed=42, sr_offset=12345,
              sr_stream=1)
    p, s, _ = Q.quantize_pack_tensor_blockwise(x.cuda(), bits, **kw)
    pc, sc, _ = Q.quantize_pack_tensor_blockwise(x, bits, **kw)
    assert torch.equal(p.cpu(), pc) and torch.equal(s.cpu(), sc)


def test_unseeded_stochastic_rounding_unbiased_and_varies():
    x = torch.full((1 << 16,), 0.3, device="cuda")
    x[0] = 1.0
    means, first = [], None
    for _ in range(16):
        p, s, n = Q.quantize_pack_tensor_blockwise(x, 4, block_size=256,
                                                   stochastic_rounding=True)
        if first is None:
            first = p.clone()
        means.append(Q.unpack_dequantize_tensor_blockwise(p, s, 4, n)[256:].mean().item())
    assert abs(sum(means) / len(means) - 0.3) < 0.01
    assert not torch.equal(first, p)


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 12, 16])
def test_per_tensor_matches_cpu(bits):
    x = torch.randn(3, 1111) * 5
    q, scale = Q.quantize_tensor(x.cuda(), bits)
    qc, scale_c = Q.quantize_tensor(x, bits)
    assert q.shape == x.shape and abs(scale - scale_c) <= 1e-7 * max(1.0, abs(scale_c))
    assert torch.equal(q.cpu(), qc)
    y = Q.dequantize_tensor(q, scale)
    assert torch.equal(y.cpu(), Q.dequantize_tensor(qc, scale))
    r = Q.roundtrip_tensor(x.cuda().to(torch.bfloat16), bits)
    assert r.dtype == torch.bfloat16 and r.is_cuda


@pytest.mark.parametrize("bits", [1, 2, 4, 8, 12, 16])
def test_pack_unpack_full_range(bits):
    qmin, qmax = Q._quant_bounds(bits)
    vals = torch.arange(qmin, qmax + 1, dtype=torch.int32).to(torch.int16)
    vals = vals.repeat(max(1, 70 // vals.numel()))
    for n in (vals.numel(), vals.numel() - 1, 9, 1):
        q = vals[:n]
        p, m = Q.pack_lowbit(q.cuda(), bits)
        pc, _ = Q.pack_lowbit(q, bits)
        assert m == n and torch.equal(p.cpu(), pc)
        assert torch.equal(Q.unpack_lowbit(p, bits, n).cpu(), q)


def test_zero_and_empty():
    p, s, n = Q.quantize_pack_tensor_blockwise(torch.zeros(300, device="cuda"), 4)
    assert s.cpu().tolist() == [1.0, 1.0] and int(p.cpu().sum()) == 150 * 0x88
    q, sc = Q.quantize_tensor(torch.zeros(10, device="cuda"), 4)
    assert sc == 1.0 and int(q.abs().sum()) == 0


@pytest.mark.performance
def test_blockwise_bandwidth_report():
    n = 1 << 26  # 256 MiB of fp32, larger than L2
    x = torch.randn(n, device="cuda") * 1e-3
    for _ in range(3):
        p, s = codec.blockwise_quantize_pack(x, 4, 256)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        p, s = codec.blockwise_quantize_pack(x, 4, 256)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 5
    gbs = (n * 4 + p.numel() + s.numel() * 2) / ms / 1e6
    print(f"blockwise_quantize_pack 4-bit fp32 {n} elems: {ms:.3f} ms, {gbs:.0f} GB/s")
    assert gbs > 1000
