"""Host quantizer: API behaviour and bit-equality with the reference's Python oracle."""

import pytest
import torch

from bitscom_b200 import quantization as Q

BITS = (1, 2, 4, 8, 12, 16)


@pytest.mark.parametrize("bad", [0, 3, 5, 15, 17, -1])
def test_validate_bitwidth_rejects(bad):
    with pytest.raises(ValueError):
        Q.validate_bitwidth(bad)


@pytest.mark.parametrize("bits", BITS)
def test_pack_unpack_identity_full_range(bits):
    qmin, qmax = Q._quant_bounds(bits)
    values = torch.arange(qmin, qmax + 1, dtype=torch.int32)
    if values.numel() > 70000:
        values = values[::7]
    q = values.to(torch.int16)
    if q.numel() < 16:
        q = q.repeat(16 // q.numel() + 1)
    for n in (q.numel(), max(1, q.numel() - 1), 1, 3, 5, 9):
        packed, numel = Q.pack_lowbit(q[:n], bits)
        assert packed.dtype == torch.uint8 and numel == n
        assert packed.numel() == Q.packed_nbytes(n, bits)
        assert torch.equal(Q.unpack_lowbit(packed, bits, n), q[:n])


def test_pack_layout_first_element_in_low_bits():
    packed, _ = Q.pack_lowbit(torch.tensor([-8, 7], dtype=torch.int16), 4)
    assert packed.tolist() == [0x0 | (0xF << 4)]
    packed, _ = Q.pack_lowbit(torch.tensor([1, 0, 1, 1, 0, 0, 0, 1, 1], dtype=torch.int16), 1)
    assert packed.tolist() == [0b10001101, 0b1]
    packed, _ = Q.pack_lowbit(torch.tensor([-2048 + 0xABC, -2048 + 0x123], dtype=torch.int16), 12)
    assert packed.tolist() == [0xBC, 0xA | (0x3 << 4), 0x12]


@pytest.mark.parametrize("bits", (2, 4, 8, 12, 16))
def test_per_tensor_roundtrip_error_bounded(bits):
    torch.manual_seed(0)
    x = torch.randn(1000)
    q, scale = Q.quantize_tensor(x, bits)
    assert q.dtype == torch.int16 and q.shape == x.shape
    y = Q.dequantize_tensor(q, scale)
    assert (y - x).abs().max().item() <= scale * 0.5 + 1e-6


def test_per_tensor_one_bit_clamps_negatives():
    q, scale = Q.quantize_tensor(torch.tensor([-1.0, 0.4, 1.0, 0.6]), 1)
    assert q.tolist() == [0, 0, 1, 1] and scale == 1.0


def test_zero_tensor_gets_unit_scale():
    q, scale = Q.quantize_tensor(torch.zeros(16), 4)
    assert scale == 1.0 and int(q.abs().sum()) == 0
    q, scales = Q.quantize_tensor_blockwise(torch.zeros(300), 4, block_size=128)
    assert scales.tolist() == [1.0, 1.0, 1.0]


def test_type_and_value_errors():
    with pytest.raises(TypeError):
        Q.quantize_tensor(torch.arange(4), 4)
    with pytest.raises(TypeError):
        Q.quantize_tensor_blockwise(torch.arange(4), 4)
    with pytest.raises(ValueError):
        Q.quantize_tensor_blockwise(torch.randn(4), 4, block_size=0)
    with pytest.raises(ValueError):
        Q.dequantize_tensor_blockwise(torch.zeros(10, dtype=torch.int16),
                                      torch.ones(3, dtype=torch.float16), block_size=8)


def test_decompress_dtype_override_and_shape():
    x = torch.randn(4, 9, dtype=torch.float16)
    c = Q.compress_tensor(x, 8)
    assert c.packed_bytes == 36 and c.shape == (4, 9) and c.dtype == torch.float16
    assert Q.decompress_tensor(c).dtype == torch.float16
    y = Q.decompress_tensor(c, dtype=torch.float32)
    assert y.dtype == torch.float32 and y.shape == x.shape
    assert Q.roundtrip_tensor(x, 8).dtype == torch.float16


@pytest.mark.parametrize("bits", (2, 4, 8))
def test_blockwise_roundtrip_cpu(bits):
    torch.manual_seed(1)
    x = torch.randn(4097) * 3
    packed, scales, n = Q.quantize_pack_tensor_blockwise(x, bits, block_size=256)
    assert n == 4097 and scales.numel() == 17
    y = Q.unpack_dequantize_tensor_blockwise(packed, scales, bits, n, block_size=256)
    assert (y - x).abs().max().item() <= scales.float().max().item() * 0.5 + 1e-3


def test_blockwise_one_bit_drops_sign():
    q, s = Q.quantize_tensor_blockwise(torch.tensor([-1.0, 0.5, 1.0, -0.2]), 1, block_size=4)
    assert q.tolist() == [1, 0, 1, 0] and s.tolist() == [1.0]


def test_empty_inputs():
    q, s = Q.quantize_tensor_blockwise(torch.empty(0), 4)
    assert q.numel() == 0 and s.numel() == 0 and s.dtype == torch.float16
    assert Q.dequantize_tensor_blockwise(q, s).numel() == 0


def test_stochastic_rounding_unbiased_and_seeded():
    x = torch.full((4096,), 0.3)
    x[0] = 1.0  # absmax 1.0 -> 4-bit scale 1/7
    means = []
    for trial in range(64):
        q, s = Q.quantize_tensor_blockwise(x, 4, block_size=4096, stochastic_rounding=True,
                                           sr_seed=trial)
        means.append(Q.dequantize_tensor_blockwise(q, s, block_size=4096)[1:].mean().item())
    assert abs(sum(means) / len(means) - 0.3) < 0.005
    a = Q.quantize_tensor_blockwise(x, 4, stochastic_rounding=True, sr_seed=7)[0]
    b = Q.quantize_tensor_blockwise(x, 4, stochastic_rounding=True, sr_seed=7)[0]
    c = Q.quantize_tensor_blockwise(x, 4, stochastic_rounding=True, sr_seed=8)[0]
    assert torch.equal(a, b) and not torch.equal(a, c)
    # unseeded draws from torch's generator, like the reference
    d = Q.quantize_tensor_blockwise(x, 4, stochastic_rounding=True)[0]
    e = Q.quantize_tensor_blockwise(x, 4, stochastic_rounding=True)[0]
    assert not torch.equal(d, e)


def test_sr_offset_selects_substream():
    x = torch.rand(512)
    whole = Q.quantize_tensor_blockwise(x, 4, block_size=256, stochastic_rounding=True,
                                        sr_seed=3)[0]
    tail = Q.quantize_tensor_blockwise(x[256:], 4, block_size=256, stochastic_rounding=True,
                                       sr_seed=3, sr_offset=256)[0]
    assert torch.equal(whole[256:], tail)


def test_sr_uniform_range_and_mean():
    u = Q.sr_uniform(Q.sr_key(1234, 0), torch.arange(1 << 16))
    assert 0.0 <= u.min().item() and u.max().item() < 1.0
    assert abs(u.mean().item() - 0.5) < 0.01
    assert len(set(u[:1000].tolist())) > 990


# ---- bit-equality with the reference's Python quantizer ------------------------------

def _inputs():
    g = torch.Generator().manual_seed(5)
    yield torch.randn(1000, generator=g)
    yield torch.randn(4097, generator=g) * 1e-3
    yield torch.linspace(-3, 3, 777)
    spikes = torch.zeros(513)
    spikes[::37] = 50.0
    spikes[5] = -1e-4
    yield spikes
    yield torch.randn(300, generator=g).to(torch.bfloat16)
    yield torch.randn(300, generator=g).to(torch.float16)
    yield torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 3.5, 7.0])  # ties go to even


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("block", (256, 64, 100, 7))
def test_blockwise_matches_reference(reference_quantization, bits, block):
    R = reference_quantization
    for x in _inputs():
        q1, s1 = Q.quantize_tensor_blockwise(x, bits, block_size=block)
        q2, s2 = R.quantize_tensor_blockwise(x, bits, block_size=block)
        assert torch.equal(q1, q2) and torch.equal(s1, s2)
        p1, _, n1 = Q.quantize_pack_tensor_blockwise(x, bits, block_size=block)
        p2, _, n2 = R.quantize_pack_tensor_blockwise(x, bits, block_size=block)
        assert n1 == n2 and torch.equal(p1, p2)
        d1 = Q.unpack_dequantize_tensor_blockwise(p1, s1, bits, n1, block_size=block)
        d2 = R.unpack_dequantize_tensor_blockwise(p2, s2, bits, n2, block_size=block)
        assert torch.equal(d1, d2)


@pytest.mark.parametrize("bits", BITS)
def test_per_tensor_matches_reference(reference_quantization, bits):
    R = reference_quantization
    for x in _inputs():
        q1, s1 = Q.quantize_tensor(x, bits)
        q2, s2 = R.quantize_tensor(x, bits)
        assert s1 == s2 and torch.equal(q1, q2)
        c1, c2 = Q.compress_tensor(x, bits), R.compress_tensor(x, bits)
        assert torch.equal(c1.packed, c2.packed)
        assert torch.equal(Q.decompress_tensor(c1), R.decompress_tensor(c2))
