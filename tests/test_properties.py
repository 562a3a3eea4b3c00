"""Property-based checks (hypothesis) of the codec and of the all-reduce model: random sizes,
bitwidths, block sizes, seeds and value scales instead of hand-picked cases."""

import math

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from bitscom_b200 import quantization as Q  # noqa: E402
from bitscom_b200.ops import cpu_codec as C  # noqa: E402
from bitscom_b200.parallel.simulate import SimState, simulate_all_reduce  # noqa: E402

BITS = st.sampled_from([1, 2, 4, 8, 12, 16])
COMMON = dict(max_examples=40, deadline=None)


def _tensor(n, seed, log_scale):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * (10.0 ** log_scale)


@settings(**COMMON)
@given(bits=BITS, n=st.integers(1, 3000), seed=st.integers(0, 2 ** 20))
def test_pack_unpack_is_the_identity_on_codes(bits, n, seed):
    qmin, qmax = Q._quant_bounds(bits)
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(qmin, qmax + 1, (n,), generator=g, dtype=torch.int16)
    packed, count = Q.pack_lowbit(q, bits)
    assert count == n and packed.numel() == Q.packed_nbytes(n, bits)
    assert torch.equal(Q.unpack_lowbit(packed, bits, n), q)


@settings(**COMMON)
@given(bits=BITS, n=st.integers(1, 5000), block=st.sampled_from([1, 3, 8, 24, 64, 256, 1000]),
       seed=st.integers(0, 2 ** 20), log_scale=st.integers(-8, 4), sr=st.booleans())
def test_cpp_codec_equals_torch_quantizer(bits, n, block, seed, log_scale, sr):
    if not C.available():
        pytest.skip("no C++ compiler")
    x = _tensor(n, seed, log_scale)
    kw = dict(block_size=block, stochastic_rounding=sr, sr_seed=seed if sr else None,
              sr_offset=seed % 977)
    q, s = Q.quantize_tensor_blockwise(x, bits, **kw)
    want, _ = Q.pack_lowbit(q, bits)
    got, got_s = C.blockwise_quantize_pack(x, bits, block, sr, seed if sr else None, seed % 977)
    assert torch.equal(got_s.view(torch.int16), s.view(torch.int16))
    assert torch.equal(got, want)
    d = C.blockwise_unpack_dequantize(got, got_s, bits, n, block)
    assert torch.equal(d, Q.dequantize_tensor_blockwise(q, s, block_size=block).view(-1))


@settings(**COMMON)
@given(bits=st.sampled_from([2, 4, 8, 12, 16]), n=st.integers(1, 4000),
       block=st.sampled_from([8, 64, 256]), seed=st.integers(0, 2 ** 20),
       log_scale=st.integers(-6, 3))
def test_nearest_rounding_error_is_at_most_half_a_step(bits, n, block, seed, log_scale):
    x = _tensor(n, seed, log_scale)
    p, s, _ = Q.quantize_pack_tensor_blockwise(x, bits, block_size=block)
    y = Q.unpack_dequantize_tensor_blockwise(p, s, bits, n, block_size=block)
    step = s.float().repeat_interleave(block)[:n]
    # half a step, plus the fp16 rounding of the scale (relative 2^-11 when normal, absolute
    # 2^-25 when the scale is an fp16 subnormal) carried by the largest code
    qmax = 2 ** (bits - 1) - 1
    bound = 0.5 * step + qmax * (step * 2.0 ** -11 + 2.0 ** -25) * 1.01
    assert ((y - x).abs() <= bound).all()


@settings(max_examples=15, deadline=None)
@given(world=st.sampled_from([2, 3, 4, 8]), bits=st.sampled_from([1, 2, 4, 8]),
       n=st.integers(1, 3000), seed=st.integers(0, 2 ** 16))
def test_model_all_reduce_agrees_across_ranks_and_tracks_the_sum(world, bits, n, seed):
    ins = [_tensor(n, seed * 16 + r, -2) for r in range(world)]
    outs = simulate_all_reduce(ins, bits, 256)
    assert all(torch.equal(outs[0], o) for o in outs[1:])          # every rank, same bits
    if bits >= 4:
        exact = torch.stack(ins).sum(0)
        scale = max(float(t.abs().max()) for t in ins)
        tol = world * 1.2 * scale / (2 ** (bits - 1) - 1)          # two roundings, W sources
        assert float((outs[0] - exact).abs().max()) <= tol


@settings(max_examples=10, deadline=None)
@given(world=st.sampled_from([2, 4]), n=st.integers(64, 2000), seed=st.integers(0, 2 ** 16))
def test_error_feedback_keeps_the_running_sum_within_one_step(world, n, seed):
    """With both error-feedback stages the accumulated result differs from the accumulated
    exact sum only by what is still parked in the residuals: it does not grow with the
    number of steps."""
    state = SimState()
    exact, approx = torch.zeros(n), torch.zeros(n)
    errs = []
    for step in range(6):
        ins = [_tensor(n, seed * 64 + step * 8 + r, -2) for r in range(world)]
        out = simulate_all_reduce(ins, 4, 256, state=state, stage2=True)[0]
        exact += torch.stack(ins).sum(0)
        approx += out
        errs.append(float((approx - exact).norm()))
    assert errs[-1] < 2.5 * max(errs[:2]) + 1e-12
    assert errs[-1] < 0.5 * math.sqrt(6) * max(errs[0], 1e-12) * 2.5
