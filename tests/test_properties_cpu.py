"""Property-based checks (hypothesis) of the small host-side formats and helpers: they must hold
for every input of the stated domain, not just for the examples of the unit tests."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from rmlx_b200.parallel import wire
from rmlx_b200.parallel.algorithms import chunk_bounds
from rmlx_b200.reference import ops as ref


@settings(max_examples=80, deadline=None, derandomize=True)
@given(st.integers(0, 5000), st.integers(1, 17))
def test_chunk_bounds_partition_the_range(n, parts):
    b = chunk_bounds(n, parts)
    assert len(b) == parts and b[0][0] == 0 and b[-1][1] == n
    assert all(b[i][1] == b[i + 1][0] for i in range(parts - 1))
    sizes = [hi - lo for lo, hi in b]
    assert max(sizes) - min(sizes) <= 1 and sorted(sizes, reverse=True) == sizes


@settings(max_examples=80, deadline=None, derandomize=True)
@given(st.integers(0, (1 << 40) - 1), st.integers(0, 255), st.integers(0, 255), st.integers(0, 255))
def test_exchange_tag_round_trip(seq, tag, slot, peer):
    word = wire.pack_exchange_tag(seq, tag, slot, peer)
    assert 0 <= word < 1 << 64 and wire.unpack_exchange_tag(word) == (seq, tag, slot, peer)


def test_exchange_tag_rejects_out_of_range_fields():
    for bad in ((1 << 40, 0, 0, 0), (0, 256, 0, 0), (0, 0, -1, 0), (0, 0, 0, 256)):
        with pytest.raises(ValueError):
            wire.pack_exchange_tag(*bad)


@settings(max_examples=50, deadline=None, derandomize=True)
@given(st.lists(st.tuples(st.integers(0, 65535), st.integers(0, 65535)), max_size=12), st.integers(1, 24),
       st.integers(0, 2**32 - 1))
def test_v3_wire_format_round_trip_and_truncation(meta, stride, seed):
    rng = np.random.default_rng(seed)
    rows = rng.integers(0, 256, (len(meta), stride), dtype=np.uint8)
    experts, positions = [m[0] for m in meta], [m[1] for m in meta]
    buf = wire.pack_v3(experts, positions, rows)
    assert len(buf) == wire.v3_payload_bytes(len(meta), stride)
    e, p, r = wire.unpack_v3(buf, stride)
    assert e == experts and p == positions and np.array_equal(r, rows)
    if meta:
        with pytest.raises(wire.ProtocolError):
            wire.unpack_v3(buf[:-1], stride)
    framed = wire.crc_frame(buf)
    assert wire.crc_verify(framed) == buf
    if buf:
        broken = bytearray(framed)
        broken[0] ^= 0x40
        with pytest.raises(wire.ProtocolError):
            wire.crc_verify(bytes(broken))


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(1, 6), st.sampled_from([64, 128, 192]), st.sampled_from([4, 8]), st.integers(0, 2**31 - 1),
       st.floats(1e-3, 50.0))
def test_affine_quantiser_error_is_bounded_by_half_a_step(n, k, bits, seed, spread):
    """|w - dequant(quant(w))| <= scale / 2 (+ the bf16 rounding of scale and bias) in every group,
    codes stay in range, and re-quantising the reconstruction is a fixed point."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * spread + torch.randn(n, 1, generator=g) * spread).float()
    packed, scales, biases = ref.quantize_affine(w, bits=bits, group_size=64)
    assert packed.shape == (n, k * bits // 32) and scales.shape == biases.shape == (n, k // 64)
    back = ref.dequantize_affine(packed, scales, biases, bits=bits, group_size=64)
    s = scales.float().repeat_interleave(64, dim=1)
    lo = w.view(n, k // 64, 64).amin(-1)
    # the stored bias is the group minimum rounded to bf16: allow that rounding on top of half a step
    slack = (biases.float() - lo).abs().repeat_interleave(64, dim=1) + 1e-5 * (w.abs() + 1)   # fp32 arithmetic
    levels = (1 << bits) - 1
    inside = (w - biases.float().repeat_interleave(64, dim=1)) / s
    clipped = (inside < -0.5) | (inside > levels + 0.5)            # beyond the representable range after rounding
    err = (back - w).abs()
    assert bool(((err <= 0.5 * s + slack) | clipped).all())
    again = ref.quantize_affine(back, bits=bits, group_size=64)
    assert torch.allclose(ref.dequantize_affine(*again, bits=bits, group_size=64), back, atol=float(s.max()) * 1.01)


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(1, 5), st.integers(1, 40), st.integers(0, 2**31 - 1))
def test_fp8_row_payload_keeps_the_row_maximum_and_three_bits(n, d, seed):
    from rmlx_b200.parallel.ep import fp8_dequant_rows, fp8_quant_rows
    x = torch.randn(n, d, generator=torch.Generator().manual_seed(seed)) * 7
    q, s = fp8_quant_rows(x)
    back = fp8_dequant_rows(q, s, torch.float32)
    amax = x.abs().amax(-1)
    assert q.dtype == torch.uint8 and torch.allclose(back.abs().amax(-1), amax, rtol=1e-6)
    # E4M3: 3 mantissa bits -> relative error at most 2^-4 of the value, plus the subnormal step of the scaled range
    assert bool(((back - x).abs() <= x.abs() / 16 + (amax / 448 * 2**-9)[:, None] + 1e-7).all())
    assert wire.fp8_unpack_tokens(wire.fp8_pack_tokens(x), n, d).shape == (n, d)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(st.integers(2, 300), st.floats(0.05, 3.0), st.integers(0, 64), st.floats(0.05, 1.0), st.floats(0.5, 2.5),
       st.integers(0, 2**31 - 1), st.lists(st.integers(0, 299), max_size=8))
def test_native_sampler_distribution_properties(vocab, temperature, top_k, top_p, penalty, seed, history):
    """For any configuration: the native distribution equals the torch-op one, sums to one, keeps at
    most top-k tokens (ties aside), and its kept mass reaches top-p of the shaped distribution."""
    from rmlx_b200.config import SamplerConfig
    from rmlx_b200.serve import native
    from rmlx_b200.serve.sampler import Sampler
    if not native.available():
        pytest.skip("host library not available")
    cfg = SamplerConfig(temperature=temperature, top_k=top_k, top_p=top_p, repetition_penalty=penalty, seed=1)
    logits = torch.randn(vocab, generator=torch.Generator().manual_seed(seed)) * 3
    hist = [h for h in history if h < vocab]
    want = Sampler(cfg).probabilities(logits, hist)
    got = native.NativeSampler(cfg).probabilities(logits, hist)
    assert torch.allclose(got, want, atol=2e-6)
    assert abs(float(got.sum()) - 1.0) < 1e-4 and bool((got >= 0).all())
    kept = int((got > 0).sum())
    if 0 < top_k < vocab:
        assert kept <= top_k
    assert kept >= 1 and int(got.argmax()) == int(want.argmax())
