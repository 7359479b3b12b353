"""Properties of the quantisers' PyTorch statements over arbitrary inputs (hypothesis): power-of-two rounding, error bounds of the
fp8 block and NVFP4 formats, and the packing round trip."""
import torch
from hypothesis import given, settings, strategies as st

from nanoengine_b200.ops import reference as ref

finite = st.floats(min_value=-8192.0, max_value=8192.0, allow_nan=False, allow_infinity=False, width=32)


@settings(derandomize=True, max_examples=200, deadline=None)
@given(st.lists(st.floats(min_value=2.0 ** -100, max_value=2.0 ** 100, allow_nan=False, width=32), min_size=1, max_size=32))
def test_ceil_pow2_is_the_next_power_of_two(xs):
    s = torch.tensor(xs, dtype=torch.float32)
    p = ref._ceil_pow2(s)
    assert bool(((p.view(torch.int32) & 0x7FFFFF) == 0).all())           # a power of two
    assert bool((p >= s).all()) and bool((p < 2 * s).all())


@settings(derandomize=True, max_examples=60, deadline=None)
@given(st.lists(finite, min_size=128, max_size=128), st.booleans())
def test_fp8_group_quantisation_error_is_bounded_by_the_format(xs, pow2):
    x = torch.tensor(xs, dtype=torch.float32).view(1, 128)
    q, s = ref.quant_fp8_1x128(x, ue8m0=pow2)
    back = ref.dequant_fp8_1x128(q, s)
    amax = float(x.abs().max())
    # e4m3 keeps 3 mantissa bits: relative step 2^-3 near the top of a binade; a power-of-two scale may waste one binade of range
    assert float((back - x).abs().max()) <= max(amax, 1e-10) * 2 ** -4 * 1.01 + 1e-12
    if pow2:
        assert bool(((s.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all())


@settings(derandomize=True, max_examples=60, deadline=None)
@given(st.lists(finite, min_size=64, max_size=64), st.floats(min_value=0.5, max_value=200.0, allow_nan=False))
def test_nvfp4_round_trip_and_error_bound(xs, g):
    x = torch.tensor(xs, dtype=torch.float32).view(1, 64)
    q, sf = ref.nvfp4_quant(x, torch.tensor([g]))
    assert q.shape == (1, 32) and sf.shape == (1, 4)
    back = ref.nvfp4_unpack(q, sf) / g
    blocks, bb = x.view(4, 16), back.view(4, 16)
    for i in range(4):
        amax = float(blocks[i].abs().max())
        sfv = float(sf.float().view(4)[i])
        if sfv == 0.0:
            assert float(bb[i].abs().max()) == 0.0
            continue
        if g * amax / 6.0 > 448.0:
            continue                                  # the block scale saturates (activations beyond the calibrated range): values clip
        # e2m1 steps are at most 2 (between 4 and 6) in units of the block scale; the e4m3 scale itself is within 1/16 of amax / 6
        assert float((bb[i] - blocks[i]).abs().max()) <= (sfv / g) * 1.0 + amax * 0.07 + 1e-12
    # re-quantising the dequantised values with the same scale is the identity on the codes
    q2, sf2 = ref.nvfp4_quant(ref.nvfp4_unpack(q, sf) / g, torch.tensor([g]))
    assert torch.equal(ref.nvfp4_unpack(q2, sf2), ref.nvfp4_unpack(q, sf)) or float(sf.float().min()) == 0.0
