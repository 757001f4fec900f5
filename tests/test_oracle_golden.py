"""Pin the numpy oracle against numbers computed by the reference's own Python modules."""

import numpy as np
import pytest

from oracle import lqq_oracle as O

CASES = ["g64_small", "g128_small", "g64_tailed", "g64_flat"]


def _qw(golden, c):
    return O.LQQWeight(golden.get(c, "q_u4"), golden.get(c, "s_u8"), golden.get(c, "offset_a"),
                       golden.get(c, "s1"), int(golden.get(c, "group")))


@pytest.mark.parametrize("c", CASES)
def test_quantize_weight_matches_reference(golden, c):
    qw = O.quantize_weight(golden.get(c, "W").astype(np.float32), int(golden.get(c, "group")))
    assert np.array_equal(qw.qweight_u4, golden.get(c, "q_u4"))
    assert np.array_equal(qw.s_u8, golden.get(c, "s_u8"))
    assert np.array_equal(qw.offset_a, golden.get(c, "offset_a"))
    assert np.array_equal(qw.s1.view(np.uint32), golden.get(c, "s1").view(np.uint32))


@pytest.mark.parametrize("c", CASES)
def test_dequant_matches_reference(golden, c):
    qw = _qw(golden, c)
    assert np.array_equal(O.dequantize_i8_xor(qw), golden.get(c, "qhat_xor"))
    assert np.array_equal(O.dequantize_i8_sub(qw), golden.get(c, "qhat_sub"))
    assert np.array_equal(O.simd_dequant_u32(qw), golden.get(c, "simd_qhat"))
    if golden.has(c, "w_hat"):
        assert np.array_equal(O.dequantize(qw).view(np.uint32), golden.get(c, "w_hat").view(np.uint32))


@pytest.mark.parametrize("c", CASES)
def test_activation_quant_matches_reference(golden, c):
    x8, asc = O.quantize_activation(golden.get(c, "X").astype(np.float32))
    assert np.array_equal(x8, golden.get(c, "x_i8"))
    assert np.array_equal(asc.view(np.uint32), golden.get(c, "ascale").view(np.uint32))


@pytest.mark.parametrize("c", CASES)
def test_matmul_and_casts_match_reference(golden, c):
    qw = _qw(golden, c)
    x8, asc = golden.get(c, "x_i8"), golden.get(c, "ascale")
    qhat = O.dequantize_i8(qw)
    acc = O.int_accumulate(x8, qhat)
    assert np.array_equal(acc, golden.get(c, "acc"))
    assert np.array_equal(O.int_accumulate_slow(x8, qhat), golden.get(c, "acc"))
    y = O.w4a8_matmul(x8, asc, qw)
    assert np.array_equal(y.view(np.uint32), golden.get(c, "y_f32").view(np.uint32))
    assert np.array_equal(O.w4a8_linear(x8, asc, qw, O.OUT_BF16), golden.get(c, "y_bf16_bits"))
    assert np.array_equal(O.w4a8_linear(x8, asc, qw, O.OUT_F16), golden.get(c, "y_f16_bits"))
    assert np.array_equal(O.scale_epilogue(acc, asc, qw.s1, O.OUT_BF16), golden.get(c, "y_bf16_bits"))


@pytest.mark.parametrize("c", CASES)
def test_packing_matches_reference(golden, c):
    qw = _qw(golden, c)
    nib = O.pack_nibbles(qw.qweight_u4)
    assert np.array_equal(nib, golden.get(c, "nibbles"))
    assert np.array_equal(O.unpack_nibbles(nib), qw.qweight_u4)
    assert np.array_equal(O.pack_lanes_u32(qw.qweight_u4).astype(np.uint32), golden.get(c, "lanes_u32"))
    assert np.array_equal(O.pack_gemv_interleaved(qw), golden.get(c, "gemv_pack"))


def test_bf16_rounding_edge_cases():
    import torch
    vals = np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, -3.4e38, 1e-40,
                     np.inf, -np.inf, 65504.0, 65520.0, 7.96, 1.0000001], dtype=np.float32)
    rng = np.random.default_rng(0)
    vals = np.concatenate([vals, rng.standard_normal(4096).astype(np.float32) * 100,
                           rng.integers(0, 2**32, 4096, dtype=np.uint64).astype(np.uint32).view(np.float32)])
    vals = vals[~np.isnan(vals)]
    t = torch.from_numpy(vals)
    ref_bf = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    ref_h = t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.f32_to_bf16_bits(vals), ref_bf)
    assert np.array_equal(O.f32_to_f16_bits(vals), ref_h)
