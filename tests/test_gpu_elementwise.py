"""GPU parity of the memory-bound ops against the CPU oracle (bit-exact), through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import random_lqq, random_tokens, to_torch_qw, bits, assert_bits_equal

pytestmark = pytest.mark.gpu

DEQUANT_SHAPES = [(1536, 4096), (1024, 4096), (2048, 4096), (1024, 14336), (6144, 4096)]


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("N,K", DEQUANT_SHAPES)
@pytest.mark.parametrize("g", [64, 128])
def test_dequant_matches_oracle(ops, N, K, g):
    """Shapes and group sizes of the reference's tests/test_kernel_dequant.py:17-30."""
    qw = random_lqq(N, K, g, seed=N + g)
    got = ops.dequant_weight_i8(to_torch_qw(qw))
    assert got.dtype == torch.int8 and got.shape == (N, K)
    assert np.array_equal(got.cpu().numpy(), O.dequantize_i8(qw))


def test_dequant_small_groups_and_quantised_weights(ops):
    W = O.synth_weight(96, 352, seed=3).astype(np.float32)
    for g in (4, 8, 16, 32, 44, 88):
        qw = O.quantize_weight(W, g)
        got = ops.dequant_weight_i8(to_torch_qw(qw))
        assert np.array_equal(got.cpu().numpy(), O.dequantize_i8(qw)), g


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,K", [(1, 4096), (7, 14336), (64, 4096), (300, 1000), (5, 24)])
def test_quant_per_token_matches_reference_formula(ops, dtype, M, K):
    """Bit-exact to quantize_activation (reference liquidgemm/quant.py:135-141): true division."""
    g = torch.Generator().manual_seed(M * 131 + K)
    x = torch.randn(M, K, generator=g)
    x[:, ::97] *= 10
    if M > 2:
        x[1] = 0.0                       # all-zero token -> scale floor 1e-12/127
        x[2] = 3e-13                     # below the floor
    x = x.to(dtype)
    xq, sc = torch.ops.liquidgemm.quant_per_token(x.cuda())
    e_q, e_s = O.quantize_activation(x.float().numpy())
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), e_s.view(np.uint32))
    assert np.array_equal(xq.cpu().numpy(), e_q)


@pytest.mark.parametrize("out_dtype", [0, 1, 2])
@pytest.mark.parametrize("M,N", [(1, 4096), (64, 6144), (100, 1001), (256, 512)])
def test_scale_epilogue_matches_oracle(ops, out_dtype, M, N):
    rng = np.random.default_rng(M + N)
    acc = rng.integers(-300000, 300000, (M, N), dtype=np.int32)
    acc[0, 0] = 2**31 - 1
    acc[-1, -1] = -2**31
    ascale = (rng.random(M, dtype=np.float32) * 0.02 + 0.01).astype(np.float32)
    s1 = (rng.random(N, dtype=np.float32) * 0.001 + 1e-5).astype(np.float32)
    got = torch.ops.liquidgemm.scale_epilogue(torch.from_numpy(acc).cuda(), torch.from_numpy(ascale).cuda(),
                                               torch.from_numpy(s1).cuda(), out_dtype)
    assert_bits_equal(got, O.scale_f32(acc, ascale, s1), out_dtype, "scale_epilogue")


@pytest.mark.parametrize("case", ["g64_small", "g128_small", "g64_tailed", "g64_flat"])
def test_golden_vectors_on_gpu(ops, golden, case):
    """The fixtures computed by the reference's own Python modules, replayed on the device."""
    qw = O.LQQWeight(golden.get(case, "q_u4"), golden.get(case, "s_u8"), golden.get(case, "offset_a"),
                     golden.get(case, "s1"), int(golden.get(case, "group")))
    assert np.array_equal(ops.dequant_weight_i8(to_torch_qw(qw)).cpu().numpy(), golden.get(case, "qhat_xor"))
    X = torch.from_numpy(golden.get(case, "X")).cuda()
    xq, sc = torch.ops.liquidgemm.quant_per_token(X)
    assert np.array_equal(xq.cpu().numpy(), golden.get(case, "x_i8"))
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), golden.get(case, "ascale").view(np.uint32))
    acc = torch.from_numpy(golden.get(case, "acc")).cuda()
    y = torch.ops.liquidgemm.scale_epilogue(acc, sc, torch.from_numpy(qw.s1).cuda(), 0)
    assert np.array_equal(bits(y), golden.get(case, "y_bf16_bits"))
    y = torch.ops.liquidgemm.scale_epilogue(acc, sc, torch.from_numpy(qw.s1).cuda(), 1)
    assert np.array_equal(bits(y), golden.get(case, "y_f16_bits"))


def test_argument_errors_raise_before_launch(ops):
    qw = to_torch_qw(random_lqq(64, 128, 64))
    with pytest.raises(RuntimeError):
        torch.ops.liquidgemm.dequant_weight(qw.qweight_u4, qw.s_u8, qw.offset_a, 64, 128, 48)
    with pytest.raises(RuntimeError):
        torch.ops.liquidgemm.scale_epilogue(torch.zeros(4, 4, device="cuda"), torch.zeros(4, device="cuda"),
                                            torch.zeros(4, device="cuda"), 0)
    with pytest.raises(RuntimeError):
        torch.ops.liquidgemm.quant_per_token(torch.zeros(4, device="cuda"))
