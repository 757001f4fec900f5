"""Decode GEMV (M <= 16) parity against the CPU oracle: bit-exact scaled outputs."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import LLAMA8B, random_lqq, random_tokens, to_torch_qw, assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


def _run(ops, qw, x, ascale, out_dtype):
    tq = to_torch_qw(qw)
    gp = ops.pack_gemv_interleaved(tq)
    return torch.ops.liquidgemm.w4a8_gemv2(torch.from_numpy(x).cuda(), gp, tq.s_u8, tq.offset_a,
                                           torch.from_numpy(ascale).cuda(), tq.s1, qw.N, qw.K, 64, out_dtype)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_gemv_matches_oracle_small(ops, M, out_dtype):
    """N=512, K=4096 as in the reference's tests/test_wgmma.py:108-124, every M bucket."""
    qw = random_lqq(512, 4096, 64, seed=M)
    x, ascale = random_tokens(M, 4096, seed=100 + M)
    got = _run(ops, qw, x, ascale, out_dtype)
    assert got.shape == (M, 512)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), out_dtype, f"gemv M={M}")


@pytest.mark.parametrize("N,K", [(200, 1152), (24, 128), (1000, 2176), (130, 14336)])
@pytest.mark.parametrize("M", [1, 4, 7, 16])
def test_gemv_ragged_shapes(ops, N, K, M):
    """N not a multiple of the rows a warp owns, K not a multiple of the 1024-k sweep."""
    qw = random_lqq(N, K, 64, seed=N + K)
    x, ascale = random_tokens(M, K, seed=M)
    got = _run(ops, qw, x, ascale, 0)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 0, f"gemv {N}x{K} M={M}")


@pytest.mark.parametrize("name", ["qkv", "gate_up", "down"])
@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_gemv_llama_shapes(ops, name, M):
    """The decode sweep of the benchmark at full size."""
    N, K = LLAMA8B[name]
    qw = random_lqq(N, K, 64, seed=7)
    x, ascale = random_tokens(M, K, seed=M)
    got = _run(ops, qw, x, ascale, 0)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 0, f"gemv {name} M={M}")


def test_gemv_quantised_weights_with_outliers(ops):
    """End to end from fp16 data: quantise (oracle), run the device path, compare with the oracle."""
    W = O.synth_weight(1024, 4096, seed=0)
    X = O.synth_activation(4, 4096, seed=1)
    qw = O.quantize_weight(W.astype(np.float32), 64)
    xq, sc = torch.ops.liquidgemm.quant_per_token(torch.from_numpy(X).cuda())
    e_q, e_s = O.quantize_activation(X.astype(np.float32))
    assert np.array_equal(xq.cpu().numpy(), e_q)
    tq = to_torch_qw(qw)
    got = torch.ops.liquidgemm.w4a8_gemv2(xq, ops.pack_gemv_interleaved(tq), tq.s_u8, tq.offset_a, sc, tq.s1,
                                          1024, 4096, 64, 1)
    assert_bits_equal(got, O.w4a8_matmul(e_q, e_s, qw), 1, "gemv fp16 end to end")


def test_gemv_rejects_bad_shapes(ops):
    qw = random_lqq(64, 256, 64)
    tq = to_torch_qw(qw)
    gp = ops.pack_gemv_interleaved(tq)
    x = torch.zeros(17, 256, dtype=torch.int8, device="cuda")
    a = torch.ones(17, device="cuda")
    with pytest.raises(RuntimeError):
        torch.ops.liquidgemm.w4a8_gemv2(x, gp, tq.s_u8, tq.offset_a, a, tq.s1, 64, 256, 64, 0)
    with pytest.raises(RuntimeError):
        torch.ops.liquidgemm.w4a8_gemv2(x[:4], gp, tq.s_u8, tq.offset_a, a[:4], tq.s1, 64, 256, 128, 0)


@pytest.mark.parametrize("M", [1, 4, 16])
def test_v1_gemm_small_m_plain_nibbles(ops, M):
    """ops.w4a8_gemm (plain pack_nibbles layout, fp32 inside) for the GEMV range."""
    qw = random_lqq(512, 4096, 64, seed=11)
    x, ascale = random_tokens(M, 4096, seed=M)
    got = ops.w4a8_gemm(torch.from_numpy(x), torch.from_numpy(ascale), to_torch_qw(qw), out_dtype=torch.float32)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 2, f"v1 M={M}")
