"""The INT8 x INT8 CTA-pair GEMM (tcgen05.mma.cta_group::2, both operands from shared memory, 256 channels x 256
tokens per tile) that the plain INT8 operators take for large token counts, against the CPU oracle on slices and
against cuBLASLt's exact INT8 GEMM on the whole result; the same calls with the pair kernel switched off must
give the same bits."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


def _operands(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    a[0, :] = -127                                        # extreme rows: the largest sums an int32 tile can see
    b[0, :] = -128
    b[N - 1, :] = 127
    sa = (rng.random(M, dtype=np.float32) * 0.02 + 0.01).astype(np.float32)
    sb = (rng.random(N, dtype=np.float32) * 0.001 + 1e-5).astype(np.float32)
    return a, b, sa, sb


# (M, N, K): two tiles per pair exactly; ragged tokens over several waves; one k-step; a long K; the 8B qkv shape
CASES = [(4096, 2560, 512), (4000, 2560, 384), (9473, 1024, 128), (2048, 6144, 4096), (1500, 7168, 2048)]


@pytest.mark.parametrize("M,N,K", CASES)
def test_int32_sums_are_exact(ops, M, N, K, monkeypatch):
    a, b, _, _ = _operands(M, N, K, seed=M + N)
    at, bt = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    got = torch.ops.liquidgemm.wgmma_i8_gemm(at, bt)
    assert torch.equal(got, torch._int_mm(at, bt.t()))
    rows = slice(M - 9, M)
    assert np.array_equal(got[rows].cpu().numpy(), O.int_accumulate(a[rows], b))
    monkeypatch.setenv("LQ_I8_PAIR", "0")
    assert torch.equal(torch.ops.liquidgemm.wgmma_i8_gemm(at, bt), got)
    ops.poll_status()


@pytest.mark.parametrize("M,N,K", CASES[:3])
@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_scaled_outputs_are_bit_exact(ops, M, N, K, out_dtype, monkeypatch):
    a, b, sa, sb = _operands(M, N, K, seed=K)
    at, bt = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    sat, sbt = torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda()
    got = torch.ops.liquidgemm.i8_gemm_scaled(at, bt, sat, sbt, out_dtype)
    # tolerance: none -- exact integer sums, two fp32 multiplies, one rounding to the output type
    for rows in (slice(0, 8), slice(M - 8, M)):
        assert_bits_equal(got[rows], O.scale_f32(O.int_accumulate(a[rows], b), sa[rows], sb), out_dtype, "i8 pair scaled")
    want = torch.ops.liquidgemm.scale_epilogue(torch._int_mm(at, bt.t()), sat, sbt, out_dtype)
    assert torch.equal(got, want)
    monkeypatch.setenv("LQ_I8_PAIR", "0")
    assert torch.equal(torch.ops.liquidgemm.i8_gemm_scaled(at, bt, sat, sbt, out_dtype), got)
    ops.poll_status()


def _seeded_shapes(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < count:
        N = 256 * int(rng.integers(1, 40))
        K = 128 * int(rng.integers(1, 48))
        M = int(rng.integers(256, 6000))
        if (N // 256) * ((M + 255) // 256) >= 60 and M * K + N * K < 300_000_000:
            out.append((M, N, K))
    return out


@pytest.mark.parametrize("M,N,K", _seeded_shapes(16, seed=2024))
def test_seeded_shapes_against_cublaslt(ops, M, N, K):
    """Sixteen seeded shapes the pair kernel serves (ragged token counts, one to 47 k-steps, one to 39 channel
    blocks, partial last waves): int32 sums equal to cuBLASLt's exact INT8 GEMM, one after the other on one
    context."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    b = torch.randint(-128, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
    got = torch.ops.liquidgemm.wgmma_i8_gemm(a, b)
    assert torch.equal(got, torch._int_mm(a, b.t()))
    ops.poll_status()
