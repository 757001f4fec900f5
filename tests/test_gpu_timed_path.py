"""Parity of the exact routes the benchmark times, at the benchmark's sizes.

Every case goes through ``torch.ops.liquidgemm.w4a8_wgmma_rs_fused`` on the tile blob with the automatic
dispatch (what ``bench.py`` and the plugin call), so whichever kernel the dispatch picks for (shape, M) --
streaming dp4a GEMV, decode tensor-core kernel with its split-K join, tile kernel -- is the one compared
with the oracle.  Shape x M grid of the reference's own kernel test (tests/test_kernel_gemm.py:17-18:
the four Llama-3.1-8B linears x M in {1, 4, 16, 64, 256}) widened to the decode sweep of the benchmark,
plus the Llama-3-70B shapes as one of eight column shards (K = 28672 is the longest reduction and the
largest biased partial sum in the 64-bit split-K join).  bf16 out, tolerance none.
"""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import LLAMA8B, assert_bits_equal, random_lqq, random_tokens, to_torch_qw

pytestmark = pytest.mark.gpu

SHARDS_70B = {"qkv/8": (1280, 8192), "o/8": (1024, 8192), "gate_up/8": (7168, 8192), "down/8": (1024, 28672)}


def _run(N, K, Ms, seed):
    from liquidgemm_b200 import ops
    qw = random_lqq(N, K, 64, seed=seed)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    q_hat = O.dequantize_i8(qw)
    toks = [random_tokens(M, K, seed=100 + M) for M in Ms]
    # one exact CPU accumulation for all token counts together
    acc = O.int_accumulate(np.concatenate([t[0] for t in toks], axis=0), q_hat)
    row = 0
    for M, (xn, scn) in zip(Ms, toks):
        x, sc = torch.from_numpy(xn).cuda(), torch.from_numpy(scn).cuda()
        for rep in range(2):       # twice: the second call meets the reduction workspace the first one left
            y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(x, blob, tq.s_u8, tq.offset_a, sc, tq.s1, N, K, 64, 0)
            assert_bits_equal(y, O.scale_f32(acc[row:row + M], scn, qw.s1), 0, f"{N}x{K} M={M} call {rep}")
        row += M
    from liquidgemm_b200._lib import lib
    assert lib.lq_poll_status(None) == 0


@pytest.mark.parametrize("name", list(LLAMA8B))
def test_llama8b_shapes_decode_and_tile_range(name):
    N, K = LLAMA8B[name]
    _run(N, K, (1, 2, 3, 4, 5, 8, 16, 32, 64, 128), seed=len(name))


@pytest.mark.parametrize("name", list(SHARDS_70B))
def test_llama70b_shards(name):
    N, K = SHARDS_70B[name]
    _run(N, K, (1, 4, 8, 16, 64), seed=7 + len(name))


def test_int32_accumulators_at_the_longest_reduction():
    """K = 28672 with all-extreme operands: |acc| reaches K * 127 * 128, the bound the join's bias assumes."""
    from liquidgemm_b200 import ops
    N, K = 256, 28672
    codes = np.zeros((N, K), np.uint8)
    step = np.ones((N, K // 64), np.uint8)
    off = np.zeros((N, K // 64), np.uint8)             # code*1 + 0 - 128 = -128 everywhere
    codes[N // 2:] = 15
    step[N // 2:] = 16
    off[N // 2:] = 15                                   # 15*16 + 15 - 128 = +127 in the second half
    qw = O.LQQWeight(codes, step, off, np.full(N, 1e-3, np.float32), 64)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    for M in (1, 8, 16):
        xn = np.full((M, K), -127, np.int8)
        xn[1::2] = 127
        acc = ops.gemm_i32(torch.from_numpy(xn).cuda(), blob, N, K).cpu().numpy()
        assert np.array_equal(acc, O.int_accumulate(xn, O.dequantize_i8(qw)))
        assert abs(int(acc[0, 0])) == K * 127 * 128
        sc = torch.full((M,), 1e-2, device="cuda")
        y = ops.gemm_fused(torch.from_numpy(xn).cuda(), blob, sc, tq.s1, N, K, 2)
        assert_bits_equal(y, O.scale_f32(acc, sc.cpu().numpy(), qw.s1), 2, f"extremes M={M}")
