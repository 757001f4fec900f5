"""The CTA-pair prefill kernel (tcgen05.mma.cta_group::2, 256 channels x 192 tokens per tile) against the CPU
oracle, through the reference's operators (256 tokens and more, layers with whole 256-channel blocks).  Cases cover a single tile, ragged token counts, several waves of tiles, the
last partial wave (whole tiles, or long tiles split along k and summed through the workspace slots), every output type, the bias and the
multi-destination epilogue; full benchmark sizes are compared with cuBLASLt's exact INT8 GEMM."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import (LLAMA8B, assert_bits_equal, bits, expected_bits, random_lqq, random_tokens, to_torch_qw,
                           with_bias_f32)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _every_served_shape_takes_the_pair_kernel(monkeypatch):
    """The automatic dispatch sends a shape to the pair kernel only where it expects it to beat the tile kernel
    (large problems); the library reads this switch at every call, so the small cases below run on it too."""
    monkeypatch.setenv("LQ_PAIR_ALWAYS", "1")


def _acc(x, qw):
    return O.int_accumulate(x, O.dequantize_i8(qw))


# (M, N, K): one tile; ragged tokens; K with an odd number of k-steps; two full waves and a partial one
# (2 x 80 tiles on 74 pairs); one tile more than a wave
CASES = [(256, 256, 128), (257, 512, 1024), (383, 256, 2176), (385, 768, 512), (7680, 512, 512), (1000, 2560, 1536),
         (14400, 256, 384)]


@pytest.mark.parametrize("M,N,K", CASES)
def test_int32_accumulators_are_exact(ops, M, N, K):
    qw = random_lqq(N, K, 64, seed=N + K + M)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=M)
    w = ops.repack_rs_weight(tq)
    got = torch.ops.liquidgemm.w4a8_wgmma_rs(torch.from_numpy(x).cuda(), w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    assert np.array_equal(got.cpu().numpy(), _acc(x, qw))
    ops.poll_status()


@pytest.mark.parametrize("M,N,K", CASES[:6])
@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_fused_outputs_are_bit_exact(ops, M, N, K, out_dtype):
    qw = random_lqq(N, K, 64, seed=N + K)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M + 1)
    w = ops.repack_rs_weight(tq)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(torch.from_numpy(x).cuda(), w, tq.s_u8, tq.offset_a,
                                                 torch.from_numpy(ascale).cuda(), tq.s1, N, K, 64, out_dtype)
    # tolerance: none -- exact integer sums, two fp32 multiplies, one rounding to the output type
    assert_bits_equal(y, O.w4a8_matmul(x, ascale, qw), out_dtype, f"pair kernel {M}x{N}x{K}")
    ops.poll_status()


@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_bias_is_added_to_the_rounded_output(ops, out_dtype):
    M, N, K = 300, 512, 1024
    qw = random_lqq(N, K, 64, seed=8)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=2)
    rng = np.random.default_rng(4)
    dt = [torch.bfloat16, torch.float16, torch.float32][out_dtype]
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(dt)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    y = torch.ops.liquidgemm.w4a8_linear_bias(torch.from_numpy(x).cuda(), blob, torch.from_numpy(ascale).cuda(), tq.s1,
                                              bias.cuda(), N, K, out_dtype)
    want = with_bias_f32(O.w4a8_matmul(x, ascale, qw), bits(bias), out_dtype)
    assert_bits_equal(y, want, out_dtype, "pair kernel with bias")
    ops.poll_status()


@pytest.mark.parametrize("M,K", [(15360, 8192), (19918, 8192), (19918, 4096), (18816, 8192), (15644, 14336)])
def test_split_tail_and_clean_workspace(ops, M, K):
    """80 long tiles on 74 pairs: the six tiles of the last wave are cut along k between the pairs (four ranges
    each; 104 tiles, the last one ragged: thirty tiles in two ranges each, also with the shortest K that is cut;
    98 tiles: three ranges; 82 tiles of 112 k-steps, the last one ragged: seven ranges)
    and summed through the workspace planes, which the completing pair re-zeroes: a second call on the same
    cached workspace gives the same bits, and so does a decode call (which shares that workspace) afterwards."""
    N = 256
    qw = random_lqq(N, K, 64, seed=21)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=5)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    assert torch.equal(acc, ref)
    want = torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0)
    y1 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    y2 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y1, want) and torch.equal(y2, want)
    for rows in (slice(0, 16), slice(M - 16, M)):      # first tile and a tile of the split wave against the CPU oracle
        assert_bits_equal(y1[rows], O.w4a8_matmul(x[rows], ascale[rows], qw), 0, "rows against the oracle")
    y8 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt[:8].contiguous(), w, tq.s_u8, tq.offset_a, at[:8].contiguous(), tq.s1,
                                                  N, K, 64, 0)
    assert_bits_equal(y8, O.w4a8_matmul(x[:8], ascale[:8], qw), 0, "decode call after the pair kernel")
    ops.poll_status()


@pytest.mark.parametrize("out_dtype", [0, 2])
def test_cut_tiles_with_bias_and_two_destinations(ops, out_dtype):
    """The completing pair's epilogue in its other forms: bias, float32 outputs, and the gather-by-stores form
    (two destinations; 2-byte outputs go through the staged 16-byte stores, float32 through the direct ones)."""
    M, N, K = 19918, 256, 4096
    qw = random_lqq(N, K, 64, seed=17)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=9)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    rng = np.random.default_rng(6)
    dt = [torch.bfloat16, torch.float16, torch.float32][out_dtype]
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(dt)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    want = torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, out_dtype)
    y = torch.ops.liquidgemm.w4a8_linear_bias(xt, blob, at, tq.s1, bias.cuda(), N, K, out_dtype)
    rows = slice(M - 40, M)                                   # the ragged last tile is one of the cut ones
    assert_bits_equal(y[rows], with_bias_f32(O.w4a8_matmul(x[rows], ascale[rows], qw), bits(bias), out_dtype), out_dtype,
                      "cut tile with bias")
    if out_dtype == 2:
        assert torch.equal(y, want + bias.cuda())             # float32: one addition, exact against torch
    NF, col0 = 768, 256
    outs = [torch.full((M, NF), -1.0, dtype=dt, device="cuda") for _ in range(2)]
    ops.gemm_fused_scatter(xt, blob, at, tq.s1, [o.data_ptr() for o in outs], NF, col0, N, K, out_dtype)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[:, col0:col0 + N], want)
        assert bool((o[:, :col0] == -1).all()) and bool((o[:, col0 + N:] == -1).all())
    y8 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt[:8].contiguous(), ops.repack_rs_weight(tq), tq.s_u8, tq.offset_a,
                                                  at[:8].contiguous(), tq.s1, N, K, 64, 0)
    assert_bits_equal(y8, O.w4a8_matmul(x[:8], ascale[:8], qw), 0, "decode call on the shared workspace afterwards")
    ops.poll_status()


def test_multi_destination_epilogue(ops):
    """The gather-by-stores form on one GPU: two full-width destinations, this layer's block at a column offset."""
    M, N, K, NF, col0 = 600, 512, 1024, 1536, 512
    qw = random_lqq(N, K, 64, seed=13)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=3)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    outs = [torch.full((M, NF), -1.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    ops.gemm_fused_scatter(torch.from_numpy(x).cuda(), blob, torch.from_numpy(ascale).cuda(), tq.s1,
                           [o.data_ptr() for o in outs], NF, col0, N, K, 0, flag_ptrs=[flags.data_ptr()] * 2, flag_index=3)
    torch.cuda.synchronize()
    want = expected_bits(O.w4a8_matmul(x, ascale, qw), 0)
    for o in outs:
        assert np.array_equal(bits(o[:, col0:col0 + N]), want)
        assert bool((o[:, :col0] == -1).all()) and bool((o[:, col0 + N:] == -1).all())
    assert int(flags[3]) == 2 * ops.decode_grid(M, N, K)
    ops.poll_status()


def test_grouped_tile_order_with_a_cut_last_wave(ops):
    """Weights too large to stay in L2 are walked in groups of eight token tiles (here 4096 x 28672: 58.7 MB of
    4-bit tiles, 160 tiles of which the last twelve are cut in six k-ranges each)."""
    M, N, K = 1920, 4096, 28672
    qw = random_lqq(N, K, 64, seed=5)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=7)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    assert torch.equal(acc, ref)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0))
    rows = slice(M - 8, M)
    assert_bits_equal(y[rows], O.w4a8_matmul(x[rows], ascale[rows], qw), 0, "rows of a cut tile against the oracle")
    ops.poll_status()


@pytest.mark.parametrize("name,M", [("qkv", 2048), ("o", 512), ("gate_up", 2048), ("down", 8192)])
def test_full_size_against_exact_int8_gemm(ops, name, M):
    N, K = LLAMA8B[name]
    qw = random_lqq(N, K, 64, seed=3)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    assert torch.equal(acc, ref)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0))
    assert np.array_equal(acc[:16].cpu().numpy(), _acc(x[:16], qw))
    ops.poll_status()


def _seeded_shapes(count, seed):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(256, 5000)), 256 * int(rng.integers(1, 17)), 128 * int(rng.integers(1, 33)))
            for _ in range(count)]


@pytest.mark.parametrize("M,N,K", _seeded_shapes(10, seed=77))
def test_seeded_shapes_against_cublaslt(ops, M, N, K):
    """Ten seeded shapes (ragged token counts, 1..32 k-steps, 1..16 channel blocks; whole, partial and cut last
    waves as they fall): int32 sums equal to cuBLASLt's exact INT8 GEMM on the dequantised weights, and the fused
    bf16 output equal to the epilogue applied to them."""
    qw = random_lqq(N, K, 64, seed=M)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=N)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    assert torch.equal(acc, ref)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0))
    ops.poll_status()
