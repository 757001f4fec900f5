"""Tensor-core W4A8 GEMM parity: exact int32 accumulators and bit-exact fused outputs."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import LLAMA8B, random_lqq, random_tokens, to_torch_qw, assert_bits_equal

pytestmark = pytest.mark.gpu

# (M, N, K) of the reference's tests/test_wgmma.py:14
SHAPES = [(128, 512, 4096), (256, 256, 512), (128, 6144, 4096), (512, 4096, 14336)]


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


def _acc(x, qw):
    return O.int_accumulate(x, O.dequantize_i8(qw))


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_i8_gemm_exact(ops, M, N, K):
    """Plain INT8 tensor-core GEMM (reference: wgmma_i8_gemm vs torch._int_mm, tests/test_wgmma.py:17-25)."""
    rng = np.random.default_rng(M + N + K)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    got = torch.ops.liquidgemm.wgmma_i8_gemm(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    assert np.array_equal(got.cpu().numpy(), O.int_accumulate(a, b))


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("packed", [False, True])
def test_w4a8_int32_exact(ops, M, N, K, packed):
    """int32 accumulators from the tile blob and from the plain nibble layout
    (reference tests/test_wgmma.py:44-64)."""
    qw = random_lqq(N, K, 64, seed=N + K)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=M)
    xt = torch.from_numpy(x).cuda()
    if packed:
        w, spack = ops.repack_rs_weight(tq), ops.build_rs_scale_pack(tq)
    else:
        from liquidgemm_b200.pack import pack_nibbles
        w, spack = pack_nibbles(tq.qweight_u4).contiguous(), tq.s_u8
    got = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, spack, tq.s_u8, tq.offset_a, N, K, 64, packed)
    assert got.dtype == torch.int32 and got.shape == (M, N)
    assert np.array_equal(got.cpu().numpy(), _acc(x, qw))


@pytest.mark.parametrize("M,N,K", SHAPES[:3])
def test_w4a8_ss_entry_point(ops, M, N, K):
    """torch.ops.liquidgemm.w4a8_wgmma keeps its signature (reference tests/test_wgmma.py:28-41)."""
    from liquidgemm_b200.pack import pack_nibbles
    qw = random_lqq(N, K, 64, seed=5)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=M)
    got = torch.ops.liquidgemm.w4a8_wgmma(torch.from_numpy(x).cuda(), pack_nibbles(tq.qweight_u4).contiguous(),
                                          tq.s_u8, tq.offset_a, N, K, 64)
    assert np.array_equal(got.cpu().numpy(), _acc(x, qw))


@pytest.mark.parametrize("M", [1, 15, 17, 30, 33, 100, 129, 200, 257, 300])
def test_any_token_count(ops, M):
    """Ragged token counts: TMA zero-fills the rows past M (reference pads with a copy,
    tests/test_wgmma.py:67-83)."""
    N, K = 512, 4096
    qw = random_lqq(N, K, 64, seed=M)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=M + 1)
    got = torch.ops.liquidgemm.w4a8_wgmma_rs(torch.from_numpy(x).cuda(), ops.repack_rs_weight(tq), tq.s_u8,
                                             tq.s_u8, tq.offset_a, N, K, 64, True)
    assert got.shape == (M, N)
    assert np.array_equal(got.cpu().numpy(), _acc(x, qw))


@pytest.mark.parametrize("N", [64, 192, 320])
def test_output_channels_not_multiple_of_tile(ops, N):
    """N % 64 == 0 is the reference contract; the 128-row tile masks the missing rows."""
    K, M = 1024, 48
    qw = random_lqq(N, K, 64, seed=N)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=2)
    got = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(torch.from_numpy(x).cuda(), ops.repack_rs_weight(tq), tq.s_u8,
                                                   tq.offset_a, torch.from_numpy(ascale).cuda(), tq.s1, N, K, 64, 0)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 0, f"N={N}")


@pytest.mark.parametrize("M", [1, 64, 100, 256])
@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_fused_equals_unfused_and_oracle(ops, M, out_dtype):
    """N=512, K=14336 forces split-K inside the fused op (reference tests/test_wgmma.py:86-104)."""
    N, K = 512, 14336
    qw = random_lqq(N, K, 64, seed=9)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    ref = torch.ops.liquidgemm.scale_epilogue(acc.contiguous(), at, tq.s1, out_dtype)
    got = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, out_dtype)
    assert got.shape == (M, N)
    assert torch.equal(got, ref), "fused path diverged from the unfused pipeline"
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), out_dtype, "fused vs oracle")


@pytest.mark.parametrize("S", [-1, 0, 1, 2, 4, 8, 16])
@pytest.mark.parametrize("M", [32, 64, 128])
def test_explicit_splitk_is_exact(ops, M, S):
    """Split-K sweep of the decode-tile configuration (0 = automatic, -1 = persistent stream-K): any setting gives the same bits."""
    N, K = 256, 14336
    qw = random_lqq(N, K, 64, seed=S + 2)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    w = ops.repack_rs_weight(tq).reshape(-1)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    acc = ops.gemm_i32(xt, w, N, K, splitk=S)
    assert np.array_equal(acc.cpu().numpy(), _acc(x, qw))
    y = ops.gemm_fused(xt, w, at, tq.s1, N, K, 0, splitk=S)
    assert_bits_equal(y, O.w4a8_matmul(x, ascale, qw), 0, f"S={S}")


def test_group_128_blob(ops):
    """group_size 128 shares one (step, offset) pair between both halves of a 128-k tile."""
    N, K, M = 256, 1024, 40
    qw = random_lqq(N, K, 128, seed=1)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=3)
    acc = ops.gemm_i32(torch.from_numpy(x).cuda(), ops.repack_rs_weight(tq).reshape(-1), N, K)
    assert np.array_equal(acc.cpu().numpy(), _acc(x, qw))


def test_extreme_values_do_not_overflow_lanes(ops):
    """All codes 15 with step 16 and offset 15 (u = 255) against tokens of +-127."""
    N, K, M = 128, 2048, 64
    qw = O.LQQWeight(np.full((N, K), 15, np.uint8), np.full((N, K // 64), 16, np.uint8),
                     np.full((N, K // 64), 15, np.uint8), np.ones(N, np.float32), 64)
    x = np.full((M, K), 127, np.int8)
    x[::2] = -127
    tq = to_torch_qw(qw)
    acc = ops.gemm_i32(torch.from_numpy(x).cuda(), ops.repack_rs_weight(tq).reshape(-1), N, K)
    assert np.array_equal(acc.cpu().numpy(), _acc(x, qw))


def test_unfused_pipeline_and_v1_large_m(ops):
    """w4a8_linear_unfused (dequant -> INT8 GEMM -> epilogue) and w4a8_gemm for M > 16
    (reference tests/test_kernel_gemm.py:21-64)."""
    N, K, M = 4096, 4096, 64
    W = O.synth_weight(N, K, seed=0)
    X = O.synth_activation(M, K, seed=1)
    qw = O.quantize_weight(W.astype(np.float32), 64)
    x, ascale = O.quantize_activation(X.astype(np.float32))
    tq = to_torch_qw(qw)
    y, acc = ops.w4a8_linear_unfused(torch.from_numpy(x), torch.from_numpy(ascale), tq, out_dtype=torch.float32)
    assert np.array_equal(acc.cpu().numpy(), _acc(x, qw))
    assert_bits_equal(y, O.w4a8_matmul(x, ascale, qw), 2, "unfused")
    y1 = ops.w4a8_gemm(torch.from_numpy(x), torch.from_numpy(ascale), tq, out_dtype=torch.float32)
    assert_bits_equal(y1, O.w4a8_matmul(x, ascale, qw), 2, "v1")
    yr = ops.w4a8_gemm_rs(torch.from_numpy(x), torch.from_numpy(ascale), tq, ops.repack_rs_weight(tq),
                          out_dtype=torch.float16)
    assert_bits_equal(yr, O.w4a8_matmul(x, ascale, qw), 1, "gemm_rs")
    y_fp = X.astype(np.float32) @ W.astype(np.float32).T
    cos = float((y.cpu().numpy() * y_fp).sum() / np.linalg.norm(y.cpu().numpy()) / np.linalg.norm(y_fp))
    # 0.1 % of the weights are x20 outliers, which stretch the per-channel scale: the 4-bit
    # reconstruction then tracks the fp product a little less closely than the reference's
    # outlier-free test data (cos > 0.99 there, tests/test_kernel_gemm.py:43)
    assert cos > 0.98


def test_i8_scaled_epilogue(ops):
    rng = np.random.default_rng(0)
    M, N, K = 77, 384, 1024
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    sa = (rng.random(M, dtype=np.float32) * 0.02 + 0.01).astype(np.float32)
    sb = (rng.random(N, dtype=np.float32) * 0.001 + 1e-5).astype(np.float32)
    got = torch.ops.liquidgemm.i8_gemm_scaled(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(),
                                              torch.from_numpy(sa).cuda(), torch.from_numpy(sb).cuda(), 0)
    assert_bits_equal(got, O.scale_f32(O.int_accumulate(a, b), sa, sb), 0, "i8 scaled")


@pytest.mark.parametrize("name,M", [("qkv", 2048), ("gate_up", 512), ("down", 2048), ("gate_up", 8192)])
def test_full_size_prefill_properties(ops, name, M):
    """Full benchmark sizes: (i) int32 result equals cuBLASLt's exact INT8 GEMM on the dequantised
    weights (the reference's own secondary oracle, liquidgemm/ops.py:106-113), (ii) the fused output
    equals the epilogue applied to those accumulators, (iii) run-to-run determinism."""
    N, K = LLAMA8B[name]
    qw = random_lqq(N, K, 64, seed=3)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    w_i8 = ops.dequant_weight_i8(tq)
    ref = torch._int_mm(xt, w_i8.t())
    assert torch.equal(acc, ref)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0))
    y2 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, y2)
    # a slice against the CPU oracle
    rows = slice(0, min(M, 16))
    assert np.array_equal(acc[rows].cpu().numpy(), _acc(x[rows], qw))


def test_device_status_word_is_clean(ops):
    from liquidgemm_b200._lib import lib
    assert lib.lq_poll_status(torch.cuda.current_stream().cuda_stream) == 0


def test_workspace_is_left_clean(ops):
    """Stream-K leaves its reduction workspace all-zero, so back-to-back calls stay exact."""
    N, K, M = 384, 14336, 24
    qw = random_lqq(N, K, 64, seed=4)
    tq = to_torch_qw(qw)
    x, _ = random_tokens(M, K, seed=5)
    xt = torch.from_numpy(x).cuda()
    w = ops.repack_rs_weight(tq).reshape(-1)
    want = _acc(x, qw)
    for _ in range(3):
        assert np.array_equal(ops.gemm_i32(xt, w, N, K, splitk=-1).cpu().numpy(), want)
    for ws in ops._WORKSPACES.values():
        assert int(ws.count_nonzero()) == 0


@pytest.mark.parametrize("M", [200, 2048])
@pytest.mark.parametrize("S", [-1, 0, 1, 3])
def test_prefill_scheduling_modes_are_exact(ops, M, S):
    """Persistent kernel: stream-K, whole tiles and a fixed split give the same bits (M > 128)."""
    N, K = 640, 2048
    qw = random_lqq(N, K, 64, seed=S + 7)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    w = ops.repack_rs_weight(tq).reshape(-1)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    assert np.array_equal(ops.gemm_i32(xt, w, N, K, splitk=S).cpu().numpy(), _acc(x, qw))
    y = ops.gemm_fused(xt, w, at, tq.s1, N, K, 1, splitk=S)
    assert_bits_equal(y, O.w4a8_matmul(x, ascale, qw), 1, f"M={M} S={S}")


@pytest.mark.parametrize("M", [1, 4, 9, 16])
def test_scatter_epilogue_writes_every_destination(ops, M):
    """The gather-by-stores epilogue: the [M, N] block lands at the right columns of several wider
    matrices (here two local buffers stand for this GPU's and a peer's output) and nowhere else."""
    N, K, LD, COL0 = 384, 2048, 1000, 256
    qw = random_lqq(N, K, 64, seed=40 + M)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    x, ascale = random_tokens(M, K, seed=M)
    outs = [torch.full((M, LD), -7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    ops.gemm_fused_scatter(torch.from_numpy(x).cuda(), blob, torch.from_numpy(ascale).cuda(), tq.s1,
                           [o.data_ptr() for o in outs], LD, COL0, N, K, 0)
    torch.cuda.synchronize()
    want = O.w4a8_matmul(x, ascale, qw)
    for o in outs:
        assert_bits_equal(o[:, COL0:COL0 + N].contiguous(), want, 0, f"scatter M={M}")
        assert bool((o[:, :COL0] == -7.0).all()) and bool((o[:, COL0 + N:] == -7.0).all())


@pytest.mark.parametrize("M", [2, 12])
def test_scatter_epilogue_signals_and_waits(ops, M):
    """Kernel-side ordering of the gather-by-stores epilogue on one GPU: launch k adds its CTA count to
    flag word k, launch k+1 waits for that count before it reads its tokens."""
    from liquidgemm_b200._lib import lib
    N, K = 640, 2048
    qw = random_lqq(N, K, 64, seed=60 + M)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    x, ascale = random_tokens(M, K, seed=M)
    xd, sd = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    grid = ops.decode_grid(M, N, K)
    assert grid > 0
    outs = [torch.zeros((M, N), dtype=torch.float16, device="cuda") for _ in range(3)]
    for k, o in enumerate(outs):
        ops.gemm_fused_scatter(xd, blob, sd, tq.s1, [o.data_ptr()], N, 0, N, K, 1, flag_ptrs=[flags.data_ptr()],
                               flag_index=k, wait_ptr=(flags.data_ptr() + 4 * (k - 1)) if k else None,
                               wait_value=grid if k else 0)
    torch.cuda.synchronize()
    want = O.w4a8_matmul(x, ascale, qw)
    for o in outs:
        assert_bits_equal(o, want, 1, f"scatter+sync M={M}")
    assert flags[:3].tolist() == [grid] * 3 and int(flags[3:].abs().sum()) == 0
    assert lib.lq_poll_status(None) == 0


def test_peer_wait_gives_up_and_reports(ops):
    """A flag that nothing sets: the kernel stops waiting after its limit, records status 303 and still
    finishes, and the context stays usable (LQ_ERR_TIMEOUT from lq_poll_status, site in the error text)."""
    from liquidgemm_b200._lib import lib
    N, K, M = 128, 256, 1
    qw = random_lqq(N, K, 64, seed=77)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    x, ascale = random_tokens(M, K, seed=3)
    xd, sd = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    ops.gemm_fused_scatter(xd, blob, sd, tq.s1, [out.data_ptr()], N, 0, N, K, 1, wait_ptr=flags.data_ptr(),
                           wait_value=5)
    torch.cuda.synchronize()
    assert lib.lq_poll_status(None) == -6                    # LQ_ERR_TIMEOUT
    assert b"site 303" in lib.lq_last_cuda_error()
    assert lib.lq_poll_status(None) == 0                     # reading clears it
    # the launch itself completed (it went on after the limit), and the next call works normally
    assert_bits_equal(out, O.w4a8_matmul(x, ascale, qw), 1, "after timeout")
    got = ops.gemm_fused(xd, blob, sd, tq.s1, N, K, 1)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 1, "next call")


@pytest.mark.parametrize("name,M", [("o", 512), ("qkv", 384), ("o", 384), ("qkv", 512), ("o", 257)])
def test_medium_token_counts(ops, name, M):
    """A few hundred tokens on the small matrices, where the dispatch switches between 64-token tiles in one wave
    and 128-token tiles cut along k: int32 sums equal to cuBLASLt's exact INT8 GEMM on the dequantised weights,
    fused output equal to the epilogue applied to them, last rows against the CPU oracle."""
    N, K = LLAMA8B[name]
    qw = random_lqq(N, K, 64, seed=M)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M + 1)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t()) if M > 16 else None
    assert torch.equal(acc, ref)
    y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, 0)
    assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, 0))
    rows = slice(M - 5, M)
    assert_bits_equal(y[rows], O.w4a8_matmul(x[rows], ascale[rows], qw), 0, "medium token counts")
    ops.poll_status()
