"""The route for very large token counts: the tile blob is unpacked to INT8 once (scratch workspace) and the
INT8 x INT8 pair kernel does the GEMM.  The limit is lowered here so that modest sizes take the route; results are
compared with the CPU oracle, with cuBLASLt's exact INT8 GEMM on the dequantised weights, and with the same call on
the W4 kernels (route switched off)."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import (assert_bits_equal, bits, random_lqq, random_tokens, to_torch_qw, with_bias_f32)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _route_from_512_tokens(monkeypatch):
    monkeypatch.setenv("LQ_UNPACK_I8_MIN_M", "512")


# (M, N, K): 60 tiles of 256 x 256 or more, K below 8192; ragged tokens; one k-step
CASES = [(2048, 2560, 512), (1999, 3072, 1024), (4096, 1024, 128), (1024, 6144, 4096)]


@pytest.mark.parametrize("M,N,K", CASES)
def test_route_is_taken_and_exact(ops, M, N, K, monkeypatch):
    from liquidgemm_b200._lib import lib
    assert lib.lq_gemm_workspace_kind(M, N, K, 0) == 1 and lib.lq_gemm_workspace_bytes(M, N, K, 0) == N * K
    assert lib.lq_gemm_launches(M, N, K, 0) == 2
    qw = random_lqq(N, K, 64, seed=N + K)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=M)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    w = ops.repack_rs_weight(tq)
    ref = torch._int_mm(xt, ops.dequant_weight_i8(tq).t())
    acc = torch.ops.liquidgemm.w4a8_wgmma_rs(xt, w, tq.s_u8, tq.s_u8, tq.offset_a, N, K, 64, True)
    assert torch.equal(acc, ref)
    rows = slice(M - 7, M)
    assert np.array_equal(acc[rows].cpu().numpy(), O.int_accumulate(x[rows], O.dequantize_i8(qw)))
    outs = {}
    for out_dtype in (0, 1, 2):
        y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, out_dtype)
        # tolerance: none -- exact integer sums, two fp32 multiplies, one rounding to the output type
        assert_bits_equal(y[rows], O.w4a8_matmul(x[rows], ascale[rows], qw), out_dtype, "unpack route")
        assert torch.equal(y, torch.ops.liquidgemm.scale_epilogue(ref, at, tq.s1, out_dtype))
        outs[out_dtype] = y
    monkeypatch.setenv("LQ_UNPACK_I8_MIN_M", "0")          # the same calls on the W4 kernels
    for out_dtype in (0, 1, 2):
        y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt, w, tq.s_u8, tq.offset_a, at, tq.s1, N, K, 64, out_dtype)
        assert torch.equal(y, outs[out_dtype])
    ops.poll_status()


@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_bias_is_added_to_the_rounded_output(ops, out_dtype):
    M, N, K = 2048, 2560, 512
    qw = random_lqq(N, K, 64, seed=8)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=2)
    rng = np.random.default_rng(4)
    dt = [torch.bfloat16, torch.float16, torch.float32][out_dtype]
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(dt)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    y = torch.ops.liquidgemm.w4a8_linear_bias(torch.from_numpy(x).cuda(), blob, torch.from_numpy(ascale).cuda(), tq.s1,
                                              bias.cuda(), N, K, out_dtype)
    rows = slice(M - 16, M)
    want = with_bias_f32(O.w4a8_matmul(x[rows], ascale[rows], qw), bits(bias), out_dtype)
    assert_bits_equal(y[rows], want, out_dtype, "unpack route with bias")
    ops.poll_status()


def test_gather_by_stores_keeps_its_own_route_and_workspace(ops):
    """The multi-destination form has no unpack route: for a shape whose single-destination call takes it, the
    scatter call runs the W4 kernels on the zeroed reduction workspace (kind from lq_scatter_workspace_kind) and
    leaves it zero: the same call twice and a decode call afterwards are exact."""
    from liquidgemm_b200._lib import lib
    M, N, K, NF, col0 = 3200, 2560, 512, 5120, 2560
    assert lib.lq_gemm_workspace_kind(M, N, K, 0) == 1
    assert lib.lq_scatter_workspace_kind(M, N, K) in (0, 2)
    qw = random_lqq(N, K, 64, seed=3)
    tq = to_torch_qw(qw)
    x, ascale = random_tokens(M, K, seed=4)
    xt, at = torch.from_numpy(x).cuda(), torch.from_numpy(ascale).cuda()
    blob = ops.repack_rs_weight(tq).reshape(-1)
    want = torch.ops.liquidgemm.scale_epilogue(torch._int_mm(xt, ops.dequant_weight_i8(tq).t()), at, tq.s1, 0)
    for _ in range(2):
        outs = [torch.full((M, NF), -1.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        ops.gemm_fused_scatter(xt, blob, at, tq.s1, [o.data_ptr() for o in outs], NF, col0, N, K, 0)
        torch.cuda.synchronize()
        for o in outs:
            assert torch.equal(o[:, col0:col0 + N], want)
            assert bool((o[:, :col0] == -1).all())
    y8 = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(xt[:8].contiguous(), ops.repack_rs_weight(tq), tq.s_u8, tq.offset_a,
                                                  at[:8].contiguous(), tq.s1, N, K, 64, 0)
    assert_bits_equal(y8, O.w4a8_matmul(x[:8], ascale[:8], qw), 0, "decode call on the shared workspace afterwards")
    ops.poll_status()
