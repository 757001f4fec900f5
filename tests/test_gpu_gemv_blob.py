"""Decode GEMV fed from the tile blob (M <= 8): bit-exact against the CPU oracle, through the C ABI."""

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
    blob = ops.repack_rs_weight(tq)
    return ops.gemv_blob(torch.from_numpy(x).cuda(), blob.reshape(-1), torch.from_numpy(ascale).cuda(), tq.s1,
                         qw.N, qw.K, out_dtype)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("out_dtype", [0, 1, 2])
def test_blob_gemv_small(ops, M, out_dtype):
    qw = random_lqq(512, 4096, 64, seed=M)
    x, ascale = random_tokens(M, 4096, seed=100 + M)
    got = _run(ops, qw, x, ascale, out_dtype)
    assert got.shape == (M, 512)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), out_dtype, f"blob gemv M={M}")


@pytest.mark.parametrize("N,K", [(200, 1152), (24, 128), (1000, 2176), (130, 14336), (128, 128), (3000, 256)])
@pytest.mark.parametrize("M", [1, 4, 7])
def test_blob_gemv_ragged_shapes(ops, N, K, M):
    """N not a multiple of 128 (padded rows), fewer tiles than CTAs, one k-tile, long K."""
    qw = random_lqq(N, K, 64, seed=N + K)
    x, ascale = random_tokens(M, K, seed=M)
    got = _run(ops, qw, x, ascale, 0)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 0, f"blob gemv {N}x{K} M={M}")


@pytest.mark.parametrize("name", ["qkv", "gate_up", "down"])
@pytest.mark.parametrize("M", [1, 4, 8])
def test_blob_gemv_llama_shapes(ops, name, M):
    N, K = LLAMA8B[name]
    qw = random_lqq(N, K, 64, seed=7)
    x, ascale = random_tokens(M, K, seed=M)
    got = _run(ops, qw, x, ascale, 0)
    assert_bits_equal(got, O.w4a8_matmul(x, ascale, qw), 0, f"blob gemv {name} M={M}")


def test_blob_gemv_leaves_workspace_zero_and_repeats(ops):
    """Stream-K partial sums go through the shared zero workspace: it must be clean after every call,
    and a second call must give the same bits."""
    from liquidgemm_b200._lib import lib
    qw = random_lqq(4096, 14336, 64, seed=3)
    x, ascale = random_tokens(4, 14336, seed=4)
    want = O.w4a8_matmul(x, ascale, qw)
    for _ in range(3):
        got = _run(ops, qw, x, ascale, 1)
        assert_bits_equal(got, want, 1, "blob gemv repeat")
    torch.cuda.synchronize()
    ws = ops._workspace(lib.lq_gemv_blob_workspace_bytes(), torch.device("cuda", torch.cuda.current_device()))
    assert int(ws.count_nonzero()) == 0
    assert lib.lq_poll_status(None) == 0


def test_blob_gemv_rejects_bad_arguments(ops):
    from liquidgemm_b200._lib import lib
    qw = random_lqq(128, 256, 64)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    x = torch.zeros(9, 256, dtype=torch.int8, device="cuda")
    a = torch.ones(9, device="cuda")
    with pytest.raises(RuntimeError):
        ops.gemv_blob(x, blob, a, tq.s1, 128, 256, 0)           # M > 8
    y = torch.empty(1, 128, dtype=torch.float32, device="cuda")
    rc = lib.lq_w4a8_gemv_blob(x.data_ptr(), blob.data_ptr(), a.data_ptr(), tq.s1.data_ptr(), y.data_ptr(), 2,
                               1, 128, 256, None, 0, None)
    assert rc == -3                                              # no workspace
    rc = lib.lq_w4a8_gemv_blob(x.data_ptr() + 1, blob.data_ptr(), a.data_ptr(), tq.s1.data_ptr(), y.data_ptr(), 2,
                               1, 128, 256, y.data_ptr(), 1 << 30, None)
    assert rc == -1                                              # misaligned tokens
