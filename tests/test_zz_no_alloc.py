"""The workspace-free GEMV entry point (scratch inside the library image) against the regular entry
point: identical bits on two calls in a row.  Collected last on purpose: it must pass both alone and
after every other GPU test has used the library."""

import ctypes

import numpy as np
import pytest
import torch

from tests.helpers import random_lqq, random_tokens, to_torch_qw, bits

pytestmark = pytest.mark.gpu


def _call_static(lib, x, blob, sc, s1, out, code, M, N, K):
    return lib.lq_w4a8_gemv_blob_static(x.data_ptr(), blob.data_ptr(), sc.data_ptr(), s1.data_ptr(), out.data_ptr(),
                                        code, M, N, K, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 14336), (4, 1000, 2176), (8, 6144, 4096)])
def test_static_scratch_gemv_matches_workspace_gemv(M, N, K):
    from liquidgemm_b200 import ops
    from liquidgemm_b200._lib import lib
    qw = random_lqq(N, K, 64, seed=N + M)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    xn, scn = random_tokens(M, K, seed=M)
    x, sc = torch.from_numpy(xn).cuda(), torch.from_numpy(scn).cuda()
    want = ops.gemv_blob(x, blob, sc, tq.s1, N, K, 1)          # the existing entry point, caller workspace
    torch.cuda.synchronize()
    for call in range(2):                                      # two calls in a row on the same scratch
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        rc = _call_static(lib, x, blob, sc, tq.s1, got, 1, M, N, K)
        assert rc == 0, lib.lq_last_cuda_error()
        torch.cuda.synchronize()
        # tolerance: none -- both entry points run the same integer sums and the same two fp32 multiplies
        assert np.array_equal(bits(got), bits(want)), f"call {call}: static-scratch GEMV differs"
    assert lib.lq_poll_status(None) == 0


def test_static_scratch_gemv_rejects_sizes_beyond_its_limit():
    from liquidgemm_b200._lib import lib
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = z.data_ptr()
    assert lib.lq_w4a8_gemv_blob_static(p, p, p, p, p, 1, 9, 128, 128, None) == -2     # more than 8 tokens
    assert lib.lq_w4a8_gemv_blob_static(p, p, p, p, p, 1, 1, 128, 100, None) == -2     # K not a multiple of 128
    assert lib.lq_w4a8_gemv_blob_static(p + 4, p, p, p, p, 1, 1, 128, 128, None) == -1  # misaligned tokens
