"""The workspace-free GEMV entry point (scratch inside the library image) against the regular entry point
and against the CPU oracle: identical bits on two calls in a row.  Collected last on purpose: it must pass
both alone and after every other GPU test has used the library.

The entry point exists for callers that cannot get device memory at the point of the call (all of it
already assigned by a serving runtime's memory plan, or a call site where no allocator may be entered), so
the tests pass caller-owned inputs and outputs only and never hand it a workspace."""

import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import assert_bits_equal, bits, random_lqq, random_tokens, to_torch_qw

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _call_static(lib, x, blob, sc, s1, out, code, M, N, K, stream=None):
    st = (stream or torch.cuda.current_stream()).cuda_stream
    return lib.lq_w4a8_gemv_blob_static(x.data_ptr(), blob.data_ptr(), sc.data_ptr(), s1.data_ptr(), out.data_ptr(),
                                        code, M, N, K, st)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 14336), (4, 1000, 2176), (8, 6144, 4096)])
def test_static_scratch_gemv_matches_workspace_gemv_and_oracle(M, N, K):
    from liquidgemm_b200 import ops
    from liquidgemm_b200._lib import lib
    qw = random_lqq(N, K, 64, seed=N + M)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    xn, scn = random_tokens(M, K, seed=M)
    x, sc = torch.from_numpy(xn).cuda(), torch.from_numpy(scn).cuda()
    want = ops.gemv_blob(x, blob, sc, tq.s1, N, K, 1)          # the existing entry point, caller workspace
    oracle = O.w4a8_matmul(xn, scn, qw)
    torch.cuda.synchronize()
    for call in range(2):                                      # two calls in a row on the same scratch
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        rc = _call_static(lib, x, blob, sc, tq.s1, got, 1, M, N, K)
        assert rc == 0, lib.lq_last_cuda_error()
        torch.cuda.synchronize()
        # tolerance: none -- both entry points run the same integer sums and the same two fp32 multiplies
        assert np.array_equal(bits(got), bits(want)), f"call {call}: static-scratch GEMV differs"
        assert_bits_equal(got, oracle, 1, f"call {call} against the oracle")
    assert lib.lq_poll_status(None) == 0


def test_static_scratch_gemv_on_a_side_stream_and_after_a_reset():
    """A non-blocking stream (every torch side stream is one) and the reset call, whose memset must be
    ordered before the next kernel of the same stream."""
    from liquidgemm_b200 import ops
    from liquidgemm_b200._lib import lib
    M, N, K = 2, 2048, 4096
    qw = random_lqq(N, K, 64, seed=3)
    tq = to_torch_qw(qw)
    blob = ops.repack_rs_weight(tq).reshape(-1)
    xn, scn = random_tokens(M, K, seed=9)
    x, sc = torch.from_numpy(xn).cuda(), torch.from_numpy(scn).cuda()
    oracle = O.w4a8_matmul(xn, scn, qw)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    got = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    with torch.cuda.stream(side):
        assert _call_static(lib, x, blob, sc, tq.s1, got, 0, M, N, K, side) == 0
        assert lib.lq_w4a8_gemv_blob_static_reset(side.cuda_stream) == 0
        assert _call_static(lib, x, blob, sc, tq.s1, got, 0, M, N, K, side) == 0
    side.synchronize()
    assert_bits_equal(got, oracle, 0, "side stream + reset")
    assert lib.lq_poll_status(None) == 0


def test_first_call_of_a_fresh_process_on_a_side_stream():
    """The one-time set-up must leave the array cleared for a kernel on any stream: a new process makes its
    very first call on a non-blocking stream and compares with the oracle."""
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        import numpy as np, torch
        from oracle import lqq_oracle as O
        from tests.helpers import assert_bits_equal, random_lqq, random_tokens, to_torch_qw
        from liquidgemm_b200 import ops
        from liquidgemm_b200._lib import lib
        M, N, K = 3, 4096, 4096
        qw = random_lqq(N, K, 64, seed=11); tq = to_torch_qw(qw)
        blob = ops.repack_rs_weight(tq).reshape(-1)
        xn, scn = random_tokens(M, K, seed=12)
        x, sc = torch.from_numpy(xn).cuda(), torch.from_numpy(scn).cuda()
        got = torch.empty((M, N), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            rc = lib.lq_w4a8_gemv_blob_static(x.data_ptr(), blob.data_ptr(), sc.data_ptr(), tq.s1.data_ptr(),
                                              got.data_ptr(), 1, M, N, K, side.cuda_stream)
        assert rc == 0, lib.lq_last_cuda_error()
        side.synchronize()
        assert_bits_equal(got, O.w4a8_matmul(xn, scn, qw), 1, "first call on a side stream")
        assert lib.lq_poll_status(None) == 0
        print("ok")
        """ % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-2000:]


def test_static_scratch_gemv_rejects_sizes_beyond_its_limit():
    from liquidgemm_b200._lib import lib
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = z.data_ptr()
    assert lib.lq_w4a8_gemv_blob_static(p, p, p, p, p, 1, 9, 128, 128, None) == -2     # more than 8 tokens
    assert lib.lq_w4a8_gemv_blob_static(p, p, p, p, p, 1, 1, 128, 100, None) == -2     # K not a multiple of 128
    assert lib.lq_w4a8_gemv_blob_static(p + 4, p, p, p, p, 1, 1, 128, 128, None) == -1  # misaligned tokens
