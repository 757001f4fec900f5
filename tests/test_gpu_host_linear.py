"""The host-buffer linear (upload + quantise + W4A8 linear + download in one C call) against the oracle."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import random_lqq, to_torch_qw, assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from liquidgemm_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("M", [1, 3, 4, 5, 16, 40, 130])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_host_linear_matches_oracle(ops, M, dtype):
    N, K = 384, 1024
    qw = random_lqq(N, K, 64, seed=M)
    tq = to_torch_qw(qw)
    layer = {"rs": ops.repack_rs_weight(tq).reshape(-1), "s1": tq.s1, "N": N, "K": K}
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(dtype).pin_memory()
    y = ops.w4a8_linear_host(x, layer)
    torch.cuda.synchronize()
    assert y.dtype == dtype and tuple(y.shape) == (M, N) and not y.is_cuda
    xq, sc = O.quantize_activation(x.float().numpy())
    code = 0 if dtype == torch.bfloat16 else 1
    assert_bits_equal(y, O.w4a8_matmul(xq, sc, qw), code, f"host linear M={M}")


def test_host_linear_reuses_buffers_back_to_back(ops):
    """Two different layers and batch sizes through the same cached scratch on one stream."""
    outs, wants = [], []
    for i, (M, N, K) in enumerate([(2, 256, 512), (9, 640, 2048), (2, 256, 512)]):
        qw = random_lqq(N, K, 64, seed=10 + i)
        tq = to_torch_qw(qw)
        layer = {"rs": ops.repack_rs_weight(tq).reshape(-1), "s1": tq.s1, "N": N, "K": K}
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(i)).half().pin_memory()
        outs.append(ops.w4a8_linear_host(x, layer))
        xq, sc = O.quantize_activation(x.float().numpy())
        wants.append(O.w4a8_matmul(xq, sc, qw))
    torch.cuda.synchronize()
    for y, w in zip(outs, wants):
        assert_bits_equal(y, w, 1, "host linear back to back")


def test_host_linear_rejects_bad_arguments(ops):
    from liquidgemm_b200._lib import lib
    assert lib.lq_w4a8_linear_host(None, 1, None, None, None, 1, 1, 128, 128, None, 0, None, 0, None) == -1
    qw = random_lqq(128, 256, 64)
    tq = to_torch_qw(qw)
    layer = {"rs": ops.repack_rs_weight(tq).reshape(-1), "s1": tq.s1, "N": 128, "K": 256}
    with pytest.raises(RuntimeError):
        ops.w4a8_linear_host(torch.zeros(2, 128, dtype=torch.float16), layer)     # K mismatch
    with pytest.raises(RuntimeError):
        ops.w4a8_linear_host(torch.zeros(2, 256, dtype=torch.float16, device="cuda"), layer)   # not a host tensor
