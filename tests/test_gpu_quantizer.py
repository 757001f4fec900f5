"""The device-side weight quantiser (``lq_quantize_weight`` through ``ops.quantize_weight_cuda`` and
``quant.quantize_weight`` on CUDA tensors) against the CPU oracle of the reference's quantiser
(liquidgemm/quant.py:61-100): codes, steps, offsets and the bits of the row scales, plus the tile blob it
writes against the separate prepack kernel.  Tolerance: none."""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O

pytestmark = pytest.mark.gpu


def _check(W_t: torch.Tensor, group: int, want_codes=True):
    from liquidgemm_b200 import ops
    want = O.quantize_weight(W_t.float().cpu().numpy(), group)
    qw, blob = ops.quantize_weight_cuda(W_t.cuda(), group, want_codes=want_codes, want_blob=True)
    assert (qw.N, qw.K) == (want.N, want.K)
    assert np.array_equal(qw.s1.cpu().numpy().view(np.uint32), want.s1.view(np.uint32)), "row scales"
    assert np.array_equal(qw.s_u8.cpu().numpy(), want.s_u8), "steps"
    assert np.array_equal(qw.offset_a.cpu().numpy(), want.offset_a), "offsets"
    if want_codes:
        assert np.array_equal(qw.qweight_u4.cpu().numpy(), want.qweight_u4), "codes"
    else:
        assert qw.qweight_u4 is None
    # the blob written by the quantiser == the prepack kernel's blob of the oracle's quantisation
    from tests.helpers import to_torch_qw
    ref_blob = ops.repack_rs_weight(to_torch_qw(want))
    assert torch.equal(blob, ref_blob), "tile blob"
    ops.poll_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("N,K", [(128, 128), (100, 256), (384, 1024), (1000, 2176)])
def test_quantiser_matches_the_oracle(N, K, group, dtype):
    W = torch.from_numpy(O.synth_weight(N, K, seed=N + K + group)).to(dtype)
    _check(W, group)


def test_golden_weights(golden):
    """The fixtures computed by the reference itself (Gaussian + outliers, heavy tails, degenerate rows)."""
    for case in golden.cases:
        W = golden.get(case, "W")
        g = int(golden.get(case, "group"))
        if W.shape[1] % 128 or g not in (64, 128):
            continue
        _check(torch.from_numpy(W.astype(np.float32)), g)


def test_degenerate_rows_and_extremes():
    """All-zero rows (scale floor 1e-12 / 119), constant rows (range 0 -> step 1), one huge outlier per row."""
    N, K = 256, 512
    W = torch.from_numpy(O.synth_weight(N, K, seed=5)).float()
    W[0] = 0.0
    W[1] = 0.37
    W[2] = -1e-30
    W[3, 17] = 1e4
    W[4] = torch.linspace(-1, 1, K)
    _check(W, 64)
    _check(W, 128, want_codes=False)


def test_full_size_layer_and_quantize_weight_dispatch():
    """A Llama-3.1-8B qkv-sized matrix through quant.quantize_weight on a CUDA tensor (which dispatches to
    the kernels), compared on every field."""
    from liquidgemm_b200.quant import quantize_weight
    N, K = 6144, 4096
    W = O.synth_weight(N, K, seed=0)
    want = O.quantize_weight(W.astype(np.float32), 64)
    qw = quantize_weight(torch.from_numpy(W).cuda(), 64)
    assert np.array_equal(qw.qweight_u4.cpu().numpy(), want.qweight_u4)
    assert np.array_equal(qw.s_u8.cpu().numpy(), want.s_u8)
    assert np.array_equal(qw.offset_a.cpu().numpy(), want.offset_a)
    assert np.array_equal(qw.s1.cpu().numpy().view(np.uint32), want.s1.view(np.uint32))


def test_shape_rules():
    from liquidgemm_b200 import ops
    with pytest.raises(RuntimeError):
        ops.quantize_weight_cuda(torch.zeros(8, 192, device="cuda", dtype=torch.float16), 64)      # K % 128
    with pytest.raises(RuntimeError):
        ops.quantize_weight_cuda(torch.zeros(8, 256, device="cuda", dtype=torch.float16), 32)      # group
