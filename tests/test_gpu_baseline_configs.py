"""The benchmark configurations end to end on the device, from fp16 data: product quantiser, device
prepack, per-token quantiser, linear -- every stage compared bit for bit with the CPU oracle.
Weights: randn * 0.02 with 0.1 % of the entries x20; activations randn, optionally 1 % hot channels x10."""

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


def _layer(ops, N, K, seed):
    """Quantise on the device with the product quantiser, check it against the oracle, build the blob."""
    from liquidgemm_b200.quant import quantize_weight
    W = O.synth_weight(N, K, seed=seed)
    want = O.quantize_weight(W.astype(np.float32), 64)
    qw = quantize_weight(torch.from_numpy(W).cuda().float(), group_size=64)
    assert np.array_equal(qw.qweight_u4.cpu().numpy(), want.qweight_u4)
    assert np.array_equal(qw.s_u8.cpu().numpy(), want.s_u8)
    assert np.array_equal(qw.offset_a.cpu().numpy(), want.offset_a)
    assert np.array_equal(qw.s1.cpu().numpy().view(np.uint32), want.s1.view(np.uint32))
    return {"rs": ops.repack_rs_weight(qw).reshape(-1), "s1": qw.s1, "s_u8": qw.s_u8, "offset_a": qw.offset_a,
            "N": N, "K": K}, want


def _check(ops, layer, want_qw, M, K, seed, hot, out_code):
    X = O.synth_activation(M, K, seed=seed, hot_channel_frac=hot)
    xq, sc = O.quantize_activation(X.astype(np.float32))
    dt = torch.float16 if out_code == 1 else torch.bfloat16
    y = ops.w4a8_linear(torch.from_numpy(X).cuda(), layer, out_dtype=dt)
    assert_bits_equal(y, O.w4a8_matmul(xq, sc, want_qw), out_code, f"M={M}")


def test_config0_qkv_m64_fp16(ops):
    """configs[0]: M = 64 tokens x the Llama-3.1-8B qkv projection (6144 x 4096), fp16 out."""
    layer, want = _layer(ops, 6144, 4096, seed=0)
    _check(ops, layer, want, 64, 4096, seed=1, hot=0.0, out_code=1)


@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_config1_decode_sweep_on_quantised_weights(ops, M):
    """configs[1] on a quantised (not code-space random) weight: the qkv shape, bf16 out."""
    layer, want = _layer(ops, 6144, 4096, seed=2)
    _check(ops, layer, want, M, 4096, seed=10 + M, hot=0.0, out_code=0)


@pytest.mark.parametrize("M", [32, 128])
def test_config2_decode_tiles(ops, M):
    layer, want = _layer(ops, 4096, 14336, seed=3)
    _check(ops, layer, want, M, 14336, seed=20 + M, hot=0.0, out_code=0)


def test_config3_prefill_with_hot_channels(ops):
    """configs[3]: prefill with 1 % of the input channels scaled x10 (M = 512 on the qkv shape)."""
    layer, want = _layer(ops, 6144, 4096, seed=4)
    _check(ops, layer, want, 512, 4096, seed=5, hot=0.01, out_code=0)
