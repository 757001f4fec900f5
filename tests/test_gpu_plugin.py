"""The plugin's load-time and forward logic on the device, in every mode, against the CPU oracle.

``prepare_layer`` + ``apply_layer`` are what ``LiquidGemmLinearMethod.process_weights_after_loading`` and
``.apply`` run (reference liquidgemm/vllm_plugin.py:136-206); here they are driven on a ``torch.nn.Module``
holding a bf16 / fp16 weight, as vLLM's loader leaves it.  Expected values: the oracle's quantiser on the
same weight, the oracle's activation quantiser on the same tokens, ``w4a8_matmul``, cast to the
activation dtype, then the bias added in that dtype (the reference's order).  Tolerance: none.
"""

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.helpers import assert_bits_equal, bits, with_bias_f32

pytestmark = pytest.mark.gpu

_CODE = {torch.bfloat16: 0, torch.float16: 1}


def _module(N, K, dtype, seed):
    W = O.synth_weight(N, K, seed=seed)                       # fp16 values
    lin = torch.nn.Module()
    lin.weight = torch.nn.Parameter(torch.from_numpy(W).to(dtype).cuda(), requires_grad=False)
    w_f32 = lin.weight.data.float().cpu().numpy()             # what the quantiser sees after the dtype cast
    return lin, O.quantize_weight(w_f32, 64)


def _expected(x: torch.Tensor, want_qw, bias, code):
    x_f32 = x.float().cpu().numpy().reshape(-1, x.shape[-1])
    xq, sc = O.quantize_activation(x_f32)
    y = O.w4a8_matmul(xq, sc, want_qw)
    if bias is not None:
        y = with_bias_f32(y, bits(bias), code)
    return y


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 3, 16, 17, 200])
@pytest.mark.parametrize("gemv", [False, True])
def test_w4_mode(dtype, M, gemv):
    from liquidgemm_b200.vllm_plugin import apply_layer, prepare_layer
    N, K = 384, 512
    lin, want = _module(N, K, dtype, seed=3)
    prepare_layer(lin, 64, True, gemv)
    assert lin.lq_enabled and not hasattr(lin, "weight") and (lin.lq_N, lin.lq_K) == (N, K)
    assert {n for n, _ in lin.named_buffers()} == {"lq_s1", "lq_rs", "lq_s_u8", "lq_offset_a"}
    assert lin.lq_gemv == gemv
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    bias = (torch.randn(N, generator=g) * 0.1).to(dtype).cuda()
    for b in (None, bias):
        y = apply_layer(lin, x, b, 64, True)
        assert y.dtype == dtype and tuple(y.shape) == (M, N)
        assert_bits_equal(y, _expected(x, want, b, _CODE[dtype]), _CODE[dtype], f"w4 M={M} bias={b is not None}")


def test_w4_mode_with_the_row_major_gemv_pack(monkeypatch):
    """LIQUIDGEMM_GEMV_PACK=1 also stores the reference's `lq_gp` buffer; results do not change."""
    from liquidgemm_b200.vllm_plugin import apply_layer, prepare_layer
    monkeypatch.setenv("LIQUIDGEMM_GEMV_PACK", "1")
    lin, want = _module(256, 256, torch.bfloat16, seed=5)
    prepare_layer(lin, 64, True, True)
    assert hasattr(lin, "lq_gp") and tuple(lin.lq_gp.shape) == (256, 128)
    x = torch.randn(2, 256, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    assert_bits_equal(apply_layer(lin, x, None, 64, True), _expected(x, want, None, 0), 0, "gemv pack")


def test_three_dimensional_activations_keep_their_leading_shape():
    from liquidgemm_b200.vllm_plugin import apply_layer, prepare_layer
    lin, want = _module(128, 256, torch.float16, seed=6)
    prepare_layer(lin, 64, True, False)
    x = torch.randn(2, 5, 256, generator=torch.Generator().manual_seed(1)).to(torch.float16).cuda()
    y = apply_layer(lin, x, None, 64, True)
    assert tuple(y.shape) == (2, 5, 128)
    assert_bits_equal(y.reshape(10, 128), _expected(x, want, None, 1), 1, "3-D input")


@pytest.mark.parametrize("M", [1, 40, 300])
def test_int8_mode(M):
    """Default mode: INT8 weights `lq_w_i8` [N, K] and `lq_s1` [N, 1] (reference :165-170), served by this
    library's own INT8 tensor-core GEMM with the scale epilogue instead of a third-party kernel; the
    numbers are those of the W4 path because the stored INT8 weights are the dequantised codes."""
    from liquidgemm_b200.vllm_plugin import apply_layer, prepare_layer
    N, K = 320, 384
    lin, want = _module(N, K, torch.bfloat16, seed=7)
    prepare_layer(lin, 64, False, False)
    assert lin.lq_enabled and tuple(lin.lq_w_i8.shape) == (N, K) and tuple(lin.lq_s1.shape) == (N, 1)
    assert np.array_equal(lin.lq_w_i8.cpu().numpy(), O.dequantize_i8(want))
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16).cuda()
    for b in (None, bias):
        y = apply_layer(lin, x, b, 64, False)
        assert_bits_equal(y, _expected(x, want, b, 0), 0, f"int8 M={M} bias={b is not None}")


@pytest.mark.parametrize("w4,N,K", [(True, 96, 320), (True, 100, 256), (False, 64, 192)])
def test_unaligned_layers_pass_through(w4, N, K):
    """Layers the kernels cannot take keep their weight and run torch.nn.functional.linear
    (reference :140-145, 176-178)."""
    from liquidgemm_b200.vllm_plugin import apply_layer, prepare_layer
    lin, _ = _module(N, K, torch.bfloat16, seed=8)
    w = lin.weight.data.clone()
    prepare_layer(lin, 64, w4, False)
    assert lin.lq_enabled is False and torch.equal(lin.weight.data, w)
    x = torch.randn(4, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    assert torch.equal(apply_layer(lin, x, b, 64, w4), torch.nn.functional.linear(x, w) + b)


@pytest.mark.parametrize("M", [2, 64])
def test_prepacked_directory_round_trip(tmp_path, M):
    """save_prepacked -> load_prepacked -> attach_prepacked -> apply_layer equals the oracle, and equals the
    layer that was quantised on the fly."""
    from liquidgemm_b200 import checkpoint as C
    from liquidgemm_b200.vllm_plugin import apply_layer, attach_prepacked, collect_prepacked, prepare_layer
    N, K = 256, 512
    model = torch.nn.Module()
    model.proj, want = _module(N, K, torch.bfloat16, seed=9)
    prepare_layer(model.proj, 64, True, False)
    C.save_prepacked(str(tmp_path), list(collect_prepacked(model)))
    entry = C.load_prepacked(str(tmp_path), device="cpu")["proj"]
    fresh = torch.nn.Module()
    fresh.weight = torch.nn.Parameter(torch.empty(N, K, dtype=torch.bfloat16, device="cuda"), requires_grad=False)
    attach_prepacked(fresh, entry)
    assert fresh.lq_rs.is_cuda and not hasattr(fresh, "weight")
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).cuda()
    y = apply_layer(fresh, x, None, 64, True)
    assert_bits_equal(y, _expected(x, want, None, 0), 0, "prepacked")
    assert torch.equal(y, apply_layer(model.proj, x, None, 64, True))


def test_vllm_method_end_to_end(monkeypatch, tmp_path):
    """The vLLM classes themselves: a ReplicatedLinear created with the config, its weight filled as the
    loader would, process_weights_after_loading, apply."""
    import types
    vllm = pytest.importorskip("vllm")
    from liquidgemm_b200 import vllm_plugin as P
    if not P._HAVE_VLLM:
        pytest.skip("vLLM's layer classes did not import")
    import vllm.distributed.parallel_state as ps
    monkeypatch.setattr(ps, "_TP", types.SimpleNamespace(rank_in_group=0, world_size=1))
    monkeypatch.setenv("VLLM_CACHE_ROOT", str(tmp_path))
    monkeypatch.setenv("LIQUIDGEMM_W4", "1")
    from vllm.model_executor.layers.linear import ReplicatedLinear
    N, K = 256, 384
    cfg = P.LiquidGemmConfig()
    lin = ReplicatedLinear(K, N, bias=False, quant_config=cfg, prefix="m.proj", params_dtype=torch.bfloat16).cuda()
    W = O.synth_weight(N, K, seed=11)
    lin.weight.data.copy_(torch.from_numpy(W).to(torch.bfloat16))
    want = O.quantize_weight(lin.weight.data.float().cpu().numpy(), 64)
    lin.quant_method.process_weights_after_loading(lin)
    x = torch.randn(6, K, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).cuda()
    y = lin.quant_method.apply(lin, x, None)
    assert_bits_equal(y, _expected(x, want, None, 0), 0, "vLLM method")
