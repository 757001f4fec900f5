"""The outer boundary under the installed vLLM, on the CPU: the config class answers vLLM's hooks the way
the reference's does (liquidgemm/vllm_plugin.py:63-108), vLLM's own ``get_quant_config`` accepts a plain
bf16 model directory, and a vLLM linear layer built with the config gets the liquidgemm method.

The forward pass (``apply``) needs the CUDA kernels and is covered by tests/test_gpu_plugin.py.
"""

import json
import os
import types

import pytest
import torch

vllm = pytest.importorskip("vllm")

from liquidgemm_b200 import checkpoint as C  # noqa: E402
from liquidgemm_b200 import vllm_plugin as P  # noqa: E402

pytestmark = pytest.mark.skipif(not P._HAVE_VLLM, reason="vLLM's layer classes did not import")


@pytest.fixture(autouse=True)
def _clean_env(monkeypatch, tmp_path):
    for k in ("LIQUIDGEMM_W4", "LIQUIDGEMM_GEMV", "LIQUIDGEMM_PREPACKED_DIR"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("VLLM_CACHE_ROOT", str(tmp_path / "cache"))


def test_config_hooks_match_the_reference():
    cfg = P.LiquidGemmConfig()
    assert cfg.get_name() == "liquidgemm"
    assert cfg.get_config_filenames() == []                 # reference liquidgemm/vllm_plugin.py:92-94
    assert cfg.get_min_capability() == 100                  # sm_100a kernels (the reference says 80)
    assert cfg.get_supported_act_dtypes() == [torch.bfloat16, torch.float16]
    assert (cfg.group_size, cfg.w4) == (64, False)          # constructor default: INT8 mode
    c2 = P.LiquidGemmConfig.from_config({})
    assert (c2.group_size, c2.w4, c2.prepacked_dir) == (64, True, None)   # from_config default: W4
    c3 = P.LiquidGemmConfig.from_config({"group_size": 128, "w4": False, "prepacked_dir": "/x"})
    assert (c3.group_size, c3.w4, c3.prepacked_dir) == (128, False, "/x")
    assert os.environ["VLLM_CACHE_ROOT"].rstrip("/").endswith("liquidgemm-int8")


def test_env_switches(monkeypatch):
    monkeypatch.setenv("LIQUIDGEMM_W4", "1")
    monkeypatch.setenv("LIQUIDGEMM_GEMV", "1")
    cfg = P.LiquidGemmConfig()
    assert cfg.w4 and cfg.gemv
    assert os.environ["VLLM_CACHE_ROOT"].rstrip("/").endswith("liquidgemm-w4-gemv")
    monkeypatch.setenv("LIQUIDGEMM_W4", "0")
    assert not P.LiquidGemmConfig.from_config({"w4": True}).w4      # the environment wins


def test_vllm_builds_the_default_config_for_a_plain_bf16_directory(tmp_path):
    """vLLM's loader only falls back to the default config when get_config_filenames() is empty; with a
    file name in that list it raises 'Cannot find the config file for liquidgemm'."""
    from vllm.model_executor.model_loader.weight_utils import get_quant_config
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text("{}")
    mc = types.SimpleNamespace(quantization="liquidgemm", hf_config=types.SimpleNamespace(), hf_overrides={},
                               quantization_config=None, model=str(model_dir), revision=None)
    cfg = get_quant_config(mc, types.SimpleNamespace(download_dir=None))
    assert isinstance(cfg, P.LiquidGemmConfig) and cfg.group_size == 64
    # a quantization_config inside the model's config.json goes through from_config
    mc.hf_config = types.SimpleNamespace(quantization_config={"quant_method": "liquidgemm", "w4": True,
                                                              "prepacked_dir": str(tmp_path / "packed")})
    cfg = get_quant_config(mc, types.SimpleNamespace(download_dir=None))
    assert cfg.w4 and cfg.prepacked_dir == str(tmp_path / "packed")


def _fake_tp(monkeypatch):
    import vllm.distributed.parallel_state as ps
    monkeypatch.setattr(ps, "_TP", types.SimpleNamespace(rank_in_group=0, world_size=1))


def test_linear_layers_get_the_method_and_a_bf16_weight(monkeypatch):
    _fake_tp(monkeypatch)
    from vllm.model_executor.layers.linear import LinearBase, ReplicatedLinear
    cfg = P.LiquidGemmConfig()
    lin = ReplicatedLinear(256, 128, bias=True, quant_config=cfg, prefix="model.layers.0.proj",
                           params_dtype=torch.bfloat16)
    assert isinstance(lin, LinearBase) and isinstance(lin.quant_method, P.LiquidGemmLinearMethod)
    assert lin.quant_method.prefix == "model.layers.0.proj"
    assert tuple(lin.weight.shape) == (128, 256) and lin.weight.dtype == torch.bfloat16
    assert lin.input_size_per_partition == 256
    assert cfg.get_quant_method(torch.nn.LayerNorm(8), "ln") is None


def test_unaligned_layer_stays_in_its_dtype(monkeypatch):
    """K % 128 != 0: no quantisation, the weight stays a plain parameter (reference :140-145, 176-178)."""
    _fake_tp(monkeypatch)
    from vllm.model_executor.layers.linear import ReplicatedLinear
    monkeypatch.setenv("LIQUIDGEMM_W4", "1")
    cfg = P.LiquidGemmConfig()
    lin = ReplicatedLinear(192, 64, bias=False, quant_config=cfg, prefix="p", params_dtype=torch.bfloat16)
    torch.nn.init.normal_(lin.weight)
    w = lin.weight.data.clone()
    lin.quant_method.process_weights_after_loading(lin)
    assert lin.lq_enabled is False and torch.equal(lin.weight.data, w)
    x = torch.randn(3, 192, dtype=torch.bfloat16)
    b = torch.randn(64, dtype=torch.bfloat16)
    y = lin.quant_method.apply(lin, x, b)
    assert torch.equal(y, torch.nn.functional.linear(x, w) + b)


def test_alignment_rules():
    assert P.layer_is_aligned(64, 128, 64, True) and not P.layer_is_aligned(32, 128, 64, True)
    assert not P.layer_is_aligned(64, 192, 64, True)
    assert P.layer_is_aligned(7, 256, 64, False)
    assert not P.layer_is_aligned(7, 192, 64, False)     # the INT8 GEMM needs K % 128 == 0


def test_prepacked_directory_feeds_process_weights(monkeypatch, tmp_path):
    """With a directory configured, a layer whose prefix it holds takes its buffers from there instead of
    quantising its weight; a layer it does not hold is left to the ordinary path."""
    _fake_tp(monkeypatch)
    from vllm.model_executor.layers.linear import ReplicatedLinear
    N, K = 128, 256
    g = torch.Generator().manual_seed(0)
    entry = {"rs": torch.randint(0, 256, (C.blob_bytes(N, K),), dtype=torch.uint8, generator=g),
             "s1": torch.rand(N, generator=g), "s_u8": torch.randint(1, 17, (N, K // 64), dtype=torch.uint8, generator=g),
             "offset_a": torch.randint(0, 256, (N, K // 64), dtype=torch.uint8, generator=g), "N": N, "K": K}
    C.save_prepacked(str(tmp_path / "packed"), [("model.layers.0.proj", entry)])
    monkeypatch.setenv("LIQUIDGEMM_W4", "1")
    monkeypatch.setenv("LIQUIDGEMM_PREPACKED_DIR", str(tmp_path / "packed"))
    cfg = P.LiquidGemmConfig()
    assert cfg.prepacked_dir == str(tmp_path / "packed")
    lin = ReplicatedLinear(K, N, bias=False, quant_config=cfg, prefix="model.layers.0.proj", params_dtype=torch.bfloat16)
    lin.quant_method.process_weights_after_loading(lin)
    assert lin.lq_enabled and not hasattr(lin, "weight") and torch.equal(lin.lq_rs, entry["rs"])
    assert cfg.prepacked_entry("model.layers.1.proj") is None
    # wrong partition shape: refused, not silently mis-sized
    lin2 = ReplicatedLinear(K, 2 * N, bias=False, quant_config=cfg, prefix="model.layers.0.proj",
                            params_dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        lin2.quant_method.process_weights_after_loading(lin2)
    # wrong group size: refused when the directory is first read
    monkeypatch.setenv("LIQUIDGEMM_PREPACKED_DIR", str(tmp_path / "packed"))
    cfg128 = P.LiquidGemmConfig(group_size=128)
    with pytest.raises(RuntimeError):
        cfg128.prepacked_entry("model.layers.0.proj")
