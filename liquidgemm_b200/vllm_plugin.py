"""vLLM quantization method ``"liquidgemm"`` backed by the B200 kernels of this package.

Same registration name, classes, layer buffers and environment switches as the reference plugin
(liquidgemm/vllm_plugin.py), so ``LLM(model, quantization="liquidgemm")`` keeps working:

* ``LIQUIDGEMM_W4=1``    store 4-bit weights and run the fused W4A8 tensor-core GEMM;
* ``LIQUIDGEMM_GEMV=1``  decode GEMV for small M (reference liquidgemm/vllm_plugin.py:157-164); here it
                         is served from the same tile blob as the GEMM, so it costs no extra memory
                         and is in fact always on;
* ``LIQUIDGEMM_SPLITK``  split-K override for M <= 128, read once by :mod:`liquidgemm_b200.ops`.

Differences that follow from the hardware target: the minimum capability is 100 (sm_100a), and
the default INT8 mode runs this package's own INT8 tensor-core GEMM with the scale epilogue
instead of vLLM's CUTLASS kernel (reference liquidgemm/vllm_plugin.py:197-204), so no
third-party GEMM sits on the path.

The pure logic lives in :class:`LinearState` / :func:`prepare_layer` / :func:`apply_layer`, which
need only torch; the vLLM classes at the bottom are thin adapters and are defined only when vLLM
imports.
"""

from __future__ import annotations

import os
from typing import Any, Optional

import torch

from .quant import quantize_weight

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def register():
    """``vllm.general_plugins`` entry point; importing the module already registered the method
    (reference liquidgemm/vllm_plugin.py:42-45)."""
    return None


def _salt_compile_cache(mode: str) -> None:
    """Give every mode its own vLLM compile cache: the mode changes the traced graph but is
    invisible to vLLM's config hash (reference liquidgemm/vllm_plugin.py:48-60)."""
    root = os.environ.get("VLLM_CACHE_ROOT", os.path.expanduser("~/.cache/vllm"))
    tag = "liquidgemm-" + mode
    if not root.rstrip("/").endswith(tag):
        os.environ["VLLM_CACHE_ROOT"] = os.path.join(root, tag)


def mode_from_env(w4_default: bool) -> tuple[bool, bool]:
    """(w4, gemv) after the environment overrides (reference liquidgemm/vllm_plugin.py:75-79,161)."""
    env = os.environ.get("LIQUIDGEMM_W4")
    w4 = (env == "1") if env is not None else w4_default
    gemv = os.environ.get("LIQUIDGEMM_GEMV") == "1"
    return w4, gemv


def layer_is_aligned(n: int, k: int, group_size: int, w4: bool) -> bool:
    """Which layers are quantised; the rest stay in their original dtype
    (reference liquidgemm/vllm_plugin.py:140-145)."""
    if w4:
        return k % 128 == 0 and n % 64 == 0
    return k % group_size == 0


def prepare_layer(layer: torch.nn.Module, group_size: int, w4: bool, gemv: bool) -> None:
    """Quantise ``layer.weight`` and attach the device buffers the forward pass uses
    (reference liquidgemm/vllm_plugin.py:136-172; same buffer names)."""
    from . import ops
    W = layer.weight.data
    n, k = W.shape
    if not layer_is_aligned(n, k, group_size, w4):
        layer.lq_enabled = False
        layer.weight = torch.nn.Parameter(W, requires_grad=False)
        return
    qw = quantize_weight(W.float(), group_size=group_size)
    dev = W.device
    layer.lq_enabled = True
    layer.lq_N, layer.lq_K = qw.N, qw.K
    if w4:
        layer.register_buffer("lq_s1", qw.s1.to(dev))
        layer.register_buffer("lq_rs", ops.repack_rs_weight(qw).to(dev))
        layer.register_buffer("lq_s_u8", qw.s_u8.to(dev))
        layer.register_buffer("lq_offset_a", qw.offset_a.to(dev))
        # LIQUIDGEMM_GEMV=1 asks for the decode GEMV.  Here the GEMV reads the tile blob, so the flag
        # needs no second copy of the weights (the reference stores `lq_gp`, doubling weight memory:
        # liquidgemm/vllm_plugin.py:157-164); LIQUIDGEMM_GEMV_PACK=1 still builds that row-major pack
        # for callers that want to drive torch.ops.liquidgemm.w4a8_gemv2 themselves.
        layer.lq_gemv = bool(gemv and qw.K % 128 == 0 and group_size == 64)
        if layer.lq_gemv and os.environ.get("LIQUIDGEMM_GEMV_PACK") == "1":
            layer.register_buffer("lq_gp", ops.pack_gemv_interleaved(qw).to(dev))
    else:
        w_i8 = torch.ops.liquidgemm.dequant_weight(qw.qweight_u4.to(dev), qw.s_u8.to(dev), qw.offset_a.to(dev),
                                                   qw.N, qw.K, group_size)
        layer.register_buffer("lq_w_i8", w_i8.contiguous())
        layer.register_buffer("lq_s1", qw.s1.to(dev).view(qw.N, 1).contiguous())
    del layer.weight


def attach_prepacked(layer: torch.nn.Module, entry: dict, device=None) -> None:
    """Give ``layer`` the buffers of :func:`prepare_layer` (W4 mode) from one entry of a prepacked
    checkpoint directory (:func:`liquidgemm_b200.checkpoint.load_prepacked`) instead of quantising its
    bf16 weight: same buffer names, nothing recomputed."""
    dev = device if device is not None else entry["rs"].device
    layer.lq_enabled = True
    layer.lq_N, layer.lq_K = int(entry["N"]), int(entry["K"])
    layer.register_buffer("lq_s1", entry["s1"].to(dev))
    layer.register_buffer("lq_rs", entry["rs"].to(dev))
    layer.register_buffer("lq_s_u8", entry["s_u8"].to(dev))
    layer.register_buffer("lq_offset_a", entry["offset_a"].to(dev))
    layer.lq_gemv = layer.lq_K % 128 == 0
    if hasattr(layer, "weight"):
        del layer.weight


def apply_layer(layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor], group_size: int,
                w4: bool) -> torch.Tensor:
    """Forward of one linear (reference liquidgemm/vllm_plugin.py:174-206)."""
    if not getattr(layer, "lq_enabled", False):
        y = torch.nn.functional.linear(x, layer.weight)
        return y if bias is None else y + bias
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    n = layer.lq_N
    odt = _DT.get(x.dtype, 0)
    x_i8, ascale = torch.ops.liquidgemm.quant_per_token(x2)
    if w4:
        from .ops import use_gemv
        if use_gemv(x_i8.shape[0], n, layer.lq_K, hasattr(layer, "lq_gp"), True):
            y = torch.ops.liquidgemm.w4a8_gemv2(x_i8, layer.lq_gp, layer.lq_s_u8, layer.lq_offset_a, ascale,
                                                layer.lq_s1, n, layer.lq_K, group_size, odt)
        else:
            y = torch.ops.liquidgemm.w4a8_wgmma_rs_fused(x_i8, layer.lq_rs, layer.lq_s_u8, layer.lq_offset_a, ascale,
                                                         layer.lq_s1, n, layer.lq_K, group_size, odt)
    else:
        y = torch.ops.liquidgemm.i8_gemm_scaled(x_i8, layer.lq_w_i8, ascale, layer.lq_s1, odt)
    y = y.reshape(*shape[:-1], n)
    return y if bias is None else y + bias


try:  # the adapters need vLLM; the logic above does not
    from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase
    from vllm.model_executor.layers.quantization import register_quantization_config
    from vllm.model_executor.layers.quantization.base_config import QuantizationConfig, QuantizeMethodBase
    from vllm.model_executor.parameter import ModelWeightParameter
    from vllm.model_executor.utils import set_weight_attrs
    _HAVE_VLLM = True
except Exception:  # pragma: no cover - exercised where vLLM is absent
    _HAVE_VLLM = False


if _HAVE_VLLM:
    from . import ops  # noqa: F401  (registers torch.ops.liquidgemm.*)

    @register_quantization_config("liquidgemm")
    class LiquidGemmConfig(QuantizationConfig):
        """Reference liquidgemm/vllm_plugin.py:63-108."""

        def __init__(self, group_size: int = 64, w4: bool = False):
            super().__init__()
            self.group_size = group_size
            self.w4, self.gemv = mode_from_env(w4)
            _salt_compile_cache(("w4" if self.w4 else "int8") + ("-gemv" if self.gemv else ""))

        @classmethod
        def get_name(cls) -> str:
            return "liquidgemm"

        @classmethod
        def get_supported_act_dtypes(cls) -> list:
            return [torch.bfloat16, torch.float16]

        @classmethod
        def get_min_capability(cls) -> int:
            return 100

        @classmethod
        def get_config_filenames(cls) -> list:
            from .checkpoint import CONFIG_NAME
            return [CONFIG_NAME]   # written by liquidgemm_b200.checkpoint.save_prepacked

        @classmethod
        def from_config(cls, config: dict) -> "LiquidGemmConfig":
            return cls(group_size=int(config.get("group_size", 64)), w4=bool(config.get("w4", True)))

        def get_quant_method(self, layer: torch.nn.Module, prefix: str):
            if isinstance(layer, LinearBase):
                return LiquidGemmLinearMethod(self)
            return None

    class LiquidGemmLinearMethod(LinearMethodBase):
        """Reference liquidgemm/vllm_plugin.py:111-206."""

        def __init__(self, cfg: "LiquidGemmConfig"):
            self.cfg = cfg

        def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                           params_dtype, **extra_weight_attrs):
            weight_loader = extra_weight_attrs.pop("weight_loader")
            weight = ModelWeightParameter(
                data=torch.empty(sum(output_partition_sizes), input_size_per_partition, dtype=params_dtype),
                input_dim=1, output_dim=0, weight_loader=weight_loader)
            layer.register_parameter("weight", weight)
            set_weight_attrs(weight, extra_weight_attrs)
            layer.input_size_per_partition = input_size_per_partition

        def process_weights_after_loading(self, layer) -> None:
            prepare_layer(layer, self.cfg.group_size, self.cfg.w4, self.cfg.gemv)

        def apply(self, layer, x, bias=None):
            return apply_layer(layer, x, bias, self.cfg.group_size, self.cfg.w4)
