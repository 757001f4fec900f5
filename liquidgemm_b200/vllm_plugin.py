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

A directory written by :func:`liquidgemm_b200.checkpoint.save_prepacked` can replace the on-the-fly
quantisation (the reference has no such format: its ``get_config_filenames`` returns ``[]`` and every
start re-quantises, liquidgemm/vllm_plugin.py:92-99,136-172).  It is selected explicitly, either by
``LIQUIDGEMM_PREPACKED_DIR=<dir>`` or by a ``"prepacked_dir"`` entry of the model's
``quantization_config``; ``get_config_filenames`` stays ``[]`` so that an ordinary bf16 checkpoint loads
exactly as with the reference.  A layer whose name is in the directory gets its buffers from there,
every other layer is quantised from its weight as before.

The pure logic lives in :func:`prepare_layer` / :func:`attach_prepacked` / :func:`apply_layer`, which need
only torch; the vLLM classes at the bottom are thin adapters and are defined only when vLLM imports.
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
    # the INT8 tensor-core GEMM of this package walks K in steps of 128 (the reference's CUTLASS path only
    # needs K % group_size == 0, liquidgemm/vllm_plugin.py:140-141)
    return k % group_size == 0 and k % 128 == 0


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
    dev = W.device
    blob = None
    if W.is_cuda and k % 128 == 0 and group_size in (64, 128):
        # quantise and prepack in two kernels, straight from the checkpoint dtype: no fp32 copy of the
        # weight, no one-code-per-byte intermediate in W4 mode, no host read
        qw, blob = ops.quantize_weight_cuda(W, group_size, want_codes=not w4, want_blob=w4)
    else:
        qw = quantize_weight(W.float(), group_size=group_size)
    layer.lq_enabled = True
    layer.lq_N, layer.lq_K = qw.N, qw.K
    if w4:
        layer.register_buffer("lq_s1", qw.s1.to(dev))
        layer.register_buffer("lq_rs", (blob if blob is not None else ops.repack_rs_weight(qw)).to(dev))
        layer.register_buffer("lq_s_u8", qw.s_u8.to(dev))
        layer.register_buffer("lq_offset_a", qw.offset_a.to(dev))
        # LIQUIDGEMM_GEMV=1 asks for the decode GEMV.  Here the GEMV reads the tile blob, so the flag
        # needs no second copy of the weights (the reference stores `lq_gp`, doubling weight memory:
        # liquidgemm/vllm_plugin.py:157-164); LIQUIDGEMM_GEMV_PACK=1 still builds that row-major pack
        # for callers that want to drive torch.ops.liquidgemm.w4a8_gemv2 themselves.
        layer.lq_gemv = bool(gemv and qw.K % 128 == 0 and group_size == 64)
        if layer.lq_gemv and os.environ.get("LIQUIDGEMM_GEMV_PACK") == "1":
            if qw.qweight_u4 is None:
                qw = quantize_weight(W.float(), group_size=group_size)
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
    if device is not None:
        dev = device
    elif hasattr(layer, "weight") and layer.weight is not None:
        dev = layer.weight.device
    else:
        dev = entry["rs"].device
    if hasattr(layer, "weight") and layer.weight is not None and tuple(layer.weight.shape) != (int(entry["N"]), int(entry["K"])):
        raise RuntimeError(f"liquidgemm: prepacked entry is {entry['N']}x{entry['K']} but the layer holds "
                           f"{tuple(layer.weight.shape)} (a directory packed for another tensor-parallel size?)")
    layer.lq_enabled = True
    layer.lq_N, layer.lq_K = int(entry["N"]), int(entry["K"])
    layer.register_buffer("lq_s1", entry["s1"].to(dev))
    layer.register_buffer("lq_rs", entry["rs"].to(dev))
    layer.register_buffer("lq_s_u8", entry["s_u8"].to(dev))
    layer.register_buffer("lq_offset_a", entry["offset_a"].to(dev))
    layer.lq_gemv = layer.lq_K % 128 == 0
    if hasattr(layer, "weight"):
        del layer.weight


def collect_prepacked(model: torch.nn.Module):
    """(name, entry) of every W4 layer of ``model`` that :func:`prepare_layer` has processed, in the form
    :func:`liquidgemm_b200.checkpoint.save_prepacked` writes; the names are the module paths vLLM passes to
    ``get_quant_method`` as ``prefix``."""
    for name, mod in model.named_modules():
        if getattr(mod, "lq_enabled", False) and hasattr(mod, "lq_rs"):
            yield name, {"rs": mod.lq_rs, "s1": mod.lq_s1, "s_u8": mod.lq_s_u8, "offset_a": mod.lq_offset_a,
                         "N": mod.lq_N, "K": mod.lq_K}


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
        if bias is not None and bias.dtype == x.dtype and x.dtype in _DT:
            # the bias rides in the kernel's epilogue, added to the rounded output exactly like the
            # separate `y + bias` of the reference (liquidgemm/vllm_plugin.py:205-206)
            y = torch.ops.liquidgemm.w4a8_linear_bias(x_i8, layer.lq_rs, ascale, layer.lq_s1, bias, n, layer.lq_K, odt)
            return y.reshape(*shape[:-1], n)
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

        def __init__(self, group_size: int = 64, w4: bool = False, prepacked_dir: Optional[str] = None):
            super().__init__()
            self.group_size = group_size
            self.w4, self.gemv = mode_from_env(w4)
            self.prepacked_dir = os.environ.get("LIQUIDGEMM_PREPACKED_DIR") or prepacked_dir
            self._prepacked = None   # read on first use: {layer name: entry on the CPU}
            _salt_compile_cache(("w4" if self.w4 else "int8") + ("-gemv" if self.gemv else ""))

        def prepacked_entry(self, prefix: str):
            """The prepacked buffers of layer ``prefix``, or None (no directory configured, INT8 mode, or
            the directory does not hold that layer)."""
            if not self.prepacked_dir or not self.w4:
                return None
            if self._prepacked is None:
                from .checkpoint import load_prepacked, read_config
                cfg = read_config(self.prepacked_dir)
                if int(cfg["group_size"]) != int(self.group_size):
                    raise RuntimeError(f"liquidgemm: {self.prepacked_dir} was packed with group size "
                                       f"{cfg['group_size']}, the method is configured for {self.group_size}")
                self._prepacked = load_prepacked(self.prepacked_dir, device="cpu")
            return self._prepacked.get(prefix)

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
            # Empty like the reference (liquidgemm/vllm_plugin.py:92-94): vLLM then builds the default
            # config for a plain bf16 checkpoint instead of demanding a json file beside it.
            return []

        @classmethod
        def from_config(cls, config: dict) -> "LiquidGemmConfig":
            return cls(group_size=int(config.get("group_size", 64)), w4=bool(config.get("w4", True)),
                       prepacked_dir=config.get("prepacked_dir"))

        def get_quant_method(self, layer: torch.nn.Module, prefix: str):
            if isinstance(layer, LinearBase):
                return LiquidGemmLinearMethod(self, prefix)
            return None

    class LiquidGemmLinearMethod(LinearMethodBase):
        """Reference liquidgemm/vllm_plugin.py:111-206."""

        def __init__(self, cfg: "LiquidGemmConfig", prefix: str = ""):
            self.cfg = cfg
            self.prefix = prefix

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
            entry = self.cfg.prepacked_entry(self.prefix)
            if entry is not None:
                attach_prepacked(layer, entry)
            else:
                prepare_layer(layer, self.cfg.group_size, self.cfg.w4, self.cfg.gemv)

        def apply(self, layer, x, bias=None):
            return apply_layer(layer, x, bias, self.cfg.group_size, self.cfg.w4)
