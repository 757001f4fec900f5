"""liquidgemm_b200: the LiquidQuant (LQQ) W4A8 linear path, written for NVIDIA B200 (sm_100a).

The package mirrors the Python surface of liquidgemm for that one path:

* :mod:`liquidgemm_b200.quant`  -- LQQ two-level weight quantiser, per-token activation quantiser
  and the integer-domain reference formula (host-side torch code, device agnostic);
* :mod:`liquidgemm_b200.pack`   -- nibble / lane packing helpers;
* :mod:`liquidgemm_b200.ops`    -- ``torch.ops.liquidgemm.*`` operators backed by the C-ABI CUDA
  library in ``liquidgemm_b200/csrc`` (imported lazily: it needs the built library);
* :mod:`liquidgemm_b200.vllm_plugin` -- the ``quantization="liquidgemm"`` vLLM method.

Importing the package itself loads no native code, exactly like liquidgemm
(reference liquidgemm/__init__.py, liquidgemm/ops.py:3-4).
"""

__version__ = "0.1.0"
