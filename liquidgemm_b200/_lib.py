"""ctypes binding of the C-ABI CUDA library (``include/liquidgemm_b200.h``).

There is no fallback: if the shared library has not been built, importing this module raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lq_b200.so")
if os.environ.get("LIQUIDGEMM_B200_TRACE") == "1":   # pipeline studies: `python -m liquidgemm_b200.build --trace`
    LIB_PATH = os.path.join(_HERE, "_lq_b200_trace.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m liquidgemm_b200.build` "
        "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback for these ops.")

lib = ctypes.CDLL(LIB_PATH)

P = c_void_p
_SIGNATURES = {
    "lq_abi_version": (c_int, []),
    "lq_error_string": (c_char_p, [c_int]),
    "lq_last_cuda_error": (c_char_p, []),
    "lq_check_device": (c_int, []),
    "lq_poll_status": (c_int, [P]),
    "lq_dequant_weight": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "lq_quant_per_token": (c_int, [P, c_int, P, P, c_int, c_int, P]),
    "lq_scale_epilogue": (c_int, [P, P, P, P, c_int, c_int, c_int, P]),
    "lq_w4a8_gemv": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P]),
    "lq_gemv_blob_workspace_bytes": (c_size_t, []),
    "lq_w4a8_gemv_blob": (c_int, [P, P, P, P, P, c_int, c_int, c_int, c_int, P, c_size_t, P]),
    "lq_w4a8_gemv_blob_static": (c_int, [P, P, P, P, P, c_int, c_int, c_int, c_int, P]),
    "lq_w4a8_gemv_blob_static_reset": (c_int, [P]),
    "lq_w4a8_gemm_fused_scatter": (c_int, [P, P, P, P, P, c_int, ctypes.c_long, ctypes.c_long, c_int, c_int, c_int,
                                           c_int, P, c_size_t, P]),
    "lq_w4a8_gemm_fused_scatter_sync": (c_int, [P, P, P, P, P, c_int, ctypes.c_long, ctypes.c_long, c_int, c_int, c_int,
                                                c_int, P, c_int, P, ctypes.c_uint, P, c_size_t, P]),
    "lq_decode_grid": (c_int, [c_int, c_int, c_int]),
    "lq_scatter_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lq_scatter_workspace_kind": (c_int, [c_int, c_int, c_int]),
    "lq_linear_host_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "lq_w4a8_linear_host": (c_int, [P, c_int, P, P, P, c_int, c_int, c_int, c_int, P, c_size_t, P, c_size_t, P]),
    "lq_gemm_v1_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lq_w4a8_gemm_v1": (c_int, [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, P, c_size_t, P]),
    "lq_tile_blob_bytes": (c_size_t, [c_int, c_int]),
    "lq_repack_tiles": (c_int, [P, c_int, P, P, P, c_int, c_int, c_int, P]),
    "lq_gemm_pick_splitk": (c_int, [c_int, c_int, c_int, c_int]),
    "lq_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lq_gemm_workspace_kind": (c_int, [c_int, c_int, c_int, c_int]),
    "lq_gemm_launches": (c_int, [c_int, c_int, c_int, c_int]),
    "lq_w4a8_linear_bias": (c_int, [P, P, P, P, P, P, c_int, c_int, c_int, c_int, P, c_size_t, P]),
    "lq_quantize_weight": (c_int, [P, c_int, c_int, c_int, c_int, P, P, P, P, P, P]),
    "lq_w4a8_gemm_i32": (c_int, [P, P, P, c_int, c_int, c_int, c_int, P, c_size_t, P]),
    "lq_w4a8_gemm_fused": (c_int, [P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, c_size_t, P]),
    "lq_i8_gemm_i32": (c_int, [P, P, P, c_int, c_int, c_int, P]),
    "lq_i8_gemm_scaled": (c_int, [P, P, P, P, P, c_int, c_int, c_int, c_int, P]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

ABI_VERSION = lib.lq_abi_version()


class LiquidGemmError(RuntimeError):
    """A C-ABI call returned a negative status."""


def check(code: int, what: str) -> None:
    """Turn a non-zero status of ``what`` into a RuntimeError (the reference raises through
    TORCH_CHECK, e.g. csrc/liquid_gemm/gemv2.cu:85-89)."""
    if code == 0:
        return
    msg = lib.lq_error_string(code).decode()
    detail = lib.lq_last_cuda_error().decode() if code == -4 or code == -6 else ""
    raise LiquidGemmError(f"{what}: {msg}" + (f" [{detail}]" if detail else ""))
