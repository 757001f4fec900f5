"""Regenerate ``tests/golden/lqq_golden.npz`` by RUNNING the reference's own Python modules.

Usage (only where the reference tree is mounted; the fixtures themselves are committed):

    python tests/golden/make_golden.py <root of the reference tree>

The reference's ``liquidgemm.quant`` / ``liquidgemm.pack`` are pure PyTorch and import as they
are.  ``liquidgemm.ops`` imports a compiled ``_C`` module and attaches fake kernels to ops that
module would have registered; here an empty stand-in ``_C`` is installed and the op schemas are
declared (schema text only, no kernels) so that the module imports and its pure-Python prepack
``pack_gemv_interleaved`` can be executed.  Nothing from the reference is copied into the
fixtures except the numbers it computes.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

CASES = [
    # name, N, K, group, M, seed, kind
    ("g64_small", 64, 256, 64, 5, 0, "synth"),
    ("g128_small", 64, 256, 128, 3, 1, "synth"),
    ("g64_tailed", 96, 384, 64, 17, 2, "tailed"),
    ("g64_flat", 64, 128, 64, 2, 3, "flat"),
]

SCHEMAS = [
    "dequant_weight(Tensor qweight, Tensor s_u8, Tensor offset_a, int N, int K, int group_size) -> Tensor",
    "w4a8_gemm(Tensor X, Tensor qweight, Tensor s_u8, Tensor offset_a, Tensor s1, Tensor ascale, int N, int K, int group_size) -> Tensor",
    "quant_per_token(Tensor x) -> Tensor[]",
    "scale_epilogue(Tensor acc, Tensor ascale, Tensor s1, int out_dtype) -> Tensor",
    "wgmma_i8_gemm(Tensor a, Tensor b) -> Tensor",
    "w4a8_wgmma(Tensor x_i8, Tensor packed, Tensor s_u8, Tensor off_a, int N, int K, int group_size) -> Tensor",
    "w4a8_wgmma_rs(Tensor x_i8, Tensor w, Tensor spack, Tensor s_u8, Tensor off_a, int N, int K, int group_size, bool packed) -> Tensor",
    "w4a8_wgmma_rs_fused(Tensor x_i8, Tensor w, Tensor s_u8, Tensor off_a, Tensor ascale, Tensor s1, int N, int K, int group_size, int out_dtype) -> Tensor",
    "w4a8_gemv2(Tensor x_i8, Tensor gpack, Tensor s_u8, Tensor off_a, Tensor ascale, Tensor s1, int N, int K, int group_size, int out_dtype) -> Tensor",
]


def make_inputs(N, K, M, seed, kind):
    g = torch.Generator().manual_seed(seed)
    if kind == "synth":
        W = torch.randn(N, K, generator=g) * 0.02
        W = torch.where(torch.rand(N, K, generator=g) < 0.01, W * 20, W)
    elif kind == "tailed":
        W = torch.randn(N, K, generator=g)
        W = W + 0.1 * torch.randn(N, 1, generator=g) * torch.randn(N, K, generator=g).abs()
    else:  # rows with tiny dynamic range, one all-zero row, one constant row
        W = torch.randn(N, K, generator=g) * 1e-3
        W[0] = 0.0
        W[1] = 0.5
    W = W.to(torch.float16).to(torch.float32)
    X = torch.randn(M, K, generator=g).to(torch.float16).to(torch.float32)
    if kind == "flat":
        X[0] = 0.0
    return W, X


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import liquidgemm  # noqa: F401
    from liquidgemm import quant, pack

    lib = torch.library.Library("liquidgemm", "DEF")
    for s in SCHEMAS:
        lib.define(s)
    sys.modules["liquidgemm._C"] = types.ModuleType("liquidgemm._C")
    from liquidgemm import ops as ref_ops

    out = {}
    for name, N, K, grp, M, seed, kind in CASES:
        W, X = make_inputs(N, K, M, seed, kind)
        qw = quant.quantize_weight(W, grp)
        x8, asc = quant.quantize_activation(X)
        y = quant.w4a8_matmul(x8, asc, qw)
        p = name + "/"
        out[p + "W"] = W.to(torch.float16).numpy()  # exactly representable: inputs were rounded to fp16
        out[p + "X"] = X.to(torch.float16).numpy()
        out[p + "group"] = np.int64(grp)
        out[p + "q_u4"] = qw.qweight_u4.numpy()
        out[p + "s_u8"] = qw.s_u8.numpy()
        out[p + "offset_a"] = qw.offset_a.numpy()
        out[p + "s1"] = qw.s1.numpy()
        out[p + "qhat_xor"] = quant._dequant_i8_via_xor(qw).numpy()
        out[p + "qhat_sub"] = quant._dequant_i8_via_sub(qw).numpy()
        if name == "g64_small":
            out[p + "w_hat"] = quant.dequantize(qw).numpy()
        out[p + "x_i8"] = x8.numpy()
        out[p + "ascale"] = asc.numpy()
        out[p + "acc"] = (x8.to(torch.int32) @ quant.dequantize_i8(qw).to(torch.int32).t()).numpy()
        out[p + "y_f32"] = y.numpy()
        out[p + "y_bf16_bits"] = y.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        out[p + "y_f16_bits"] = y.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
        out[p + "nibbles"] = pack.pack_nibbles(qw.qweight_u4).numpy()
        out[p + "lanes_u32"] = pack.pack_lanes_u32(qw.qweight_u4).numpy().astype(np.uint32)
        out[p + "simd_qhat"] = pack.simd_dequant_u32(qw).numpy()
        out[p + "gemv_pack"] = ref_ops.pack_gemv_interleaved(qw).numpy()
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "lqq_golden.npz"), **out)
    print("wrote", os.path.join(here, "lqq_golden.npz"), "with", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
