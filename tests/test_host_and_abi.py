"""CPU-only checks: the C ABI exports what the header declares, the operator layer mirrors the
reference's schemas, fake kernels give the right shapes, host-side packs and plugin logic."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import lqq_oracle as O
from tests.conftest import ROOT, REFERENCE_ROOT, have_reference
from tests.helpers import random_lqq, to_torch_qw


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "liquidgemm_b200.h")).read()
    return sorted(set(re.findall(r"LQ_API\s+[\w\s\*]+?\b(lq_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from liquidgemm_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in include/liquidgemm_b200.h but not exported"
        assert n in _lib._SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib.lq_abi_version() == 1
    assert _lib.lib.lq_error_string(-2).decode().startswith("shape")


def test_size_helpers_without_gpu():
    from liquidgemm_b200._lib import lib
    assert lib.lq_tile_blob_bytes(6144, 4096) == 48 * 32 * 8704
    assert lib.lq_tile_blob_bytes(100, 256) == 1 * 2 * 8704      # rows padded to 128
    assert lib.lq_tile_blob_bytes(128, 100) == 0                 # K % 128 != 0
    assert lib.lq_gemm_pick_splitk(64, 4096, 14336, 0) == 0      # stream-K by default
    assert lib.lq_gemm_pick_splitk(64, 4096, 14336, 4) == 4      # LIQUIDGEMM_SPLITK applies for M <= 128
    assert lib.lq_gemm_pick_splitk(256, 4096, 14336, 4) == 0     # ... and not above
    assert lib.lq_gemm_pick_splitk(64, 4096, 256, 8) == 2        # clamped to K/128
    assert lib.lq_gemm_workspace_bytes(64, 4096, 14336, 1) == 0
    assert lib.lq_gemm_workspace_bytes(64, 4096, 14336, 4) == 4 * 64 * 4096 * 4
    assert lib.lq_gemm_workspace_kind(64, 4096, 14336, 4) == 1
    assert lib.lq_gemm_workspace_kind(2048, 4224, 14336, 0) == 0     # tile kernel, one k-range: no workspace
    assert lib.lq_gemm_workspace_kind(2048, 4096, 14336, -1) == 2
    assert lib.lq_gemm_workspace_kind(2, 4096, 14336, 0) == 2        # streaming decode kernels
    assert lib.lq_gemm_workspace_kind(8, 6144, 4096, 0) == 2         # streaming tensor-core kernel, atomic join
    assert lib.lq_gemm_workspace_kind(8, 4096, 14336, 0) == 1        # larger matrix: tile kernel with split-K planes
    assert lib.lq_gemm_workspace_kind(64, 4096, 14336, 0) == 1       # tile kernel with split-K planes
    assert lib.lq_gemm_workspace_kind(4096, 28672, 4096, 0) == 2     # pair kernel, last wave split along k
    assert lib.lq_gemm_workspace_kind(8192, 6144, 4096, 0) == 1      # unpack to INT8 scratch, then the INT8 pair kernel
    assert lib.lq_gemm_workspace_bytes(8192, 6144, 4096, 0) == 6144 * 4096
    assert lib.lq_gemm_launches(8192, 6144, 4096, 0) == 2
    assert lib.lq_gemm_workspace_kind(8192, 4096, 14336, 0) == 2     # pair kernel, last wave split along k
    assert lib.lq_gemm_launches(8, 6144, 4096, 0) == 1 and lib.lq_gemm_launches(64, 4096, 14336, 0) == 2
    assert lib.lq_scatter_workspace_bytes(8, 4096, 14336) > 0
    assert lib.lq_gemm_workspace_kind(2048, 4096, 14336, 1) == 0


def test_bad_arguments_return_codes_without_touching_the_gpu():
    from liquidgemm_b200._lib import lib
    assert lib.lq_dequant_weight(None, None, None, None, 4, 4, 4, None) == -1
    buf = (ctypes.c_uint8 * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.lq_dequant_weight(p, p, p, p, 4, 6, 4, None) == -2          # K % 4
    assert lib.lq_w4a8_gemv(p, p, p, p, p, p, p, 0, 17, 64, 128, 64, None) == -2   # M > 16
    assert lib.lq_w4a8_gemv(p, p, p, p, p, p, p, 0, 4, 64, 128, 32, None) == -2    # group != 64
    assert lib.lq_w4a8_gemm_fused(p, p, p, p, p, 0, 4, 64, 100, 0, None, 0, None) == -2  # K % 128
    assert lib.lq_scale_epilogue(p, p, p, p, 7, 4, 4, None) == -1          # unknown dtype


def test_operator_schemas_match_the_reference():
    from liquidgemm_b200 import ops
    want = {
        "dequant_weight": "liquidgemm::dequant_weight(Tensor qweight, Tensor s_u8, Tensor offset_a, int N, int K, int group_size) -> Tensor",
        "quant_per_token": "liquidgemm::quant_per_token(Tensor x) -> Tensor[]",
        "w4a8_gemv2": "liquidgemm::w4a8_gemv2(Tensor x_i8, Tensor gpack, Tensor s_u8, Tensor off_a, Tensor ascale, Tensor s1, int N, int K, int group_size, int out_dtype) -> Tensor",
        "w4a8_wgmma_rs": "liquidgemm::w4a8_wgmma_rs(Tensor x_i8, Tensor w, Tensor spack, Tensor s_u8, Tensor off_a, int N, int K, int group_size, bool packed) -> Tensor",
    }
    for name, schema in want.items():
        assert str(getattr(torch.ops.liquidgemm, name).default._schema) == schema
    if have_reference():
        src = open(os.path.join(REFERENCE_ROOT, "csrc", "liquid_gemm", "torch_bindings.cpp")).read()
        joined = re.sub(r'"\s*\n\s*"', "", src)
        for name, sig in ops._SCHEMAS.items():
            if name in ("i8_gemm_scaled", "w4a8_linear_bias", "wgmma_rs_a_coords"):
                continue
            assert (name + sig) in joined, f"schema of {name} differs from the reference's torch_bindings.cpp"


def test_fake_kernels_shapes_and_dtypes():
    from liquidgemm_b200 import ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        M, N, K = 5, 256, 512
        x = torch.empty(M, K, dtype=torch.int8, device="cuda")
        u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device="cuda")
        f32 = lambda *s: torch.empty(*s, dtype=torch.float32, device="cuda")
        T = torch.ops.liquidgemm
        assert T.dequant_weight(u8(N, K), u8(N, 8), u8(N, 8), N, K, 64).shape == (N, K)
        q, s = T.quant_per_token(torch.empty(M, K, dtype=torch.bfloat16, device="cuda"))
        assert q.dtype == torch.int8 and s.shape == (M,)
        for code, dt in ((0, torch.bfloat16), (1, torch.float16), (2, torch.float32)):
            assert T.scale_epilogue(torch.empty(M, N, dtype=torch.int32, device="cuda"), f32(M), f32(N), code).dtype == dt
            assert T.w4a8_gemv2(x, u8(N, K // 2), u8(N, 8), u8(N, 8), f32(M), f32(N), N, K, 64, code).dtype == dt
            assert T.w4a8_wgmma_rs_fused(x, u8(2 * 4 * 8704), u8(N, 8), u8(N, 8), f32(M), f32(N), N, K, 64, code).shape == (M, N)
        assert T.w4a8_wgmma_rs(x, u8(1), u8(1), u8(N, 8), u8(N, 8), N, K, 64, True).dtype == torch.int32
        assert T.w4a8_wgmma(x, u8(N, K // 2), u8(N, 8), u8(N, 8), N, K, 64).shape == (M, N)
        assert T.wgmma_i8_gemm(x, torch.empty(N, K, dtype=torch.int8, device="cuda")).shape == (M, N)
        assert T.w4a8_gemm(x, u8(N, K // 2), u8(N, 8), u8(N, 8), f32(N), f32(M), N, K, 64).dtype == torch.float32


def test_host_side_packs():
    from liquidgemm_b200 import ops
    qw = random_lqq(200, 512, 64, seed=3)
    tq = to_torch_qw(qw, device="cpu")
    assert np.array_equal(ops.pack_gemv_interleaved(tq).numpy(), O.pack_gemv_interleaved(qw))
    sp = ops.build_rs_scale_pack(tq).numpy()           # [2, 4, 128, 4]
    assert sp.shape == (2, 4, 128, 4)
    for n in (0, 77, 199):
        for kt in range(4):
            want = [qw.s_u8[n, 2 * kt], qw.offset_a[n, 2 * kt], qw.s_u8[n, 2 * kt + 1], qw.offset_a[n, 2 * kt + 1]]
            assert sp[n // 128, kt, n % 128].tolist() == want
    assert sp[1, 0, 100].tolist() == [1, 128, 1, 128]   # padding rows reconstruct to zero
    assert ops.tile_coords().shape == (128, 128, 2)


def test_ops_reject_cpu_tensors():
    from liquidgemm_b200 import ops  # noqa: F401
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.liquidgemm.quant_per_token(torch.zeros(2, 16))


def test_plugin_mode_logic(monkeypatch):
    from liquidgemm_b200 import vllm_plugin as vp
    monkeypatch.delenv("LIQUIDGEMM_W4", raising=False)
    monkeypatch.delenv("LIQUIDGEMM_GEMV", raising=False)
    assert vp.mode_from_env(False) == (False, False) and vp.mode_from_env(True) == (True, False)
    monkeypatch.setenv("LIQUIDGEMM_W4", "1")
    monkeypatch.setenv("LIQUIDGEMM_GEMV", "1")
    assert vp.mode_from_env(False) == (True, True)
    monkeypatch.setenv("LIQUIDGEMM_W4", "0")
    assert vp.mode_from_env(True)[0] is False
    assert vp.layer_is_aligned(6144, 4096, 64, True) and not vp.layer_is_aligned(6144, 4000, 64, True)
    assert not vp.layer_is_aligned(100, 4096, 64, True) and vp.layer_is_aligned(100, 4096, 64, False)
    monkeypatch.setenv("VLLM_CACHE_ROOT", "/tmp/vc")
    vp._salt_compile_cache("w4-gemv")
    assert os.environ["VLLM_CACHE_ROOT"] == "/tmp/vc/liquidgemm-w4-gemv"
    vp._salt_compile_cache("w4-gemv")
    assert os.environ["VLLM_CACHE_ROOT"] == "/tmp/vc/liquidgemm-w4-gemv"


@pytest.mark.skipif(not have_reference(), reason="reference tree not mounted")
def test_quantiser_matches_imported_reference_on_fresh_inputs():
    """Differential test against the reference's own modules on inputs that are not in the fixtures."""
    import importlib.util
    import sys
    spec = importlib.util.spec_from_file_location("ref_lq_quant", os.path.join(REFERENCE_ROOT, "liquidgemm", "quant.py"))
    ref = importlib.util.module_from_spec(spec)
    sys.modules["ref_lq_quant"] = ref
    spec.loader.exec_module(ref)
    from liquidgemm_b200 import quant
    g = torch.Generator().manual_seed(123)
    for (N, K, grp) in [(96, 512, 64), (64, 384, 128), (40, 256, 32)]:
        W = torch.randn(N, K, generator=g) * 0.02
        W = torch.where(torch.rand(N, K, generator=g) < 0.002, W * 20, W)
        X = torch.randn(7, K, generator=g)
        a, b = ref.quantize_weight(W, grp), quant.quantize_weight(W, grp)
        c = O.quantize_weight(W.numpy(), grp)
        for f in ("qweight_u4", "s_u8", "offset_a", "s1"):
            assert torch.equal(getattr(a, f), getattr(b, f)), f
            assert np.array_equal(getattr(a, f).numpy(), getattr(c, f)), f
        xa, sa = ref.quantize_activation(X)
        xb, sb = quant.quantize_activation(X)
        assert torch.equal(xa, xb) and torch.equal(sa, sb)
        assert torch.equal(ref.w4a8_matmul(xa, sa, a), quant.w4a8_matmul(xb, sb, b))
        assert np.array_equal(ref.w4a8_matmul(xa, sa, a).numpy(), O.w4a8_matmul(xa.numpy(), sa.numpy(), c))
