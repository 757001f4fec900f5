"""Helpers shared by the GPU parity tests: seeded LQQ data and bit-level comparisons."""

from __future__ import annotations

import numpy as np
import torch

from oracle import lqq_oracle as O

LLAMA8B = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}


def random_lqq(N: int, K: int, group: int = 64, seed: int = 0) -> O.LQQWeight:
    """A valid LQQ weight drawn directly in code space: every step in 1..16 and every offset that
    keeps code*step + offset within 0..255 is reachable, which is harsher than quantising a
    Gaussian (and much cheaper for the full-size shapes)."""
    rng = np.random.default_rng(seed)
    G = K // group
    codes = rng.integers(0, 16, (N, K), dtype=np.uint8)
    step = rng.integers(1, 17, (N, G), dtype=np.int32)
    room = 255 - 15 * step
    off = (rng.random((N, G)) * (room + 1)).astype(np.int32)
    off = np.minimum(off, room)
    s1 = (rng.random(N, dtype=np.float32) * np.float32(0.01) + np.float32(1e-4)).astype(np.float32)
    return O.LQQWeight(codes, step.astype(np.uint8), off.astype(np.uint8), s1, group)


def random_tokens(M: int, K: int, seed: int = 1):
    rng = np.random.default_rng(seed)
    x = rng.integers(-127, 128, (M, K), dtype=np.int8)   # +127 included
    ascale = (rng.random(M, dtype=np.float32) * np.float32(0.02) + np.float32(0.01)).astype(np.float32)
    return x, ascale


def to_torch_qw(qw: O.LQQWeight, device="cuda"):
    from liquidgemm_b200.quant import LiquidQuantWeight
    return LiquidQuantWeight(torch.from_numpy(qw.qweight_u4).to(device), torch.from_numpy(qw.s_u8).to(device),
                             torch.from_numpy(qw.offset_a).to(device), torch.from_numpy(qw.s1).to(device),
                             qw.group_size)


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw bit patterns of a bf16/fp16 tensor as uint16, fp32 as uint32, ints unchanged."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float32:
        return t.numpy().view(np.uint32)
    return t.numpy()


def expected_bits(y_f32: np.ndarray, out_dtype: int) -> np.ndarray:
    e = O.cast_out_bits(y_f32, out_dtype)
    return e.view(np.uint32) if out_dtype == O.OUT_F32 else e


def assert_bits_equal(got: torch.Tensor, y_f32: np.ndarray, out_dtype: int, what: str = ""):
    g = bits(got)
    e = expected_bits(y_f32, out_dtype)
    if not np.array_equal(g, e):
        bad = np.argwhere(g != e)
        raise AssertionError(f"{what}: {len(bad)} of {g.size} elements differ; first at {bad[0].tolist()}: "
                             f"got 0x{int(g[tuple(bad[0])]):x} want 0x{int(e[tuple(bad[0])]):x}")


def bits_to_f32(b: np.ndarray, out_dtype: int) -> np.ndarray:
    """Exact float32 value of bf16 / fp16 / fp32 bit patterns."""
    if out_dtype == O.OUT_BF16:
        return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)
    if out_dtype == O.OUT_F16:
        return b.view(np.float16).astype(np.float32)
    return b.view(np.float32)


def with_bias_f32(y_f32: np.ndarray, bias_bits: np.ndarray, out_dtype: int) -> np.ndarray:
    """What ``y.to(T) + bias`` gives in PyTorch for T = bf16 / fp16 / fp32 (the reference adds the bias to
    the already cast output, liquidgemm/vllm_plugin.py:205-206): round the product to T, add the bias in
    float32, round again (the caller casts the returned float32 to T)."""
    y_t = bits_to_f32(expected_bits(y_f32, out_dtype), out_dtype)
    return (y_t + bits_to_f32(bias_bits, out_dtype)[None, :]).astype(np.float32)
