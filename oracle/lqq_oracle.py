"""CPU oracle for the LiquidQuant (LQQ) W4A8 linear path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the arithmetic of the reference's pure-PyTorch ground truth
(``liquidgemm/quant.py`` and ``liquidgemm/pack.py``) plus the operator-level formulas of its
CUDA entry points, so that the CUDA kernels of this repository can be compared bit for bit
against something that runs on any host.  Nothing in the product package may import it: only
the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.

Parity status: **pinned**.  Every function below is checked (tests/test_oracle_golden.py)
against fixtures in ``tests/golden/`` that were produced by running the reference's own
Python modules (see ``tests/golden/make_golden.py``), and -- when the reference tree is
mounted -- differentially against the imported reference on fresh seeded inputs.

Conventions: weights are ``[N, K]`` (out_features, in_features); groups run along K.
All float arithmetic is IEEE binary32 with round-to-nearest-even, matching torch on CPU.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

# reference liquidgemm/quant.py:30-32
L1_QMAX = 119      # level-1 symmetric range: 127 - 16/2
U4_MAX = 15        # level-2 code range
STEP_MAX = 16      # level-2 integer step range [1, 16]


@dataclass
class LQQWeight:
    """Mirror of ``LiquidQuantWeight`` (reference liquidgemm/quant.py:35-58) on numpy arrays."""

    qweight_u4: np.ndarray  # [N, K] uint8, 0..15
    s_u8: np.ndarray        # [N, G] uint8, 1..16
    offset_a: np.ndarray    # [N, G] uint8, 128 + group minimum
    s1: np.ndarray          # [N]    float32
    group_size: int

    @property
    def N(self) -> int:
        return int(self.qweight_u4.shape[0])

    @property
    def K(self) -> int:
        return int(self.qweight_u4.shape[1])


# --------------------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------------------

def quantize_weight(W: np.ndarray, group_size: int = 64) -> LQQWeight:
    """Two-level LQQ quantiser (reference liquidgemm/quant.py:61-100).

    Level 1: ``s1 = max(amax_row, 1e-12) / 119``; ``q = clamp(rint(W / s1), -119, 119)``.
    Level 2 per group of ``group_size`` along K: ``step = clamp(ceil((max-min)/15), 1, 16)``,
    ``code = clamp(rint((q - min) / step), 0, 15)``, ``offset = 128 + min``.
    ``np.rint`` rounds half to even exactly like ``torch.round``.
    """
    W = np.asarray(W)
    assert W.ndim == 2
    N, K = W.shape
    assert K % group_size == 0
    G = K // group_size
    Wf = W.astype(np.float32)

    amax = np.abs(Wf).max(axis=1)
    s1 = (np.maximum(amax, np.float32(1e-12)) / np.float32(L1_QMAX)).astype(np.float32)
    q = np.rint(Wf / s1[:, None]).astype(np.float32)
    q = np.clip(q, -L1_QMAX, L1_QMAX).astype(np.int32)

    qg = q.reshape(N, G, group_size)
    lo = qg.min(axis=2)
    hi = qg.max(axis=2)
    step = np.ceil((hi - lo).astype(np.float32) / np.float32(U4_MAX))
    step = np.clip(step, 1, STEP_MAX).astype(np.int32)
    code = np.rint((qg - lo[:, :, None]).astype(np.float32) / step[:, :, None].astype(np.float32))
    code = np.clip(code, 0, U4_MAX).astype(np.int32).reshape(N, K)
    off = (128 + lo).astype(np.int32)

    # invariants asserted by the reference (quant.py:88-92)
    assert step.min() >= 1 and step.max() <= STEP_MAX
    u = code.reshape(N, G, group_size) * step[:, :, None] + off[:, :, None]
    assert u.min() >= 0 and u.max() <= 255
    return LQQWeight(code.astype(np.uint8), step.astype(np.uint8), off.astype(np.uint8),
                     s1, group_size)


def quantize_activation(X: np.ndarray):
    """Per-token symmetric INT8 (reference liquidgemm/quant.py:135-141).

    ``ascale = max(amax_row, 1e-12) / 127``; ``x8 = clamp(rint(X / ascale), -127, 127)``
    with a true fp32 division.
    """
    Xf = np.asarray(X).astype(np.float32)
    assert Xf.ndim == 2
    amax = np.abs(Xf).max(axis=1) if Xf.shape[1] else np.zeros(Xf.shape[0], np.float32)
    ascale = (np.maximum(amax, np.float32(1e-12)) / np.float32(127.0)).astype(np.float32)
    x8 = np.clip(np.rint(Xf / ascale[:, None]), -127, 127).astype(np.int8)
    return x8, ascale


# --------------------------------------------------------------------------------------
# dequantisers
# --------------------------------------------------------------------------------------

def _expand_groups(qw: LQQWeight):
    g = qw.group_size
    s = np.repeat(qw.s_u8.astype(np.int32), g, axis=1)
    a = np.repeat(qw.offset_a.astype(np.int32), g, axis=1)
    return s, a


def dequantize_i8_xor(qw: LQQWeight) -> np.ndarray:
    """``(code*step + offset) XOR 0x80`` as int8 (reference liquidgemm/quant.py:103-112)."""
    s, a = _expand_groups(qw)
    u = (qw.qweight_u4.astype(np.int32) * s + a).astype(np.uint8)
    return (u ^ np.uint8(0x80)).view(np.int8)


def dequantize_i8_sub(qw: LQQWeight) -> np.ndarray:
    """``code*step + offset - 128`` as int8 (reference liquidgemm/quant.py:115-122)."""
    s, a = _expand_groups(qw)
    return (qw.qweight_u4.astype(np.int32) * s + a - 128).astype(np.int8)


def dequantize_i8(qw: LQQWeight) -> np.ndarray:
    """Reference liquidgemm/quant.py:125-127."""
    return dequantize_i8_xor(qw)


def dequantize(qw: LQQWeight) -> np.ndarray:
    """Float reconstruction ``q_hat * s1`` (reference liquidgemm/quant.py:130-132)."""
    return dequantize_i8(qw).astype(np.float32) * qw.s1[:, None]


# --------------------------------------------------------------------------------------
# integer GEMM + epilogue
# --------------------------------------------------------------------------------------

def int_accumulate(x_i8: np.ndarray, q_hat: np.ndarray) -> np.ndarray:
    """Exact ``x_i8 @ q_hat.T`` as int32.

    Computed through float64 BLAS: every product is an integer below 2**14 and every partial
    sum stays below K*127*128 < 2**53, so the float64 result is the exact integer
    (the reference accumulates in int32, liquidgemm/quant.py:151).
    """
    K = x_i8.shape[1]
    assert K * 127 * 128 < 2 ** 31
    acc = x_i8.astype(np.float64) @ q_hat.astype(np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def int_accumulate_slow(x_i8: np.ndarray, q_hat: np.ndarray) -> np.ndarray:
    """Same as :func:`int_accumulate` with pure integer arithmetic (small cases only)."""
    return (x_i8.astype(np.int64) @ q_hat.astype(np.int64).T).astype(np.int32)


def scale_f32(acc: np.ndarray, ascale: np.ndarray, s1: np.ndarray) -> np.ndarray:
    """``float(acc) * ascale[m] * s1[n]`` evaluated left to right in fp32
    (reference liquidgemm/quant.py:152, csrc/liquid_gemm/epilogue.cu:57)."""
    y = acc.astype(np.float32)
    y = (y * ascale.astype(np.float32)[:, None]).astype(np.float32)
    y = (y * s1.astype(np.float32)[None, :]).astype(np.float32)
    return y


def w4a8_matmul(x_i8: np.ndarray, ascale: np.ndarray, qw: LQQWeight) -> np.ndarray:
    """The parity formula (reference liquidgemm/quant.py:144-153); returns fp32 ``[M, N]``."""
    return scale_f32(int_accumulate(x_i8, dequantize_i8(qw)), ascale, qw.s1)


def f32_to_bf16_bits(y: np.ndarray) -> np.ndarray:
    """Round fp32 to bfloat16 (nearest even), returned as uint16 bit patterns."""
    b = np.ascontiguousarray(y, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b.astype(np.uint64) + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((b[nan] >> 16) | 0x0040).astype(np.uint16)
    return r


def f32_to_f16_bits(y: np.ndarray) -> np.ndarray:
    """Round fp32 to binary16 (nearest even), returned as uint16 bit patterns."""
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(y, dtype=np.float32).astype(np.float16).view(np.uint16)


OUT_BF16, OUT_F16, OUT_F32 = 0, 1, 2  # reference csrc/liquid_gemm/w4a8_wgmma.cu:626-627


def cast_out_bits(y: np.ndarray, out_dtype: int) -> np.ndarray:
    """Output cast used by every fused epilogue; returns raw bits (uint16) or fp32 values."""
    if out_dtype == OUT_BF16:
        return f32_to_bf16_bits(y)
    if out_dtype == OUT_F16:
        return f32_to_f16_bits(y)
    return np.ascontiguousarray(y, dtype=np.float32)


def scale_epilogue(acc, ascale, s1, out_dtype):
    """Reference csrc/liquid_gemm/epilogue.cu:48-59."""
    return cast_out_bits(scale_f32(acc, ascale, s1), out_dtype)


def w4a8_linear(x_i8, ascale, qw: LQQWeight, out_dtype: int):
    """What ``w4a8_wgmma_rs_fused`` / ``w4a8_gemv2`` must produce
    (reference csrc/liquid_gemm/w4a8_wgmma.cu:39-56, gemv2.cu:70-77)."""
    return cast_out_bits(w4a8_matmul(x_i8, ascale, qw), out_dtype)


# --------------------------------------------------------------------------------------
# packing
# --------------------------------------------------------------------------------------

def pack_nibbles(q_u4: np.ndarray) -> np.ndarray:
    """Two codes per byte, even k in the low nibble (reference liquidgemm/pack.py:27-32)."""
    assert q_u4.dtype == np.uint8 and q_u4.shape[-1] % 2 == 0
    return (q_u4[..., 0::2] | (q_u4[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_nibbles` (reference liquidgemm/pack.py:35-40)."""
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return out


def pack_lanes_u32(q_u4: np.ndarray) -> np.ndarray:
    """Four consecutive codes in the four byte lanes of one 32-bit word
    (reference liquidgemm/pack.py:43-52); int64 array of uint32 patterns."""
    N = q_u4.shape[0]
    v = q_u4.astype(np.int64).reshape(N, -1, 4)
    return v[..., 0] | (v[..., 1] << 8) | (v[..., 2] << 16) | (v[..., 3] << 24)


def simd_dequant_u32(qw: LQQWeight) -> np.ndarray:
    """One 32-bit multiply-add and one 32-bit XOR per four codes, masked to 32 bits
    (reference liquidgemm/pack.py:55-78)."""
    N, K, g = qw.N, qw.K, qw.group_size
    assert g % 4 == 0
    words = pack_lanes_u32(qw.qweight_u4)
    s = np.repeat(qw.s_u8.astype(np.int64), g // 4, axis=1)
    a = np.repeat(qw.offset_a.astype(np.int64), g // 4, axis=1) * 0x01010101
    w = (((words * s) & 0xFFFFFFFF) + a) & 0xFFFFFFFF
    w ^= 0x80808080
    lanes = np.stack([(w >> (8 * i)) & 0xFF for i in range(4)], axis=-1)
    return lanes.reshape(N, K).astype(np.uint8).view(np.int8)


def pack_gemv_interleaved(qw: LQQWeight) -> np.ndarray:
    """Row-major ``[N, K/2]`` where byte b of octet h is ``w[8h+b] | w[8h+4+b] << 4``
    (reference liquidgemm/ops.py:68-75)."""
    q = qw.qweight_u4
    N, K = q.shape
    o = q.reshape(N, K // 8, 2, 4)
    return (o[:, :, 0, :] | (o[:, :, 1, :] << 4)).astype(np.uint8).reshape(N, K // 2)


# --------------------------------------------------------------------------------------
# seeded synthetic inputs shared by tests and the benchmark
# --------------------------------------------------------------------------------------

def synth_weight(N: int, K: int, seed: int = 0, outlier_frac: float = 1e-3) -> np.ndarray:
    """fp16 weights ~N(0, 0.02) with ``outlier_frac`` of the entries scaled by 20."""
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
    mask = rng.random((N, K), dtype=np.float32) < outlier_frac
    W[mask] *= np.float32(20.0)
    return W.astype(np.float16)


def synth_activation(M: int, K: int, seed: int = 1, hot_channel_frac: float = 0.0) -> np.ndarray:
    """fp16 activations ~N(0, 1); optionally a fraction of the K channels scaled by 10."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((M, K), dtype=np.float32)
    if hot_channel_frac > 0:
        n_hot = max(1, int(round(K * hot_channel_frac)))
        cols = rng.permutation(K)[:n_hot]
        X[:, cols] *= np.float32(10.0)
    return X.astype(np.float16)
