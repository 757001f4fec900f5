"""LiquidQuant (LQQ) quantisers and the integer-domain reference formula, on torch tensors.

Same public names and semantics as liquidgemm/quant.py of the reference (cited per function);
the code is device agnostic and is what the vLLM method runs once per layer at load time.

Scheme.  A weight row is first mapped to INT8 with a per-row scale and a *protective* range of
+-119, then each run of ``group_size`` values along K is re-coded as 4-bit codes with an
integer step in 1..16 and an 8-bit offset ``a = 128 + min``.  Reconstruction is

    u = code * step + a        (always within 0..255, so it never carries between byte lanes)
    q_hat = u XOR 0x80         (biased byte -> two's complement, equal to u - 128)
    w_hat = q_hat * s1

The 8-count margin under 127 is half of the largest step, so rounding at level 2 can not leave
the INT8 range.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

INT8_PROTECTIVE_MAX = 119   # reference liquidgemm/quant.py:30
UINT4_MAX = 15              # reference liquidgemm/quant.py:31
S_U8_MAX = 16               # reference liquidgemm/quant.py:32


@dataclass
class LiquidQuantWeight:
    """Quantised weight container (reference liquidgemm/quant.py:35-58).

    ``qweight_u4`` [N, K] uint8 codes 0..15 (one per byte), ``s_u8`` [N, G] uint8 steps 1..16,
    ``offset_a`` [N, G] uint8 offsets, ``s1`` [N] float32 row scales, G = K // group_size.
    """

    qweight_u4: torch.Tensor
    s_u8: torch.Tensor
    offset_a: torch.Tensor
    s1: torch.Tensor
    group_size: int

    # ``qweight_u4`` may be None when the codes were packed straight into a tile blob and never stored one
    # per byte (liquidgemm_b200.ops.quantize_weight_cuda(..., want_codes=False)); the sizes then come from
    # the group arrays.
    @property
    def N(self) -> int:
        return self.s_u8.shape[0]

    @property
    def K(self) -> int:
        return self.s_u8.shape[1] * self.group_size

    def to(self, device) -> "LiquidQuantWeight":
        """Copy of the container with every tensor on ``device``."""
        codes = None if self.qweight_u4 is None else self.qweight_u4.to(device)
        return LiquidQuantWeight(codes, self.s_u8.to(device), self.offset_a.to(device), self.s1.to(device),
                                 self.group_size)


def _const(like: torch.Tensor, value: float) -> torch.Tensor:
    """0-dim float32 tensor on the device of ``like`` (see the note on division in quantize_weight)."""
    return torch.tensor(float(value), dtype=torch.float32, device=like.device)


def quantize_weight(W: torch.Tensor, group_size: int = 64) -> LiquidQuantWeight:
    """Quantise ``W`` [N, K] (reference liquidgemm/quant.py:61-100)."""
    if W.dim() != 2:
        raise AssertionError("expected [N, K]")
    n_rows, n_cols = W.shape
    if n_cols % group_size:
        raise AssertionError(f"K={n_cols} not divisible by group_size={group_size}")
    n_groups = n_cols // group_size
    if W.is_cuda and n_cols % 128 == 0 and group_size in (64, 128) and \
            W.dtype in (torch.float32, torch.float16, torch.bfloat16):
        # on the device the whole quantiser is two kernels of the native library (same bits as below)
        from . import ops
        return ops.quantize_weight_cuda(W, group_size, want_codes=True, want_blob=False)[0]
    w32 = W.detach().to(torch.float32)

    # level 1: one symmetric scale per output channel.  The divisor is a tensor on purpose: torch's
    # CUDA kernels turn division by a Python scalar into a multiplication by its reciprocal, which
    # can differ from the CPU result in the last bit; tensor / tensor is an IEEE division everywhere.
    row_scale = w32.abs().amax(dim=1).clamp_min(1e-12) / _const(w32, INT8_PROTECTIVE_MAX)
    q8 = torch.round(w32 / row_scale.unsqueeze(1))
    q8 = q8.clamp_(-INT8_PROTECTIVE_MAX, INT8_PROTECTIVE_MAX).to(torch.int32)

    # level 2: asymmetric 4-bit codes with an integer step per group
    grouped = q8.view(n_rows, n_groups, group_size)
    g_lo = grouped.amin(dim=2)
    g_hi = grouped.amax(dim=2)
    # ceil(range / 15) in integers: identical to the float form for 0 <= range <= 238, on any device
    step = torch.div(g_hi - g_lo + (UINT4_MAX - 1), UINT4_MAX, rounding_mode="floor").clamp_(1, S_U8_MAX)
    step = step.to(torch.int32)
    codes = torch.round((grouped - g_lo.unsqueeze(2)).to(torch.float32) / step.unsqueeze(2).to(torch.float32))
    codes = codes.clamp_(0, UINT4_MAX).to(torch.int32)
    offset = (g_lo + 128).to(torch.int32)

    # the guarantees the packed dequant relies on; one host read instead of five
    recon = codes * step.unsqueeze(2) + offset.unsqueeze(2)
    bounds = torch.stack([step.amin(), step.amax(), recon.amin(), recon.amax()]).tolist()
    if not (bounds[0] >= 1 and bounds[1] <= S_U8_MAX and bounds[2] >= 0 and bounds[3] <= 255):
        raise AssertionError(f"LQQ overflow invariant violated: {bounds}")

    return LiquidQuantWeight(
        qweight_u4=codes.view(n_rows, n_cols).to(torch.uint8),
        s_u8=step.to(torch.uint8),
        offset_a=offset.to(torch.uint8),
        s1=row_scale.to(torch.float32),
        group_size=group_size,
    )


def _biased_u8(qw: LiquidQuantWeight) -> torch.Tensor:
    g = qw.group_size
    codes = qw.qweight_u4.to(torch.int32).view(qw.N, qw.K // g, g)
    u = codes * qw.s_u8.to(torch.int32).unsqueeze(2) + qw.offset_a.to(torch.int32).unsqueeze(2)
    return u.view(qw.N, qw.K)


def _dequant_i8_via_xor(qw: LiquidQuantWeight) -> torch.Tensor:
    """``(code*step + a) XOR 0x80`` (reference liquidgemm/quant.py:103-112)."""
    u8 = _biased_u8(qw).to(torch.uint8)
    return (u8 ^ 0x80).view(torch.int8)


def _dequant_i8_via_sub(qw: LiquidQuantWeight) -> torch.Tensor:
    """``code*step + a - 128`` (reference liquidgemm/quant.py:115-122)."""
    return (_biased_u8(qw) - 128).to(torch.int8)


def dequantize_i8(qw: LiquidQuantWeight) -> torch.Tensor:
    """INT8 reconstruction, XOR form (reference liquidgemm/quant.py:125-127)."""
    return _dequant_i8_via_xor(qw)


def dequantize(qw: LiquidQuantWeight) -> torch.Tensor:
    """Float reconstruction [N, K] (reference liquidgemm/quant.py:130-132)."""
    return dequantize_i8(qw).to(torch.float32) * qw.s1.unsqueeze(1)


def quantize_activation(X: torch.Tensor):
    """Per-token symmetric INT8; returns ``(x_i8, ascale)`` (reference liquidgemm/quant.py:135-141)."""
    if X.dim() != 2:
        raise AssertionError("expected [M, K]")
    x32 = X.detach().to(torch.float32)
    ascale = x32.abs().amax(dim=1).clamp_min(1e-12) / _const(x32, 127.0)
    x_i8 = torch.round(x32 / ascale.unsqueeze(1)).clamp_(-127, 127).to(torch.int8)
    return x_i8, ascale.to(torch.float32)


def w4a8_matmul(x_i8: torch.Tensor, ascale: torch.Tensor, qw: LiquidQuantWeight) -> torch.Tensor:
    """``Y[m,n] = float(sum_k x[m,k]*q_hat[n,k]) * ascale[m] * s1[n]`` in fp32
    (reference liquidgemm/quant.py:144-153).  This is the formula every fused kernel matches."""
    q_hat = dequantize_i8(qw).to(torch.int32)
    acc = x_i8.to(torch.int32) @ q_hat.t()
    return acc.to(torch.float32) * ascale.unsqueeze(1) * qw.s1.unsqueeze(0)
