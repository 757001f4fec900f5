"""Nibble and byte-lane packing helpers (same names as liquidgemm/pack.py of the reference).

``simd_dequant_u32`` evaluates the packed dequant the way the GPU does -- one 32-bit
multiply-add and one 32-bit XOR for four codes -- with every intermediate masked to 32 bits,
so that a carry between byte lanes, if one were possible, would show up as a wrong neighbour.
"""

from __future__ import annotations

import torch

from .quant import LiquidQuantWeight

MASK32 = 0xFFFFFFFF


def pack_nibbles(q_u4: torch.Tensor) -> torch.Tensor:
    """[.., K] codes -> [.., K/2] bytes, even k in the low nibble (reference liquidgemm/pack.py:27-32)."""
    if q_u4.dtype != torch.uint8 or q_u4.shape[-1] % 2:
        raise AssertionError("expected uint8 codes with an even last dimension")
    pairs = q_u4.reshape(*q_u4.shape[:-1], q_u4.shape[-1] // 2, 2)
    return (pairs[..., 0] | (pairs[..., 1] << 4)).to(torch.uint8)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_nibbles` (reference liquidgemm/pack.py:35-40)."""
    both = torch.stack([packed & 0x0F, packed >> 4], dim=-1)
    return both.reshape(*packed.shape[:-1], packed.shape[-1] * 2).to(torch.uint8)


def pack_lanes_u32(q_u4: torch.Tensor) -> torch.Tensor:
    """Four consecutive codes -> the four byte lanes of one 32-bit word, [N, K/4] int64
    (reference liquidgemm/pack.py:43-52)."""
    if q_u4.shape[-1] % 4:
        raise AssertionError("K must be a multiple of 4")
    quads = q_u4.to(torch.int64).view(q_u4.shape[0], -1, 4)
    shifts = torch.tensor([0, 8, 16, 24], dtype=torch.int64, device=q_u4.device)
    return (quads << shifts).sum(dim=-1)


def simd_dequant_u32(qw: LiquidQuantWeight) -> torch.Tensor:
    """Packed 4-lane dequant on 32-bit words -> int8 [N, K] (reference liquidgemm/pack.py:55-78)."""
    g = qw.group_size
    if g % 4:
        raise AssertionError("group_size must be a multiple of 4")
    words = pack_lanes_u32(qw.qweight_u4)
    per_word = g // 4
    step = qw.s_u8.to(torch.int64).repeat_interleave(per_word, dim=1)
    off = qw.offset_a.to(torch.int64).repeat_interleave(per_word, dim=1) * 0x01010101
    mad = (((words * step) & MASK32) + off) & MASK32
    flipped = mad ^ 0x80808080
    shifts = torch.tensor([0, 8, 16, 24], dtype=torch.int64, device=words.device)
    lanes = (flipped.unsqueeze(-1) >> shifts) & 0xFF
    return lanes.reshape(qw.N, qw.K).to(torch.uint8).view(torch.int8)
