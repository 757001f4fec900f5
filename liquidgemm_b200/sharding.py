"""Column (output-channel) sharding of LQQ linears across the GPUs of one node.

Every LQQ quantity is per output channel -- row scales ``s1[N]``, group steps/offsets ``[N, G]``,
weight rows -- so rank r of P owns rows ``[r*N/P, (r+1)*N/P)`` and quantises / prepacks them with no
cross-rank statistic; quantising a shard equals slicing the quantised full matrix.  Activations
are replicated.  The only exchange is an all-gather of the ``[M, N/P]`` outputs along N, issued
only where the consumer needs the full vector.  The reference has no distributed code at all
(under vLLM tensor parallelism it only receives per-partition sizes,
liquidgemm/vllm_plugin.py:115-134); this module is what its benchmark configuration for
70B-shape layers on 1/2/4/8 GPUs needs.
"""

from __future__ import annotations

import torch

from .quant import LiquidQuantWeight


def shard_range(n_rows: int, rank: int, world: int, align: int = 64) -> tuple[int, int]:
    """Rows owned by ``rank``: equal contiguous blocks, each a multiple of ``align`` rows."""
    if n_rows % (world * align):
        raise ValueError(f"N={n_rows} cannot be split into {world} shards of a multiple of {align} rows")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def shard_weight(qw: LiquidQuantWeight, rank: int, world: int, align: int = 64) -> LiquidQuantWeight:
    """The rank's slice of a quantised weight (views, no copy)."""
    lo, hi = shard_range(qw.N, rank, world, align)
    return LiquidQuantWeight(qw.qweight_u4[lo:hi], qw.s_u8[lo:hi], qw.offset_a[lo:hi], qw.s1[lo:hi], qw.group_size)


def gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather ``[M, N/P]`` shards into ``[M, N]`` (NCCL over NVLink on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m, n_local = y_local.shape
    stacked = torch.empty((world * m, n_local), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stacked, y_local.contiguous(), group=group)
    return stacked.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)
