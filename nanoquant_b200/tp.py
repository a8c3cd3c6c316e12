"""Output-dimension tensor parallelism for one quantised linear.

The reference has no distributed code.  For 70B-class layers the second factor
``U [M, R]`` is split by output rows over the G GPUs of one node: rank g keeps rows
``[g*M/G, (g+1)*M/G)`` of ``U`` and the matching slice of ``scale_post``; ``V``,
``scale_pre``, ``scale_mid`` and the activations are replicated, so the small rank-R
intermediate is computed redundantly on every GPU and the only exchange is one
all-gather of the ``[T, M/G]`` output shards (NCCL over NVLink, issued on the compute
stream).  Per-GPU bytes: ``R*N/8 + R*M/(8G)`` + scales + activations.

Nothing here reads another GPU's memory directly and no TMA multicast is involved.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_bounds(M: int, world: int, rank: int, multiple: int = 16):
    """Row range of `rank`; every shard is a multiple of `multiple` rows (a tile row group)."""
    if M % (world * multiple):
        raise ValueError(f"out_features {M} is not a multiple of world size {world} x {multiple}")
    per = M // world
    return rank * per, (rank + 1) * per


def shard_rows_tiles(u_tiles: torch.Tensor, M: int, world: int, rank: int) -> torch.Tensor:
    """Slice of a tile-layout factor ``[M/16, chunks, 128]`` holding this rank's output rows.
    Row groups of 16 rows are contiguous in the tile layout, so the shard is a view."""
    lo, hi = shard_bounds(M, world, rank)
    return u_tiles[lo // 16: hi // 16]


def shard_rows_packed(u_packed: torch.Tensor, M: int, world: int, rank: int) -> torch.Tensor:
    """The same for a rows-layout factor ``[M, R/32]`` (checkpoint or ``half2`` words)."""
    lo, hi = shard_bounds(M, world, rank)
    return u_packed[lo:hi]


@dataclass
class TPLinearShard:
    """What one rank holds of a layer."""
    v_tiles: torch.Tensor            # [R/16, ceil(N/256), 128], replicated
    u_tiles: torch.Tensor            # this rank's rows of U
    s_in: torch.Tensor               # [N], replicated
    s_mid: Optional[torch.Tensor]    # [R], replicated
    s_out: torch.Tensor              # [M/G]
    N: int
    R: int
    M: int                           # full output width
    world: int
    rank: int

    @classmethod
    def from_full(cls, v_tiles, u_tiles, s_in, s_mid, s_out, N, R, M, world, rank):
        lo, hi = shard_bounds(M, world, rank)
        return cls(v_tiles, shard_rows_tiles(u_tiles, M, world, rank).contiguous(), s_in, s_mid,
                   s_out[lo:hi].contiguous(), N, R, M, world, rank)


def gather_outputs(y_local: torch.Tensor, world: int, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather ``[T, M/G]`` shards into ``[T, M]`` (rank-major along the last dimension)."""
    T, m = y_local.shape
    if world == 1:
        return y_local
    if T == 1:
        # one token: the rank-major concatenation IS the row; gather straight into the output
        full = out if out is not None else torch.empty((1, world * m), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(full.view(-1), y_local.reshape(-1), group=group)
        return full
    stage = torch.empty((world * T, m), dtype=y_local.dtype, device=y_local.device)   # rank-major concatenation
    dist.all_gather_into_tensor(stage, y_local.contiguous(), group=group)
    full = stage.view(world, T, m).permute(1, 0, 2).reshape(T, world * m)
    if out is not None:
        out.copy_(full)
        return out
    return full


def tp_linear_forward(x: torch.Tensor, shard: TPLinearShard, group=None,
                      local_fn: Optional[Callable] = None) -> torch.Tensor:
    """``y[T, M]`` on every rank.  ``local_fn(x, shard) -> [T, M/G]`` computes the local shard;
    by default the CUDA kernels through ``nq_linear_fwd``."""
    if local_fn is None:
        from . import ops
        y_local = ops.linear_forward(x, shard.s_in, shard.v_tiles, shard.s_mid, shard.u_tiles, shard.s_out, shard.R)
    else:
        y_local = local_fn(x, shard)
    return gather_outputs(y_local, shard.world, group=group)
