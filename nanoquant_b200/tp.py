"""Output-dimension tensor parallelism for one quantised linear.

The reference has no distributed code.  For 70B-class layers the second factor
``U [M, R]`` is split by output rows over the G GPUs of one node: rank g keeps rows
``[g*M/G, (g+1)*M/G)`` of ``U`` and the matching slice of ``scale_post``; ``V``,
``scale_pre``, ``scale_mid`` and the activations are replicated, so the small rank-R
intermediate is computed redundantly on every GPU and the only exchange is one
all-gather of the ``[T, M/G]`` output shards (NCCL over NVLink, issued on the compute
stream).  Per-GPU bytes: ``R*N/8 + R*M/(8G)`` + scales + activations.

Two collectives are available: NCCL (``gather_outputs``) and ``PeerGather``, one small kernel per call that
stores the shard into every rank's symmetric-memory buffer with plain peer stores and waits (bounded) for the
peers' flags, which can be captured in a CUDA graph together with the GEMV / GEMM launches.  No TMA multicast
and no multimem is involved anywhere.
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


class PeerGather:
    """All-gather over peer memory (``nq_allgather_push``) on a symmetric-memory arena.

    ``PeerGather(nbytes, group)`` allocates ``nbytes`` of gather regions (plus the flag words) in symmetric
    memory on every rank.  ``region(shape, dtype)`` carves a ``[world, *shape]`` region out of the arena;
    ``gather(shard, region)`` launches the push on the current stream and returns the region, which holds
    every rank's shard once the kernel has completed (stream order).  Consecutive gathers must use different
    regions.  Multicast objects are not created (``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` is set before the
    rendezvous)."""

    FLAGS_BYTES = 256

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        self._lib, self._L, self._ct = _lib, _lib.lib(), ctypes
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        total = self.FLAGS_BYTES + (nbytes + 255) // 256 * 256
        self.arena = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, group)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        assert bases[self.rank] == self.arena.data_ptr()
        self._bases = (ctypes.c_void_p * self.world)(*bases)
        self.state = torch.zeros(self._L.nq_allgather_state_bytes(), dtype=torch.uint8, device=device)
        self._next = self.FLAGS_BYTES
        torch.cuda.synchronize(device)
        dist.barrier(group)     # every rank has zeroed its flags before anybody signals

    def region(self, shape, dtype) -> torch.Tensor:
        """A ``[world, *shape]`` view of the arena (same offset on every rank: call in the same order everywhere)."""
        n = self.world * int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        if self._next + n > self.arena.numel():
            raise RuntimeError("PeerGather arena exhausted")
        view = self.arena[self._next:self._next + n].view(dtype).view(self.world, *shape)
        self._next += (n + 255) // 256 * 256
        return view

    def gather(self, shard: torch.Tensor, region: torch.Tensor) -> torch.Tensor:
        if not shard.is_contiguous() or shard.numel() * shard.element_size() * self.world != region.numel() * region.element_size():
            raise ValueError("shard must be contiguous and 1/world of the region")
        off = region.data_ptr() - self.arena.data_ptr()
        st = self._L.nq_allgather_push(shard.data_ptr(), shard.numel() * shard.element_size(), self._bases, 0, off,
                                       self.state.data_ptr(), self.world, self.rank,
                                       torch.cuda.current_stream(shard.device).cuda_stream)
        self._lib.check(st, "nq_allgather_push")
        return region

    def status(self) -> int:
        return self._L.nq_allgather_status(self.state.data_ptr(), torch.cuda.current_stream(self.arena.device).cuda_stream)
