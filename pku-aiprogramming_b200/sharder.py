"""Batch x head sharder: spreads the B*H independent attention slices over the ranks of one
process group (one process per GPU) and all-gathers the outputs.

Every (batch, head) slice is independent in forward and backward, so no collective sits
on the data path; the only exchange is an all-gather of O.  `[B,H,S,D]` is contiguous in
the flattened slice index, so each rank's shard of O is one contiguous block and
`all_gather_into_tensor` lands the final layout without a repack.  Gradients stay with
the rank that owns the slice.

The compute callbacks default to the CUDA kernels of this package; tests inject their own
to exercise the partitioning and gathering logic on CPU ranks (gloo).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import capi


class SliceSharder:
    def __init__(self, n_slices: int, world: Optional[int] = None, rank: Optional[int] = None, group=None):
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_slices, self.world, self.rank, self.group = int(n_slices), int(world), int(rank), group
        self.begin, self.count = capi.shard_range(n_slices, world, rank)
        self.even = (n_slices % world) == 0

    # ---- views -------------------------------------------------------------------------
    def shard_of(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's contiguous block of a `[B,H,...]` tensor, as `[1,count,...]`."""
        flat = full.reshape(self.n_slices, *full.shape[2:])
        return flat[self.begin:self.begin + self.count].unsqueeze(0)

    def range_of(self, rank: int):
        return capi.shard_range(self.n_slices, self.world, rank)

    # ---- collective --------------------------------------------------------------------
    def all_gather(self, shard: torch.Tensor, out_full: Optional[torch.Tensor] = None, async_op: bool = False):
        """Gathers `[1,count,rows,D]` shards into `[n_slices,rows,D]` (returned flat in the slice
        index).  Returns (tensor, work-or-None)."""
        tail = tuple(shard.shape[2:])
        if out_full is None:
            out_full = torch.empty((self.n_slices, *tail), dtype=shard.dtype, device=shard.device)
        if self.world == 1:
            out_full.copy_(shard.reshape(self.count, *tail))
            return out_full, None
        if self.even:
            work = dist.all_gather_into_tensor(out_full, shard.reshape(self.count, *tail).contiguous(),
                                               group=self.group, async_op=async_op)
            return out_full, work
        # uneven split: pad every shard to the largest count, gather, then compact
        max_count = -(-self.n_slices // self.world)
        padded = torch.zeros((max_count, *tail), dtype=shard.dtype, device=shard.device)
        padded[:self.count].copy_(shard.reshape(self.count, *tail))
        tmp = torch.empty((self.world * max_count, *tail), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(tmp, padded, group=self.group)
        for r in range(self.world):
            b, c = self.range_of(r)
            out_full[b:b + c].copy_(tmp[r * max_count:r * max_count + c])
        return out_full, None

    # ---- sharded op ----------------------------------------------------------------------
    def forward(self, q, k, v, causal=False, scale=None, fwd: Optional[Callable] = None, gather: bool = True):
        """q,k,v: this rank's shards `[1,count,rows,D]`.  Returns (out_shard, lse_shard, out_full)."""
        if fwd is None:
            from .functional import attention_forward as fwd
        out, lse = fwd(q, k, v, causal=causal, scale=scale)
        full = None
        if gather:
            full, _ = self.all_gather(out)
        return out, lse, full
