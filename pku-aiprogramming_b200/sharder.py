"""Batch x head sharder: spreads the B*H independent attention slices over the ranks of one
process group (one process per GPU) and all-gathers the outputs.

Every (batch, head) slice is independent in forward and backward, so no collective sits
on the data path; the only exchange is an all-gather of O.  `[B,H,S,D]` is contiguous in
the flattened slice index, so each rank's shard of O is one contiguous block and
`all_gather_into_tensor` lands the final layout without a repack.  Gradients stay with
the rank that owns the slice.

`ShardedAttention` is the product path on GPUs: it drives the library's own multi-GPU entry points
(`tt_mgpu_*`: the library owns the NCCL communicator and a side stream per device, shards, launches
and all-gathers).  torch.distributed is used once, to hand rank 0's NCCL id to the other ranks.
`SliceSharder` keeps the same partition in Python over a torch process group; its compute callbacks
can be replaced, which is how the partitioning and gathering logic is exercised on CPU ranks (gloo).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import capi


class ShardedAttention:
    """One rank of a group of GPUs computing attention over all B*H slices (see `tt_mgpu_*` in
    include/tt_attn.h).  Construct it on every rank with the rank's device current:

        sa = ShardedAttention.from_process_group()          # ids travel over torch.distributed
        out, lse, out_full = sa.forward(q, k, v, B, H, causal=True)      # q, k, v: this rank's shards
        dq, dk, dv = sa.backward(q, k, v, out, lse, dout, B, H, causal=True)   # overlaps the gather of out
        sa.wait()                                            # current stream waits for the gathers
    """

    def __init__(self, world: int, rank: int, id_bytes: bytes):
        import ctypes
        self.world, self.rank = int(world), int(rank)
        self._h = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(bytes(id_bytes), 128)
        capi.check(capi.lib.tt_mgpu_init(ctypes.byref(self._h), self.world, self.rank, buf))

    @staticmethod
    def unique_id() -> bytes:
        import ctypes
        buf = ctypes.create_string_buffer(128)
        capi.check(capi.lib.tt_mgpu_unique_id(buf))
        return bytes(buf.raw)

    @classmethod
    def from_process_group(cls, group=None, device=None):
        """Rank 0 creates the NCCL id; one broadcast over the (already initialised) torch process group
        carries it to the others."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        carrier = device if dist.get_backend(group) == "nccl" else torch.device("cpu")
        t = torch.zeros(128, dtype=torch.uint8, device=carrier)
        if rank == 0:
            t.copy_(torch.frombuffer(bytearray(cls.unique_id()), dtype=torch.uint8))
        dist.broadcast(t, src=0, group=group)
        return cls(world, rank, bytes(t.cpu().numpy().tobytes()))

    def close(self):
        if self._h is not None and self._h.value:
            capi.check(capi.lib.tt_mgpu_destroy(self._h))
        self._h = None

    def _desc(self, q, k, B, H, causal, scale):
        from .functional import _DT
        count, S, D = q.shape[-3], q.shape[-2], q.shape[-1]
        if B * H != count * self.world:
            raise ValueError(f"a shard of {count} slices on each of {self.world} ranks does not make B*H = {B * H}")
        hkv_local = k.shape[-3]
        if count % hkv_local != 0:
            raise ValueError("key/value heads of the shard must divide its query heads")
        return capi.make_desc(B, H, S, k.shape[-2], D, _DT[q.dtype], causal, scale, Hkv=H // (count // hkv_local))

    def forward(self, q, k, v, B, H, causal=False, scale=None, out=None, lse=None, out_full=None, gather=True):
        """q `[1,count,S,D]`, k, v `[1,count/group,L,D]`: this rank's shards of a `[B,H,...]` problem.
        Returns (out, lse, out_full); out_full `[B*H,S,D]` is complete once `wait()` has been called and the
        stream has reached that point."""
        import ctypes
        from .functional import _p, _stream_ptr
        d = self._desc(q, k, B, H, causal, scale)
        count, S, D = q.shape[-3], q.shape[-2], q.shape[-1]
        out = torch.empty_like(q) if out is None else out
        lse = torch.empty((1, count, S), dtype=torch.float32, device=q.device) if lse is None else lse
        if gather and out_full is None:
            out_full = torch.empty((B * H, S, D), dtype=q.dtype, device=q.device)
        capi.check(capi.lib.tt_mgpu_attn_fwd(self._h, ctypes.byref(d), _p(q), _p(k), _p(v), _p(out), _p(lse),
                                             _p(out_full) if gather else None, _stream_ptr(q)))
        return out, lse, (out_full if gather else None)

    def backward(self, q, k, v, out, lse, dout, B, H, causal=False, scale=None, workspace=None, gather_grads=False):
        """(dq, dk, dv) of this rank's shard; with `gather_grads` also the all-gathered
        (dq_full, dk_full, dv_full), complete after `wait()`."""
        import ctypes
        from .functional import _p, _stream_ptr
        d = self._desc(q, k, B, H, causal, scale)
        need = int(capi.lib.tt_mgpu_bwd_workspace_bytes(self._h, ctypes.byref(d)))
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fulls = (None, None, None)
        if gather_grads:
            fulls = tuple(torch.empty((self.world * t.shape[-3], *t.shape[-2:]), dtype=t.dtype, device=t.device) for t in (dq, dk, dv))
        capi.check(capi.lib.tt_mgpu_attn_bwd(self._h, ctypes.byref(d), _p(q), _p(k), _p(v), _p(out), _p(lse), _p(dout),
                                             _p(dq), _p(dk), _p(dv), _p(fulls[0]), _p(fulls[1]), _p(fulls[2]), _p(workspace),
                                             workspace.numel() * workspace.element_size(), _stream_ptr(q)))
        return (dq, dk, dv) + (fulls if gather_grads else ())

    def wait(self, device=None):
        import ctypes
        st = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        capi.check(capi.lib.tt_mgpu_wait(self._h, st))


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
