"""Multi-GPU partitioning of tree attention: by independent trees or by heads.

Every (tree, head, query block) is independent (the reference's programs never communicate,
fstattention.py:42-45), so the path shards without any exchange inside it: a batch of trees is
split over the ranks tree-wise, a single large tree head-wise.  The only collective is the
all-gather that reassembles the output, and callers that keep the output sharded for the next
layer skip even that (``gather=False``).  One process per GPU.  The gather comes in two forms:
``torch.distributed`` (NCCL) after the kernel, or - ``GatheredOutput`` - done by the attention
kernel itself, whose CTAs store each finished tile into every rank's copy of the output over
NVLink while the other CTAs still compute.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

AXES = {"tree": 0, "head": 1}


def shard_bounds(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split: the first ``n_units % world`` ranks hold one unit more."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def local_slice(t: torch.Tensor, axis: str, world: int, rank: int) -> torch.Tensor:
    """This rank's part of a full ``[Z, H, N, D]`` tensor (a view)."""
    dim = AXES[axis]
    lo, hi = shard_bounds(t.shape[dim], world, rank)
    return t.narrow(dim, lo, hi - lo)


class GatheredOutput:
    """The full output tensor ``[Z_total, H_total, N, D]`` of a sharded call, one copy per rank,
    every copy mapped into every rank's address space (torch symmetric memory: CUDA
    virtual-memory allocations exported between the processes of one node, at most 8 ranks).

    ``sharded_fst_attention(..., scatter_to=g)`` lets the attention kernel write this rank's
    rows into all copies; ``g.meet()`` is the cross-rank barrier (on the current stream) after
    which ``g.local`` is complete and before which nobody may reuse the buffer.  Collective:
    every rank of ``group`` constructs it, in the same order.
    """

    def __init__(self, full_shape, dtype, device, group=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm
        group = dist.group.WORLD if group is None else group
        self.group = group
        self.local = symm.empty(*full_shape, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, group)
        self.n_ranks = dist.get_world_size(group)
        if self.n_ranks > 8:
            raise ValueError("at most 8 ranks")
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank = dist.get_rank(group)
        if ptrs[self.rank] != self.local.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe the local buffer")
        self.pointer_array = (ctypes.c_void_p * self.n_ranks)(*ptrs)
        self.z0 = self.h0 = 0

    def target(self, axis: str, n_local: int):
        """Where this rank's shard lands: sets the (tree, head) origin for a shard of ``n_local``
        units along ``axis`` and returns ``self`` for ``fst_attention(..., scatter=...)``."""
        rank = dist.get_rank(self.group)
        lo, hi = shard_bounds(self.local.shape[AXES[axis]], self.n_ranks, rank)
        if hi - lo != n_local:
            raise ValueError("local shard does not match the partition")
        self.z0, self.h0 = (lo, 0) if axis == "tree" else (0, lo)
        return self

    def meet(self):
        """Barrier between the ranks on the current stream (device side: no host wait)."""
        self.handle.barrier()


def all_gather_outputs(o_local: torch.Tensor, axis: str, n_total: int, group=None, *,
                       out: Optional[torch.Tensor] = None, async_op: bool = False):
    """Reassemble the full output from every rank's shard along ``axis``.

    Equal shards that are contiguous in the full tensor (tree axis, or head axis with Z == 1)
    are gathered in place into one buffer (``out`` when given: nothing is allocated then);
    otherwise shards are padded to the largest one, gathered and trimmed.  With ``async_op``
    (in-place case only) the collective is enqueued behind the work already on the current
    stream and ``(full, work)`` is returned at once: the caller goes on launching the next
    layer's attention and calls ``work.wait()`` before it reads ``full``.
    """
    world = dist.get_world_size(group)
    dim = AXES[axis]
    sizes = [hi - lo for lo, hi in (shard_bounds(n_total, world, r) for r in range(world))]
    if o_local.shape[dim] != sizes[dist.get_rank(group)]:
        raise ValueError("local shard does not match the partition")
    full_shape = list(o_local.shape)
    full_shape[dim] = n_total
    in_place = len(set(sizes)) == 1 and (dim == 0 or o_local.shape[0] == 1)
    if out is not None and (list(out.shape) != full_shape or out.dtype != o_local.dtype or not out.is_contiguous()):
        raise ValueError("out must be a contiguous tensor of the full shape")
    if in_place:
        full = torch.empty(full_shape, dtype=o_local.dtype, device=o_local.device) if out is None else out
        work = dist.all_gather_into_tensor(full.view(-1), o_local.contiguous().view(-1), group=group,
                                           async_op=async_op)
        return (full, work) if async_op else full
    if async_op:
        raise ValueError("async_op needs equal shards that are contiguous in the full tensor")
    pad_shape = list(o_local.shape)
    pad_shape[dim] = max(sizes)
    padded = torch.zeros(pad_shape, dtype=o_local.dtype, device=o_local.device)
    padded.narrow(dim, 0, o_local.shape[dim]).copy_(o_local)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    full = torch.cat([p.narrow(dim, 0, s) for p, s in zip(parts, sizes)], dim=dim)
    if out is not None:
        out.copy_(full)
        return out
    return full


def sharded_fst_attention(q_local, k_local, v_local, meta_local, sm_scale: float, axis: str,
                          n_total: int, *, group=None, gather: bool = True,
                          gathered: Optional[torch.Tensor] = None, async_gather: bool = False,
                          scatter_to: Optional[GatheredOutput] = None,
                          attention: Optional[Callable] = None, **kwargs):
    """Tree attention on this rank's shard, then (optionally) the all-gather of outputs.

    ``axis="tree"``: the tensors hold this rank's trees (batch elements) and ``meta_local``
    their metadata.  ``axis="head"``: the tensors hold this rank's heads of every batch element
    and ``meta_local`` is the full tree metadata, identical on all ranks.  ``n_total`` is the
    global number of trees or heads.  ``gathered`` receives the full output (no allocation);
    ``async_gather`` returns ``(full, work)`` with the collective still under way, so that the
    next layer's attention overlaps it (``work.wait()`` before reading ``full``).
    ``scatter_to`` (a ``GatheredOutput``) replaces kernel + collective by one kernel that writes
    this rank's rows into every rank's copy, followed by the ranks' barrier on the stream; the
    full tensor (``scatter_to.local``) is returned.  Other keyword arguments (``out=``,
    ``kernel=`` ...) go to ``fst_attention``.
    """
    if axis not in AXES:
        raise ValueError("axis must be 'tree' or 'head'")
    if attention is None:
        from .fstattention import fst_attention as attention
    if scatter_to is not None:
        n_local = q_local.shape[AXES[axis]]
        full = attention(q_local, k_local, v_local, meta_local, sm_scale=sm_scale,
                         scatter=scatter_to.target(axis, n_local), **kwargs)
        scatter_to.meet()
        return full
    o_local = attention(q_local, k_local, v_local, meta_local, sm_scale=sm_scale, **kwargs)
    if not gather or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return o_local
    return all_gather_outputs(o_local, axis, n_total, group, out=gathered, async_op=async_gather)
