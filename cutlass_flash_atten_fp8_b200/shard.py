"""(batch x head) sharding across the GPUs of one box.

Every (batch, head) slice of the attention is independent - the reference maps
the flattened index to grid.y (csrc/flash_attention.cu:339,364,594-597) - so rank
r of N takes a contiguous range of the flattened batch*heads axis, which is a
contiguous byte range of each [batch, heads, seqlen, head_dim] tensor.  The hot
path has no collective; gathering O on one rank is optional and timed apart.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_slices: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) of `n_slices` owned by `rank`; sizes differ by at most one,
    the first (n_slices % world_size) ranks hold the longer ranges."""
    if world_size <= 0 or not (0 <= rank < world_size) or n_slices < 0:
        raise ValueError("need 0 <= rank < world_size and n_slices >= 0")
    base, rem = divmod(n_slices, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def all_ranges(n_slices: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_range(n_slices, world_size, r) for r in range(world_size)]


def global_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """Element-wise MAX over ranks of a small tensor of |x| maxima, so that per-tensor
    quantisation scales do not depend on how the slices are sharded.  Set-up only."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        local_amax = local_amax.clone()
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


def gather_output(o_local: torch.Tensor, n_slices: int, dst: int = 0, group=None) -> Optional[torch.Tensor]:
    """Optional gather of the per-rank O slices ([n_local, seqlen, head_dim]) on rank
    `dst` in flattened (batch*heads) order.  Returns the full tensor on dst, else None.
    `dst` and the shard order are ranks WITHIN `group` (the default group: global ranks)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return o_local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ranges = all_ranges(n_slices, world)
    # torch's point-to-point and gather calls name peers by GLOBAL rank, whatever the group

    def glob(r: int) -> int:
        return r if group is None else dist.get_global_rank(group, r)

    if rank == dst:
        full = torch.empty((n_slices,) + tuple(o_local.shape[1:]), dtype=o_local.dtype, device=o_local.device)
        parts = [full[lo:hi] for lo, hi in ranges]
        if len({hi - lo for lo, hi in ranges}) == 1:
            dist.gather(o_local, gather_list=parts, dst=glob(dst), group=group)
        else:
            reqs = []
            for r, (lo, hi) in enumerate(ranges):
                if r == dst:
                    parts[r].copy_(o_local)
                elif hi > lo:
                    reqs.append(dist.irecv(parts[r], src=glob(r), group=group))
            for q in reqs:
                q.wait()
        return full
    if len({hi - lo for lo, hi in ranges}) == 1:
        dist.gather(o_local, gather_list=None, dst=glob(dst), group=group)
    elif o_local.shape[0] > 0:
        dist.send(o_local, dst=glob(dst), group=group)
    return None
