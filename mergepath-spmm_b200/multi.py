"""Row-slab sharding for one process per GPU (no reference counterpart: the reference is single-GPU).

Rows of C are independent given all of B, so the path shards without a data-path collective:
rank g owns rows [bounds[g], bounds[g+1]) with bounds chosen for equal non-zero counts
(mps_slab_bounds), keeps a full copy of B, and writes its own slab of C.  A replicated C, when asked
for, is one all-gather of the slabs padded to the tallest (torch.distributed: NCCL on GPUs, gloo in
the CPU tests of this logic)."""
from __future__ import annotations

import numpy as np

try:
    import torch
    import torch.distributed as dist
except Exception:  # pragma: no cover
    torch = None
    dist = None


def slab_of(row_ptr, col_idx, val, rank: int, world: int, bounds=None):
    """This rank's slab of a CSR held as numpy arrays or torch tensors (any device):
    (row0, row1, row_ptr rebased to 0, col_idx slice, val slice)."""
    from . import slab_bounds
    if bounds is None:
        host_rp = row_ptr.cpu().numpy() if torch is not None and isinstance(row_ptr, torch.Tensor) else row_ptr
        bounds = slab_bounds(host_rp, world)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    k0, k1 = int(row_ptr[r0]), int(row_ptr[r1])
    rp = row_ptr[r0:r1 + 1] - k0
    if torch is not None and isinstance(rp, torch.Tensor):
        rp = rp.contiguous()
        cols = col_idx[k0:k1].clone()
        vals = None if val is None else val[k0:k1].clone()
    else:
        rp = np.ascontiguousarray(rp, np.int32)
        cols = np.ascontiguousarray(col_idx[k0:k1])
        vals = None if val is None else np.ascontiguousarray(val[k0:k1])
    return r0, r1, rp, cols, vals


def gather_c(c_slab, bounds, group=None):
    """All-gather of unequal C slabs: every rank gets the full (N, dim) C.  Slabs are padded to the
    tallest so a single all_gather_into_tensor moves them."""
    world = dist.get_world_size(group)
    heights = [int(bounds[g + 1]) - int(bounds[g]) for g in range(world)]
    tall, dim = max(heights), c_slab.shape[1]
    mine = torch.zeros((tall, dim), dtype=c_slab.dtype, device=c_slab.device)
    mine[: c_slab.shape[0]] = c_slab
    full = torch.empty((world * tall, dim), dtype=c_slab.dtype, device=c_slab.device)
    dist.all_gather_into_tensor(full, mine, group=group)
    return torch.cat([full[g * tall: g * tall + heights[g]] for g in range(world)])
