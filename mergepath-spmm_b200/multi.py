"""Row-slab sharding for one process per GPU (no reference counterpart: the reference is single-GPU).

Rows of C are independent given all of B, so the path shards without a data-path collective:
rank g owns rows [bounds[g], bounds[g+1]) with bounds chosen for equal non-zero counts
(mps_slab_bounds), keeps a full copy of B, and writes its own slab of C.  B reaches the ranks once over
PCIe in total: every rank uploads an equal block of its rows and one all-gather completes each copy
(replicate_b).  A replicated C, when asked for, is one broadcast per slab into place - slab heights
differ widely, so nothing is padded (gather_c).  torch.distributed: NCCL on GPUs, gloo in the CPU tests
of this logic."""
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


def b_block(n_cols: int, rank: int, world: int):
    """Rows [r0, r1) of B that rank `rank` uploads: equal blocks of ceil(n_cols / world) rows (the last may be short)."""
    blk = (n_cols + world - 1) // world
    r0 = min(rank * blk, n_cols)
    return r0, min(r0 + blk, n_cols), blk


def replicate_b(b_rows_host, n_cols: int, device=None, group=None, out=None):
    """Every rank passes only ITS block of B's rows (b_block; a host tensor, pinned for an asynchronous copy) and gets
    the whole B (n_cols x dim) on its device: one H2D copy of the block into its place, then one all-gather of equal
    blocks in place - over NVLink with NCCL - so that B crosses PCIe once in total instead of once per rank.  The
    returned tensor is complete once the work queued on the current stream has run (the collective is stream-ordered);
    its storage holds world * ceil(n_cols / world) rows, of which the first n_cols are B."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    r0, r1, blk = b_block(n_cols, rank, world)
    dim = b_rows_host.shape[1]
    assert b_rows_host.shape[0] == r1 - r0, "this rank's block of B has the wrong number of rows"
    if out is None:
        out = torch.empty((world * blk, dim), dtype=b_rows_host.dtype, device=device)
    if r1 > r0:
        out[r0:r1].copy_(b_rows_host, non_blocking=True)
    mine = out[rank * blk:(rank + 1) * blk]
    if dist.get_backend(group) != "nccl":
        mine = mine.clone()  # only NCCL defines the in-place form (input = this rank's block of the output)
    dist.all_gather_into_tensor(out, mine, group=group)
    return out[:n_cols]


def gather_c(c_slab, bounds, group=None, out=None):
    """Replicated C from unequal slabs: every rank ends with the full (N, dim) C.  One broadcast per slab straight
    into its rows of the result (started together, so NCCL runs them back to back); no padding, the bytes moved are
    the bytes of C."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n, dim = int(bounds[world]), c_slab.shape[1]
    if out is None:
        out = torch.empty((n, dim), dtype=c_slab.dtype, device=c_slab.device)
    out[int(bounds[rank]):int(bounds[rank + 1])].copy_(c_slab)
    works = []
    for g in range(world):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        if r1 > r0:
            works.append(dist.broadcast(out[r0:r1], src=dist.get_global_rank(group, g) if group is not None else g, group=group, async_op=True))
    for w in works:
        w.wait()
    return out
