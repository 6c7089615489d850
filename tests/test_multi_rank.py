"""The N > 1 host logic on CPU ranks (gloo, world sizes 2 and 3): slab bounds, rebasing, B completed from
per-rank blocks, the unpadded gather of C.  The multiply itself is the GPU's job; here each rank fills its slab with the
oracle's fp64 loop (as the checker's stand-in) so that the plumbing can be verified without a GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as entry
    mps = entry.load_package()
    orc = entry.load_oracle()
    from mergepath_spmm_b200 import graphs, multi
    import cases
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 8, seed=1)
    bounds = mps.slab_bounds(rp, world)
    r0, r1, srp, scol, sval = multi.slab_of(rp, col, val, rank, world, bounds)
    assert srp[0] == 0 and srp[-1] == len(scol) == rp[r1] - rp[r0]
    c_slab = torch.from_numpy(orc.spmm_f64(srp, scol, sval, B).astype(np.float32))
    full = multi.gather_c(c_slab, bounds)
    want = orc.spmm_f64(rp, col, val, B).astype(np.float32)
    ok = bool(np.array_equal(full.numpy(), want))
    # B from per-rank blocks: every rank contributes rows [b0, b1) only and ends with all of B
    b0, b1, blk = multi.b_block(n, rank, world)
    assert blk * world >= n and (rank < world - 1 or b1 == n)
    whole = multi.replicate_b(torch.from_numpy(B[b0:b1].copy()), n)
    ok = ok and whole.shape == (n, 8) and bool(np.array_equal(whole.numpy(), B))
    # torch tensors take the same path as numpy arrays
    r0t, r1t, srp_t, scol_t, sval_t = multi.slab_of(torch.from_numpy(rp), torch.from_numpy(col), torch.from_numpy(val), rank, world)
    ok = ok and (r0t, r1t) == (r0, r1) and np.array_equal(srp_t.numpy(), srp) and np.array_equal(scol_t.numpy(), scol)
    # nnz balance: no rank holds more than its share plus one row
    share = torch.tensor([len(scol)], dtype=torch.int64)
    shares = [torch.zeros_like(share) for _ in range(world)]
    dist.all_gather(shares, share)
    biggest_row = int(np.diff(rp).max())
    ok = ok and max(int(s) for s in shares) <= len(col) / world + biggest_row
    with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_cpu_ranks_slab_and_gather(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.ok").read() == "1"
