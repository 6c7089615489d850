"""Two ranks on two GPUs (NCCL): each rank holds a row slab of A and a block of B's rows on the host, completes B with
multi.replicate_b (all-gather over NVLink), multiplies through mps_spmm_host_resident_b, and the slabs of C are
replicated with multi.gather_c (one broadcast per slab, no padding).  Every rank must end with the C that one GPU
computes slab by slab.  Skipped on a box with fewer than two devices."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    mps = entry.load_package()
    from mergepath_spmm_b200 import graphs, multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    rp, col = graphs.rmat_csr(17, 16, seed=7)
    val = graphs.gcn_values(rp, col)
    n, dim = len(rp) - 1, 32
    B = graphs.dense_uniform(n, dim, seed=8)
    bounds = mps.slab_bounds(rp, world, "items", 4)
    r0, r1, srp, scol, sval = multi.slab_of(rp, col, val, rank, world, bounds)
    b0, b1, _ = multi.b_block(n, rank, world)
    ok = True
    for _ in range(2):
        d_B = multi.replicate_b(torch.from_numpy(B[b0:b1].copy()).pin_memory(), n, device=dev)
        out = torch.full((r1 - r0, dim), float("nan"), dtype=torch.float32).pin_memory()
        mps.spmm_host_resident_b(srp, scol, sval, d_B, out, cost=16)
        ok = ok and bool(torch.equal(d_B.cpu(), torch.from_numpy(B)))
        # the same slab through the plan path on this GPU, B uploaded whole
        want = mps.spmm(torch.from_numpy(srp).to(dev), torch.from_numpy(scol).to(dev), torch.from_numpy(sval).to(dev), torch.from_numpy(B).to(dev), cost=16)
        ok = ok and bool(torch.equal(out.to(dev), want))
        full = multi.gather_c(want, bounds)
        pieces = [torch.zeros_like(full) for _ in range(world)]
        dist.all_gather(pieces, full)
        ok = ok and all(bool(torch.equal(p, full)) for p in pieces) and bool(torch.equal(full[r0:r1], want))
    mps.capi.lib().mps_host_workspace_release()
    with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
        f.write("1" if ok else "0")
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_ranks_complete_b_over_nccl_and_replicate_c(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two devices")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.ok").read() == "1"
