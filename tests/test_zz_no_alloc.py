"""mps_spmm_noalloc: the entry point for callers that may not allocate device memory (its scratch is
a fixed array inside the library).  Collected last on purpose: a run that stops at the first failure
has then already run every other test.

Checked here, through the C ABI, on two different problems back to back and then the first again
(the shared scratch keeps the previous call's contents, so stale data would show):
  - the output equals the plan-based entry points' output bit for bit (same kernels, same layout);
  - free device memory does not move across the calls;
  - a problem whose scratch exceeds the built-in array is refused with a message, not attempted."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _problem(graphs, cuda, which):
    if which == "rmat_f32":
        rp, col = cases.c1_rmat()
        val = graphs.gcn_values(rp, col)
        B = graphs.dense_uniform(len(rp) - 1, 64, seed=1)
    else:
        rp, col = cases.c2_batched(300)
        val = graphs.gcn_values(rp, col, "f16")
        B = graphs.dense_normal_f16(len(rp) - 1, 16, seed=2)
    dev = [torch.from_numpy(np.ascontiguousarray(a)).to(cuda) for a in (rp, col, val, B)]
    return dev


def _with_plan(mps, cuda, rp, col, val, B, cost):
    plan = mps.Plan(rp.numel() - 1, col.numel(), B.shape[1], mps.F16 if B.dtype == torch.float16 else mps.F32, cost, device=cuda)
    plan.partition(rp)
    out = plan.spmm(rp, col, val, B)
    plan.sync_check()
    plan.close()
    return out


def test_noalloc_matches_plan_path_on_consecutive_calls(mps, graphs, cuda):
    first = _problem(graphs, cuda, "rmat_f32")
    second = _problem(graphs, cuda, "batched_f16")
    want_first = _with_plan(mps, cuda, *first, cost=8)
    want_second = _with_plan(mps, cuda, *second, cost=8)
    out_first = torch.full_like(want_first, float("nan"))
    out_second = torch.full_like(want_second, float("nan"))
    out_again = torch.full_like(want_first, float("nan"))

    mps.spmm_noalloc(*first, out=out_first, cost=8)           # also the per-device set-up call
    assert torch.equal(out_first, want_first)

    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(cuda)[0]
    mps.spmm_noalloc(*second, out=out_second, cost=8)         # a different shape and dtype right after
    mps.spmm_noalloc(*first, out=out_again, cost=8)           # and the first one again
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info(cuda)[0]

    assert torch.equal(out_second, want_second)
    assert torch.equal(out_again, want_first)
    assert free_after == free_before, "the no-allocation entry point changed the amount of free device memory"


def test_noalloc_unit_values_and_other_cost(mps, graphs, cuda):
    rp, col, _val, B = _problem(graphs, cuda, "rmat_f32")
    want = _with_plan(mps, cuda, rp, col, None, B, cost=32)
    out = torch.empty_like(want)
    for _ in range(2):
        out.fill_(float("nan"))
        mps.spmm_noalloc(rp, col, None, B, out=out, cost=32)
        assert torch.equal(out, want)


def test_noalloc_mid_size_runs_the_separate_fixup_on_the_static_array(mps, graphs, cuda):
    """Between 2,049 and 32,768 tiles the cross-tile fix-up is a kernel of its own that reads the tile carries, the
    per-tile counts and the long-row list out of the static array; twice in a row, with a small problem in between
    that overwrites the front of the array."""
    rp, col = graphs.rmat_csr(17, 32, seed=9)
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 32, seed=6)
    big = [torch.from_numpy(np.ascontiguousarray(a)).to(cuda) for a in (rp, col, val, B)]
    lay = mps.layout_query(len(rp) - 1, len(col), 32, mps.F32, 16)
    assert 2048 < lay["n_tiles"] <= 32768 and lay["fused_fixup"] == 0
    want = _with_plan(mps, cuda, *big, cost=16)
    small = _problem(graphs, cuda, "rmat_f32")
    want_small = _with_plan(mps, cuda, *small, cost=8)
    out = torch.empty_like(want)
    out_small = torch.empty_like(want_small)
    for _ in range(2):
        out.fill_(float("nan"))
        mps.spmm_noalloc(*big, out=out, cost=16)
        assert torch.equal(out, want)
        mps.spmm_noalloc(*small, out=out_small, cost=8)
        assert torch.equal(out_small, want_small)


def test_noalloc_refuses_what_does_not_fit(mps, cuda):
    """The shape is refused before any pointer is used.  It is chosen so that it cannot fit under any
    tile layout: 2*10^9 merge items need more than 32,768 tiles even if a tile filled all of an SM's
    shared memory (~17k items), so the small buffers passed here are never read."""
    z = torch.zeros(64, dtype=torch.int32, device=cuda)
    f = torch.zeros(64, dtype=torch.float32, device=cuda)
    rc = mps.capi.lib().mps_spmm_noalloc(1 << 24, 2_000_000_000, 128, mps.F32, 8, 1, C.c_void_p(z.data_ptr()), C.c_void_p(z.data_ptr()),
                                         None, C.c_void_p(f.data_ptr()), C.c_void_p(f.data_ptr()), None)
    assert rc == mps.capi.ERR_UNSUPPORTED
    msg = mps.capi.lib().mps_last_error().decode()
    assert "tiles" in msg and "mps_plan_create" in msg
