"""The single-process multi-GPU driver (mps_multi_*).  On a one-GPU box the slab logic is still
exercised by placing several slabs on the same device; the NCCL gather needs two or more devices."""
import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


def _single(mps, cuda, rp, col, val, B, cost):
    d = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    return mps.spmm(d(rp), d(col), d(val), d(B), cost=cost).cpu().numpy()


@pytest.mark.parametrize("n_slabs", [1, 2, 5])
def test_slabs_on_one_device_equal_their_own_single_runs(mps, orc, graphs, cuda, n_slabs):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 64, seed=1)
    m = mps.MultiGpu(rp, col, val, n, 64, mps.F32, cost=16, n_gpus=n_slabs, devices=[0] * n_slabs)
    m.set_b(B)
    ms, _ = m.spmm(repeat=2)
    assert ms > 0
    got = m.get_c()
    bounds = mps.slab_bounds(rp, n_slabs, "items", 4)
    for g in range(n_slabs):
        s = m.slab(g)
        assert (s["row0"], s["row1"]) == (int(bounds[g]), int(bounds[g + 1]))
        r0, r1 = s["row0"], s["row1"]
        want = _single(mps, cuda, mps.slab_rebase(rp, r0, r1), col[rp[r0]:rp[r1]], val[rp[r0]:rp[r1]], B, 16)
        assert np.array_equal(_bits(got[r0:r1]), _bits(want)), g
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(got.astype(np.float64) - orc.spmm_f64(rp, col, val, B)) <= 1e-6 + 1e-5 * scale).all()
    m.close()


def test_fp16_and_unit_values(mps, orc, graphs, cuda):
    rp, col = cases.c2_batched(200)
    n = len(rp) - 1
    B = graphs.dense_normal_f16(n, 16, seed=2)
    m = mps.MultiGpu(rp, col, None, n, 16, mps.F16, cost=8, n_gpus=3, devices=[0, 0, 0])
    m.set_b(B)
    m.spmm()
    got = m.get_c().astype(np.float64)
    ref = orc.spmm_f64(rp, col, None, B, is_half=True)
    assert (np.abs(got - ref) <= 1e-6 + 1e-2 * np.maximum(orc.spmm_abs_f64(rp, col, None, B, is_half=True), np.abs(ref))).all()
    m.close()


def test_errors_are_codes(mps, cuda):
    rp, col = cases.c2_batched(20)
    n = len(rp) - 1
    with pytest.raises(mps.MpsError) as e:
        mps.MultiGpu(rp, col, None, n, 16, n_gpus=2, devices=[0, 99])
    assert e.value.code == mps.capi.ERR_ARG
    m = mps.MultiGpu(rp, col, None, n, 16, n_gpus=1)
    with pytest.raises(mps.MpsError) as e:
        m.spmm()
    assert e.value.code == mps.capi.ERR_STATE  # B not set
    m.close()


def test_gather_over_nccl_makes_every_copy_complete(mps, graphs, cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("the NCCL gather needs at least two devices")
    g = min(torch.cuda.device_count(), 4)
    rp, col = graphs.rmat_csr(16, 16, seed=7)
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 32, seed=8)
    m = mps.MultiGpu(rp, col, val, n, 32, mps.F32, cost=16, n_gpus=g)
    m.set_b(B)
    ms, ms_gather = m.spmm(repeat=3, gather_c=True)
    assert ms > 0 and ms_gather > 0
    slabs = m.get_c(-1)
    for d in range(g):
        assert np.array_equal(_bits(m.get_c(d)), _bits(slabs)), d
    m.close()
