"""Numeric legs of the oracle against each other and against scipy (all on the CPU)."""
import numpy as np
import pytest
import scipy.sparse as sp

import cases


def _rand_b(n, dim, seed=1, half=False):
    from mergepath_spmm_b200 import graphs
    b = graphs.dense_uniform(n, dim, seed)
    return b.astype(np.float16) if half else b


def _csr(rp, col, val, n_cols):
    v = np.ones(len(col), np.float64) if val is None else val.astype(np.float64)
    return sp.csr_matrix((v, col, rp), shape=(len(rp) - 1, n_cols))


def test_fp64_loop_matches_scipy(orc, graphs):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = _rand_b(len(rp) - 1, 16)
    got = orc.spmm_f64(rp, col, val, B)
    want = _csr(rp, col, val, len(rp) - 1) @ B.astype(np.float64)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_c1_shape_is_the_configured_one():
    rp, col = cases.c1_rmat()
    assert len(rp) - 1 == 4096
    assert 90_000 < len(col) < 135_168  # 2*65536 + 4096 minus duplicates
    # symmetric, self-loops present, columns sorted and unique per row
    A = _csr(rp, col, None, 4096)
    assert (A != A.T).nnz == 0 and (A.diagonal() == 1).all()
    for i in (0, 1, 17, 4095):
        r = col[rp[i]:rp[i + 1]]
        assert (np.diff(r) > 0).all()


def test_c2_shape_is_the_configured_one(graphs):
    rp, col = cases.c2_batched()
    n = len(rp) - 1
    assert 40_000 < n < 48_000 and 180_000 < len(col) < 280_000
    val = graphs.gcn_values(rp, col)
    assert val.dtype == np.float32 and (val > 0).all() and (val <= 1).all()


@pytest.mark.parametrize("dim,cost,nch,cpu", [(16, 8, 256, 4), (64, 8, 64, 4), (64, 4, 16, 1), (128, 32, 32, 4), (20, 8, 32, 32), (5, 3, 7, 1)])
def test_tile_model_close_to_fp64(orc, graphs, dim, cost, nch, cpu):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = _rand_b(len(rp) - 1, dim)
    got = orc.tile_model(rp, col, val, B, cost, nch, cpu, 32)
    ref = orc.spmm_f64(rp, col, val, B)
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(got - ref) <= 1e-6 + 1e-5 * scale).all()


@pytest.mark.parametrize("name", sorted(cases.edge_cases().keys()))
def test_tile_model_edge_cases(orc, name):
    rp, col = cases.edge_cases()[name]
    n = len(rp) - 1
    n_cols = max(int(col.max()) + 1 if len(col) else 1, n)
    rng = np.random.default_rng(3)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    B = rng.uniform(-1, 1, (n_cols, 12)).astype(np.float32)
    for cost, nch, cpu, long_chain in ((1, 4, 1, 2), (3, 8, 2, 32), (8, 64, 4, 32), (8, 1, 1, 1), (2, 12, 12, 3)):
        got = orc.tile_model(rp, col, val, B, cost, nch, cpu, long_chain)
        ref = orc.spmm_f64(rp, col, val, B)
        scale = orc.spmm_abs_f64(rp, col, val, B)
        assert (np.abs(got - ref) <= 1e-6 + 1e-5 * scale).all(), (name, cost, nch)


def test_tile_model_long_chain_path_is_exercised(orc):
    """A 5000-nnz row cut into tiles of 2 chunks x 2 items spans >32 tiles: the strand order runs."""
    rp, col = cases.edge_cases()["one_giant_row"]
    rng = np.random.default_rng(5)
    B = rng.uniform(-1, 1, (6000, 8)).astype(np.float32)
    a = orc.tile_model(rp, col, None, B, 1, 2, 1, 32)
    b = orc.tile_model(rp, col, None, B, 1, 2, 1, 10**9)  # same chunks, plain order
    ref = orc.spmm_f64(rp, col, None, B)
    assert np.allclose(a, ref, rtol=1e-5, atol=1e-4) and np.allclose(b, ref, rtol=1e-5, atol=1e-4)
    assert not np.array_equal(a, b)  # different summation order => some bit differs


def test_tile_model_fp16(orc, graphs):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col, "f16")
    B = graphs.dense_normal_f16(len(rp) - 1, 32, seed=1)
    got = orc.tile_model(rp, col, val, B, 8, 64, 4, 32, is_half=True).astype(np.float64)
    ref = orc.spmm_f64(rp, col, val, B, is_half=True)
    scale = orc.spmm_abs_f64(rp, col, val, B, is_half=True)
    assert (np.abs(got - ref) <= 1e-6 + 1e-2 * np.maximum(scale, np.abs(ref))).all()


def test_reference_kernel_emulation_unit_degrees(orc):
    """With degrees == 1 the reference kernel is a unit-valued SpMM, except that the zero sentinel
    (src/MergePathSpMM.cu:365-369,467) drops chunk 0's tail share of row 0."""
    rp, col = cases.c1_rmat()
    n = len(rp) - 1
    B = _rand_b(n, 16)
    p = orc.chunk_count(n, len(col), 8)
    ipt = orc.items_per_chunk(n, len(col), p)
    got = orc.ref_kernel_emulate_f32(rp, col, np.ones(n + 1, np.int32), B, p)
    ref = orc.spmm_f64(rp, col, None, B)
    scale = orc.spmm_abs_f64(rp, col, None, B)
    ok = np.abs(got - ref) <= 1e-6 + 1e-5 * scale
    assert ok[1:].all()
    assert rp[1] > ipt - 1, "row 0 must be longer than chunk 0 for the quirk to show"
    lost = B[col[: ipt - 1]].astype(np.float64).sum(axis=0)
    assert np.allclose(ref[0] - got[0], lost, rtol=1e-5, atol=1e-4)


def test_omp_baseline_matches_fp64(orc, graphs):
    rp, col = cases.c2_batched(200)
    val = graphs.gcn_values(rp, col)
    B = _rand_b(len(rp) - 1, 16)
    got, used = orc.spmm_f32_omp(rp, col, val, B)
    assert used >= 1
    assert np.allclose(got, orc.spmm_f64(rp, col, val, B), rtol=1e-5, atol=1e-6)


def test_generators_host_equals_torch_cpu(graphs):
    """The same hash drives numpy and torch generation; torch on CPU stands in for the GPU here."""
    import torch
    u, v = graphs.rmat_edges(10, 5000, seed=3)
    ut, vt = graphs.rmat_edges(10, 5000, seed=3, device=torch.device("cpu"))
    assert np.array_equal(u, ut.numpy()) and np.array_equal(v, vt.numpy())
    rp, col = graphs.csr_from_edges(u, v, 1024)
    rpt, colt = graphs.csr_from_edges(ut, vt, 1024)
    assert np.array_equal(rp, rpt.numpy()) and np.array_equal(col, colt.numpy())
    assert np.array_equal(graphs.gcn_values(rp, col), graphs.gcn_values(rpt, colt).numpy())
    assert np.array_equal(graphs.dense_uniform(100, 7, 5), graphs.dense_uniform(100, 7, 5, device=torch.device("cpu")).numpy())


def test_scaled_model_close_to_fp64(orc, graphs):
    """value(i, j) = row_scale[i] * col_scale[j] with the row factor applied to the finished row."""
    rp, col = cases.c1_rmat()
    n = len(rp) - 1
    dinv = (1.0 / np.sqrt(np.diff(rp).astype(np.float64))).astype(np.float32)
    B = _rand_b(n, 24)
    got = orc.tile_model_scaled(rp, col, dinv, dinv, B, 8, 64, 4, 32)
    rows = np.repeat(np.arange(n), np.diff(rp))
    val64 = dinv.astype(np.float64)[rows] * dinv.astype(np.float64)[col]
    A = sp.csr_matrix((val64, col, rp), shape=(n, n))
    ref = A @ B.astype(np.float64)
    scale = abs(A) @ np.abs(B.astype(np.float64))
    assert (np.abs(got - ref) <= 1e-6 + 1e-5 * scale).all()
    # and close to the explicit GCN values (which round the product of the two factors once more)
    explicit = orc.tile_model(rp, col, graphs.gcn_values(rp, col), B, 8, 64, 4, 32)
    assert (np.abs(got - explicit) <= 1e-6 + 1e-5 * scale).all()
