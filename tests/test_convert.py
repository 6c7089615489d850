"""Edge list / .npz -> CSR against scipy's coo_matrix(...).tocsr(), which is what the reference's
converters run (scripts/npz_to_csr.py:13-19)."""
import os
import subprocess

import numpy as np
import pytest
import scipy.sparse as sp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _scipy_csr(src, dst, n):
    m = sp.coo_matrix((np.ones(len(src)), (src, dst)), shape=(n, n)).tocsr()
    m.sort_indices()
    return m.indptr.astype(np.int32), m.indices.astype(np.int32)


@pytest.mark.parametrize("n,e,seed", [(300, 4000, 0), (5000, 200000, 1), (50, 0, 2), (1, 5, 3), (70000, 300000, 4)])
def test_coo_to_csr_equals_scipy(mps, n, e, seed):
    rng = np.random.default_rng(seed)
    src, dst = rng.integers(0, n, e), rng.integers(0, n, e)
    for threads in (1, 0):
        rp, col = mps.coo_to_csr(src, dst, n, threads)
        want_rp, want_col = _scipy_csr(src, dst, n)
        assert np.array_equal(rp, want_rp) and np.array_equal(col, want_col)


def test_size_is_inferred_and_bad_indices_are_errors(mps):
    rp, col = mps.coo_to_csr([0, 5, 5, 2], [1, 0, 0, 9])
    assert len(rp) - 1 == 10 and rp[-1] == 3  # the duplicate (5, 0) collapsed
    with pytest.raises(mps.MpsError):
        mps.coo_to_csr([0, -1], [1, 0])
    with pytest.raises(mps.MpsError):
        mps.coo_to_csr([0, 7], [1, 0], n_nodes=4)


@pytest.mark.parametrize("compressed,dtype", [(False, np.int64), (True, np.int64), (False, np.int32)])
def test_npz_reader_and_cli(tmp_path, mps, compressed, dtype):
    rng = np.random.default_rng(5)
    n, e = 2000, 60000
    src, dst = rng.integers(0, n, e).astype(dtype), rng.integers(0, n, e).astype(dtype)
    src[0], dst[0] = n - 1, n - 1  # make sure the inferred size is n
    p = str(tmp_path / "g.npz")
    (np.savez_compressed if compressed else np.savez)(p, src_li=src, dst_li=dst, num_nodes=np.int64(n))
    rp, col = mps.npz_to_csr(p)
    want_rp, want_col = _scipy_csr(src, dst, n)
    assert np.array_equal(rp, want_rp) and np.array_equal(col, want_col)
    from mergepath_spmm_b200 import build
    build.build_cli()
    out = str(tmp_path / "g.csr")
    r = subprocess.run([os.path.join(build.LIBDIR, "npz_to_csr"), "--graph", p, "--output", out], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    rp2, col2 = mps.load_csr(out)
    assert np.array_equal(rp2, want_rp) and np.array_equal(col2, want_col)


def test_npz_errors(tmp_path, mps):
    p = str(tmp_path / "bad.npz")
    np.savez(p, src_li=np.arange(5))
    with pytest.raises(mps.MpsError) as e:
        mps.npz_to_csr(p)
    assert "dst_li" in str(e.value)
    open(p, "wb").write(b"not a zip at all, just some bytes that are long enough........")
    with pytest.raises(mps.MpsError):
        mps.npz_to_csr(p)
    np.savez(p, src_li=np.zeros((3, 2), np.int64), dst_li=np.zeros((3, 2), np.int64))
    with pytest.raises(mps.MpsError) as e:
        mps.npz_to_csr(p)
    assert "one-dimensional" in str(e.value)


@pytest.mark.gpu
@pytest.mark.parametrize("n,e,seed", [(300, 4000, 0), (70000, 300000, 4), (1 << 20, 3_000_000, 5), (7, 0, 6)])
def test_device_conversion_equals_host(mps, cuda, n, e, seed):
    import torch
    rng = np.random.default_rng(seed)
    src, dst = rng.integers(0, n, e), rng.integers(0, n, e)
    rp, col = mps.coo_to_csr(src, dst, n)
    d_rp, d_col = mps.coo_to_csr_device(torch.from_numpy(src).to(cuda), torch.from_numpy(dst).to(cuda), n)
    assert np.array_equal(d_rp.cpu().numpy(), rp) and np.array_equal(d_col.cpu().numpy(), col)
    if e:
        bad = torch.from_numpy(src).to(cuda).clone()
        bad[0] = n
        with pytest.raises(mps.MpsError):
            mps.coo_to_csr_device(bad, torch.from_numpy(dst).to(cuda), n)


@pytest.mark.gpu
@pytest.mark.parametrize("n_rows,n_cols,e,seed,dtype", [(300, 200, 4000, 0, "f32"), (5000, 70000, 300000, 4, "f16"), (1 << 20, 1 << 19, 3_000_000, 5, "f32"),
                                                      (7, 9, 0, 6, None), (1, 1, 1, 7, "f32")])
def test_device_transpose_equals_scipy(mps, cuda, n_rows, n_cols, e, seed, dtype):
    """CSR of the transpose: same structure and value order as scipy's csr.T.tocsr() (columns ascending per row)."""
    import torch
    rng = np.random.default_rng(seed)
    keys = np.unique(rng.integers(0, n_rows * n_cols, e))
    r, c = keys // n_cols, keys % n_cols
    np_dtype = {"f32": np.float32, "f16": np.float16, None: np.float32}[dtype]
    v = rng.uniform(-1, 1, len(keys)).astype(np_dtype)
    A = sp.csr_matrix((v.astype(np.float64), (r, c)), shape=(n_rows, n_cols))
    A.sort_indices()
    want = A.T.tocsr()
    want.sort_indices()
    d_rp = torch.from_numpy(A.indptr.astype(np.int32)).to(cuda)
    d_col = torch.from_numpy(A.indices.astype(np.int32)).to(cuda)
    d_val = None if dtype is None else torch.from_numpy(A.data.astype(np_dtype)).to(cuda)
    rp_t, col_t, val_t = mps.csr_transpose_device(d_rp, d_col, d_val, n_cols)
    assert np.array_equal(rp_t.cpu().numpy(), want.indptr) and np.array_equal(col_t.cpu().numpy(), want.indices)
    if dtype is None:
        assert val_t is None
    else:
        assert np.array_equal(val_t.cpu().numpy(), want.data.astype(np_dtype))
    if len(keys):
        bad = d_col.clone()
        bad[0] = n_cols
        with pytest.raises(mps.MpsError):
            mps.csr_transpose_device(d_rp, bad, d_val, n_cols)


@pytest.mark.gpu
def test_backward_product_through_the_transpose(mps, orc, cuda):
    """dB = A^T dC with a rectangular, unsymmetric A: transpose once on the device, then the ordinary plan calls."""
    import torch
    rng = np.random.default_rng(3)
    n_rows, n_cols, dim = 20000, 12000, 32
    lengths = rng.zipf(1.6, n_rows).clip(0, 4000)
    lengths = np.minimum(lengths, n_cols)
    rp = np.zeros(n_rows + 1, np.int32)
    rp[1:] = np.cumsum(lengths)
    col = np.concatenate([np.sort(rng.choice(n_cols, int(m), replace=False)) for m in lengths]).astype(np.int32)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    dC = rng.uniform(-1, 1, (n_rows, dim)).astype(np.float32)
    d = [torch.from_numpy(a).to(cuda) for a in (rp, col, val, dC)]
    rp_t, col_t, val_t = mps.csr_transpose_device(d[0], d[1], d[2], n_cols)
    plan = mps.Plan(n_cols, len(col), dim, mps.F32, 8, device=cuda)
    plan.partition(rp_t)
    got = plan.spmm(rp_t, col_t, val_t, d[3]).cpu().numpy()
    plan.sync_check()
    info = plan.info()
    h_rp, h_col, h_val = (t.cpu().numpy() for t in (rp_t, col_t, val_t))
    model = orc.tile_model(h_rp, h_col, h_val, dC, 8, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], unit_items=info["unit_items"])
    assert np.array_equal(got.view(np.uint32), model.view(np.uint32))
    # against the definition, without using the transposed arrays: dB[j] = sum over (i, j) of a_ij * dC[i]
    want = np.zeros((n_cols, dim), np.float64)
    rows = np.repeat(np.arange(n_rows), np.diff(rp))
    np.add.at(want, col, val.astype(np.float64)[:, None] * dC.astype(np.float64)[rows])
    scale = np.zeros((n_cols, dim), np.float64)
    np.add.at(scale, col, np.abs(val.astype(np.float64))[:, None] * np.abs(dC.astype(np.float64))[rows])
    assert (np.abs(got - want) <= 1e-6 + 1e-5 * scale).all()
    plan.close()
