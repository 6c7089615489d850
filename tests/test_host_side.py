"""Host-side pieces of the C ABI that need no GPU: the host partition / schedule entry points against the
reference's golden vectors, validation of a caller's CSR in the host-buffer calls, and the automatic tile
layout for every `cost` the reference's command line accepts (src/MergePathSpMM.cu:113-124 takes any)."""
import ctypes as C
import os

import numpy as np
import pytest

import cases

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_partition.npz")


def test_host_partition_and_schedule_bit_exact_with_reference_vectors(mps):
    g = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in g.files})
    checked = 0
    for name in names:
        rp = g[f"{name}/row_ptr"]
        for key in [k for k in g.files if k.startswith(name + "/cost") and k.endswith("/xy")]:
            cost = int(key.split("/")[1][4:])
            p = int(g[f"{name}/cost{cost}/n_chunks"])
            for threads in (1, 0):
                assert np.array_equal(mps.partition_host(rp, p, threads), g[key]), (name, cost)
                assert np.array_equal(mps.schedule_host(rp, p, threads), g[f"{name}/cost{cost}/six"]), (name, cost)
            checked += 1
    assert checked >= 30


def test_host_partition_on_a_mid_size_graph_equals_the_oracle(mps, orc, graphs):
    rp, _ = graphs.rmat_csr(15, 16, seed=2)
    for cost in (4, 32, 1000):
        p, _ = mps.chunk_count(len(rp) - 1, int(rp[-1]), cost)
        assert np.array_equal(mps.partition_host(rp, p), orc.partition(rp, p))
        assert np.array_equal(mps.schedule_host(rp, p), orc.schedule(rp, p))
    with pytest.raises(mps.MpsError) as e:
        mps.partition_host(rp, 0)
    assert e.value.code == mps.capi.ERR_ARG


def test_host_partition_and_schedule_equal_the_oracle_on_random_row_lengths(mps, orc):
    """Property test: any row-length sequence (empty rows, one huge row, runs of equal lengths) and any chunk count
    give the coordinates and the six schedule arrays of the oracle, which is pinned to the reference's vectors."""
    from hypothesis import given, settings, strategies as st, HealthCheck
    lengths = st.lists(st.one_of(st.just(0), st.integers(0, 5), st.integers(0, 300)), min_size=1, max_size=200)

    @settings(max_examples=120, deadline=None, suppress_health_check=list(HealthCheck))
    @given(lengths, st.integers(1, 64), st.integers(0, 2))
    def run(lens, cost, threads):
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        p, _ = mps.chunk_count(len(rp) - 1, int(rp[-1]), cost)
        assert np.array_equal(mps.partition_host(rp, p, threads), orc.partition(rp, p))
        assert np.array_equal(mps.schedule_host(rp, p, threads), orc.schedule(rp, p))

    run()


def _host_call(mps, rp, col, n_cols, dim=8):
    n = len(rp) - 1
    B = np.zeros((n_cols, dim), np.float32)
    out = np.zeros((n, dim), np.float32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    return mps.capi.lib().mps_spmm_host(n, n_cols, len(col), dim, mps.F32, 8, 1, p(rp), p(col), None, p(B), p(out))


def test_host_buffer_call_rejects_a_bad_csr_before_anything_runs(mps):
    """A caller's bad index must come back as MPS_ERR_ARG, not become a gather outside B on the device; the
    check is host code, so it also answers on a machine without a GPU (where a valid call gets MPS_ERR_CUDA)."""
    rp, col = cases.c2_batched(40)
    n = len(rp) - 1
    lib = mps.capi.lib()
    bad = col.copy(); bad[len(bad) // 2] = n                      # one past the last row of B
    assert _host_call(mps, rp, bad, n) == mps.capi.ERR_ARG
    assert f"col_idx[{len(bad) // 2}] = {n}" in lib.mps_last_error().decode()
    bad = col.copy(); bad[3] = -1
    assert _host_call(mps, rp, bad, n) == mps.capi.ERR_ARG
    dec = rp.copy(); dec[7] = dec[8] + 1                         # row 7 ends before it starts
    assert _host_call(mps, dec, col, n) == mps.capi.ERR_ARG
    assert "row_ptr decreases at row 7" in lib.mps_last_error().decode()
    first = rp.copy(); first[0] = 1
    assert _host_call(mps, first, col, n) == mps.capi.ERR_ARG
    # a large col_idx takes the background-thread path of the scan
    big_rp = np.arange(0, 300001, 3, dtype=np.int32)
    big_col = np.zeros(300000, np.int32); big_col[-1] = 100000
    assert _host_call(mps, big_rp, big_col, 100000) == mps.capi.ERR_ARG
    import torch
    if not torch.cuda.is_available():
        assert _host_call(mps, rp, col, n) == mps.capi.ERR_CUDA  # valid arrays: only the device is missing


def test_scaled_host_call_checks_its_arguments(mps):
    """mps_spmm_host_scaled: both factors NULL is an argument error; a bad CSR is reported as for mps_spmm_host."""
    rp, col = cases.c2_batched(40)
    n = len(rp) - 1
    B = np.zeros((n, 8), np.float32)
    ones = np.ones(n, np.float32)
    with pytest.raises(mps.MpsError) as e:
        mps.spmm_host_scaled(rp, col, None, None, B)
    assert e.value.code == mps.capi.ERR_ARG
    bad = col.copy(); bad[5] = n
    with pytest.raises(mps.MpsError) as e:
        mps.spmm_host_scaled(rp, bad, ones, ones, B)
    assert e.value.code == mps.capi.ERR_ARG and f"col_idx[5] = {n}" in str(e.value)
    dec = rp.copy(); dec[7] = dec[8] + 1
    with pytest.raises(mps.MpsError) as e:
        mps.spmm_host_scaled(dec, col, ones, None, B)
    assert e.value.code == mps.capi.ERR_ARG
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(mps.MpsError) as e:
            mps.spmm_host_scaled(rp, col, ones, ones, B)
        assert e.value.code == mps.capi.ERR_CUDA


def test_multi_gpu_driver_rejects_a_bad_csr_before_touching_a_device(mps):
    rp, col = cases.c2_batched(40)
    n = len(rp) - 1
    bad = col.copy(); bad[10] = n + 5
    with pytest.raises(mps.MpsError) as e:
        mps.MultiGpu(rp, bad, None, n, 16, n_gpus=1)
    assert e.value.code == mps.capi.ERR_ARG and "col_idx[10]" in str(e.value)
    dec = rp.copy(); dec[-2] = dec[-1] + 1
    with pytest.raises(mps.MpsError) as e:
        mps.MultiGpu(dec, col, None, n, 16, n_gpus=1)
    assert e.value.code == mps.capi.ERR_ARG


@pytest.mark.parametrize("dim", [4, 16, 64, 128])
@pytest.mark.parametrize("cost", [1, 8, 600, 1000, 2000, 5000, 10000, 10**6, 2**31 - 1])
def test_every_cost_has_a_layout_that_fits_shared_memory(mps, dim, cost):
    """`cost` fixes the reported chunk diagonals; the execution tile is cut finer when a chunk is longer than a tile
    can stage, so no value the reference program accepts is refused."""
    n, nnz = 1 << 21, 65_637_498
    for dtype in (mps.F32, mps.F16):
        lay = mps.layout_query(n, nnz, dim, dtype, cost)
        assert lay["shared_bytes_per_block"] <= 64 * 1024
        assert lay["tile_items"] == lay["unit_items"] * lay["units_per_tile"]
        assert (lay["n_tiles"] - 1) * lay["tile_items"] < n + 1 + nnz <= lay["n_tiles"] * lay["tile_items"]
        _, ipt = mps.chunk_count(n, nnz, cost)
        if lay["units_per_chunk"] > 1:   # a unit is a part of one chunk
            k = lay["units_per_chunk"]
            assert lay["unit_items"] == -(-ipt // k)
        else:                            # a unit is a whole number of chunks
            assert lay["unit_items"] % ipt == 0
    small = mps.layout_query(4096, 100882, 16, mps.F32, 10**6)
    assert small["shared_bytes_per_block"] <= 64 * 1024 and small["n_tiles"] >= 1


def test_tile_model_with_sub_chunk_units_still_close_to_fp64(orc, graphs):
    """The CPU model follows any unit size, not only whole chunks."""
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 16, seed=1)
    ref = orc.spmm_f64(rp, col, val, B)
    scale = orc.spmm_abs_f64(rp, col, val, B)
    for unit_items, units in ((7, 4), (51, 16), (1000, 2), (10**6, 1)):
        got = orc.tile_model(rp, col, val, B, 8, units, 1, 32, unit_items=unit_items)
        assert (np.abs(got.astype(np.float64) - ref) <= 1e-6 + 1e-5 * scale).all(), (unit_items, units)
    a = orc.tile_model(rp, col, val, B, 8, 64, 4, 32)
    p = orc.chunk_count(len(rp) - 1, len(col), 8)
    ipt = orc.items_per_chunk(len(rp) - 1, len(col), p)
    b = orc.tile_model(rp, col, val, B, 8, 16, 1, 32, unit_items=4 * ipt)   # the same layout named in items
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
