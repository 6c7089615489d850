"""Parity of the CUDA path (through the C ABI) with the oracle, on a B200.

Three gates per case:
  1. partition coordinates and the six schedule arrays: bit-exact with the reference's own
     functions (golden vectors) and with the oracle's restatement;
  2. C bit-exact with the CPU model of the kernel's summation order (oracle section 5);
  3. C within tolerance of the fp64 loop: fp32 |d| <= 1e-6 + 1e-5*scale, fp16 1e-2, where
     scale = sum_k |a_ik b_kj| (element-wise relative error is unbounded under cancellation; the
     fraction of elements that also meet the literal |d| <= 1e-6 + 1e-5*|ref| form is reported
     for the benchmark configurations).
"""
import os

import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_partition.npz")


def _dev(a, cuda):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


def _run(mps, cuda, rp, col, val, B, cost, tune=None, tpw=1, walk=None):
    n, nnz, dim = len(rp) - 1, len(col), B.shape[1]
    half = B.dtype == np.float16
    plan = mps.Plan(n, nnz, dim, mps.F16 if half else mps.F32, cost, tpw, device=cuda)
    if tune:
        plan.tune(**tune)
    if walk is not None:
        plan.set_walk(walk)
    d_rp, d_col, d_val, d_B = _dev(rp, cuda), _dev(col, cuda), _dev(val, cuda), _dev(B, cuda)
    plan.partition(d_rp)
    out = torch.full((n, dim), float("nan"), dtype=d_B.dtype, device=cuda)  # every element must be overwritten
    plan.spmm(d_rp, d_col, d_val, d_B, out=out)
    plan.sync_check()
    info = plan.info()
    plan.close()
    return out.cpu().numpy(), info


def _check(orc, rp, col, val, B, got, info, cost, tol):
    half = B.dtype == np.float16
    model = orc.tile_model(rp, col, val, B, cost, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], is_half=half, unit_items=info["unit_items"],
                           groups=info["groups_per_unit"])
    assert not np.isnan(got.astype(np.float32)).any(), "some element of C was never written"
    same = _bits(got) == _bits(model)
    assert same.all(), f"{(~same).sum()} elements differ from the CPU model (first at {np.argwhere(~same)[0]})"
    ref = orc.spmm_f64(rp, col, val, B, is_half=half)
    scale = orc.spmm_abs_f64(rp, col, val, B, is_half=half)
    err = np.abs(got.astype(np.float64) - ref)
    bound = 1e-6 + tol * (np.maximum(scale, np.abs(ref)) if half else scale)
    assert (err <= bound).all(), f"max error {err.max()} beyond tolerance"
    return float((err <= 1e-6 + tol * np.abs(ref)).mean())


# ------------------------------------------------------------------ partition / schedule

def test_partition_and_schedule_bit_exact_with_reference_vectors(mps, orc, cuda):
    g = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in g.files})
    checked = 0
    for name in names:
        rp = g[f"{name}/row_ptr"]
        d_rp = _dev(rp, cuda)
        for key in [k for k in g.files if k.startswith(name + "/cost") and k.endswith("/xy")]:
            cost = int(key.split("/")[1][4:])
            p = int(g[f"{name}/cost{cost}/n_chunks"])
            assert mps.chunk_count(len(rp) - 1, int(rp[-1]), cost)[0] == p
            xy = mps.partition_device(d_rp, p).cpu().numpy()
            assert np.array_equal(xy, g[key]), (name, cost)
            six = mps.schedule_device(d_rp, p).cpu().numpy()
            assert np.array_equal(six, g[f"{name}/cost{cost}/six"]), (name, cost)
            checked += 1
    assert checked >= 30


def test_partition_bit_exact_with_oracle_on_a_mid_size_graph(mps, orc, graphs, cuda):
    rp, _ = graphs.rmat_csr(17, 16, seed=2)
    d_rp = _dev(rp, cuda)
    for cost in (4, 8, 16, 32):
        p, _ = mps.chunk_count(len(rp) - 1, int(rp[-1]), cost)
        assert np.array_equal(mps.partition_device(d_rp, p).cpu().numpy(), orc.partition(rp, p)), cost
        assert np.array_equal(mps.schedule_device(d_rp, p).cpu().numpy(), orc.schedule(rp, p)), cost


# ------------------------------------------------------------------ SpMM, benchmark configurations

@pytest.mark.parametrize("dim", [16, 32, 64, 128])
@pytest.mark.parametrize("cost", [4, 8, 16, 32])
def test_c1_rmat_fp32(mps, orc, graphs, cuda, dim, cost):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, dim, seed=1)
    got, info = _run(mps, cuda, rp, col, val, B, cost, tpw=32)  # tpw 32 as configuration 1 asks: clamped
    assert info["threads_per_warp"] == (32 // dim if dim <= 32 else 1)
    _check(orc, rp, col, val, B, got, info, cost, 1e-5)


def test_c1_unit_values_as_the_csr_file_has_none(mps, orc, graphs, cuda):
    rp, col = cases.c1_rmat()
    B = graphs.dense_uniform(len(rp) - 1, 16, seed=1)
    got, info = _run(mps, cuda, rp, col, None, B, 8)
    _check(orc, rp, col, None, B, got, info, 8, 1e-5)
    ones = np.ones(len(col), np.float32)
    got2, _ = _run(mps, cuda, rp, col, ones, B, 8)
    assert np.array_equal(_bits(got), _bits(got2))


def test_c2_batched_structured(mps, orc, graphs, cuda):
    rp, col = cases.c2_batched()
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 16, seed=1)
    got, info = _run(mps, cuda, rp, col, val, B, 8)
    frac = _check(orc, rp, col, val, B, got, info, 8, 1e-5)
    assert frac > 0.999  # short rows: the literal element-wise form holds almost everywhere


@pytest.mark.parametrize("dim", [128, 64, 8])
def test_c4_fp16_storage_fp32_accumulate(mps, orc, graphs, cuda, dim):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col, "f16")
    B = graphs.dense_normal_f16(len(rp) - 1, dim, seed=1)
    got, info = _run(mps, cuda, rp, col, val, B, 8)
    assert got.dtype == np.float16
    _check(orc, rp, col, val, B, got, info, 8, 1e-2)
    # against an fp32 run of the same operands: within 1e-2 relative of the result's scale
    got32, _ = _run(mps, cuda, rp, col, val.astype(np.float32), B.astype(np.float32), 8)
    scale = orc.spmm_abs_f64(rp, col, val, B, is_half=True)
    assert (np.abs(got.astype(np.float64) - got32) <= 1e-6 + 1e-2 * np.maximum(scale, np.abs(got32))).all()


# ------------------------------------------------------------------ shapes and edge cases

@pytest.mark.parametrize("dim", [4, 8, 12, 24, 48, 96, 100, 160, 256, 260, 1, 5, 7, 33, 70])
def test_generic_dims_fp32(mps, orc, graphs, cuda, dim):
    rp, col = cases.c2_batched(120)
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, dim, seed=2)
    got, info = _run(mps, cuda, rp, col, val, B, 8)
    _check(orc, rp, col, val, B, got, info, 8, 1e-5)


@pytest.mark.parametrize("dim", [16, 40, 256, 264, 3, 20])
def test_generic_dims_fp16(mps, orc, graphs, cuda, dim):
    rp, col = cases.c2_batched(120)
    val = graphs.gcn_values(rp, col, "f16")
    B = graphs.dense_normal_f16(len(rp) - 1, dim, seed=2)
    got, info = _run(mps, cuda, rp, col, val, B, 8)
    _check(orc, rp, col, val, B, got, info, 8, 1e-2)


@pytest.mark.parametrize("name", sorted(cases.edge_cases().keys()))
def test_edge_case_graphs(mps, orc, cuda, name):
    rp, col = cases.edge_cases()[name]
    n = len(rp) - 1
    n_cols = max(int(col.max()) + 1 if len(col) else 1, n)
    rng = np.random.default_rng(3)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    for dim in (12, 64, 5):
        B = rng.uniform(-1, 1, (n_cols, dim)).astype(np.float32)
        for cost, tune in ((1, None), (3, dict(chunks_per_unit=3)), (8, dict(fused_fixup=0)), (8, dict(chunks_per_unit=1)), (32, dict(unroll=8))):
            got, info = _run(mps, cuda, rp, col, val, B, cost, tune)
            _check(orc, rp, col, val, B, got, info, cost, 1e-5)


@pytest.mark.parametrize("dim,half,walk", [(64, False, None), (16, False, None), (128, True, None), (20, False, None), (16, False, 1)])
def test_tiles_with_more_row_ends_than_the_row_ptr_window_holds(mps, orc, cuda, dim, half, walk):
    """The shared-memory window for row_ptr holds a quarter of a tile's merge items; tiles of very short and empty rows
    have more markers than that and read row_ptr from global memory instead.  Same sums either way."""
    rng = np.random.default_rng(17)
    lens = rng.integers(0, 3, 300_000)
    lens[1000:1200] = 0                      # a run of empty rows
    lens[50_000] = 40_000                    # and one long row among them
    rp, col = cases.from_lengths(lens, 200_000, 23)
    val = rng.uniform(-1, 1, len(col)).astype(np.float16 if half else np.float32)
    B = rng.uniform(-1, 1, (200_000, dim)).astype(np.float16 if half else np.float32)
    got, info = _run(mps, cuda, rp, col, val, B, 16, walk=walk)
    assert info["tile_items"] >= 400 and (lens <= 2).mean() > 0.99   # markers per tile ~ tile_items / 2 > tile_items / 4
    _check(orc, rp, col, val, B, got, info, 16, 1e-2 if half else 1e-5)


def test_long_rows_take_the_strand_order(mps, orc, cuda):
    """A row spanning more than long_chain tiles is summed in 16 interleaved strands, still by the tile
    block whose contribution arrives last: one kernel per SpMM."""
    rp, col = cases.edge_cases()["one_giant_row"]
    rng = np.random.default_rng(5)
    B = rng.uniform(-1, 1, (6000, 64)).astype(np.float32)
    for fused in (1, 0):
        got, info = _run(mps, cuda, rp, col, None, B, 1, dict(chunks_per_unit=1, fused_fixup=fused))
        # fused: the last-arriving tile block sums the 150-tile chain; unfused: one fix-up launch whose first block takes the long row
        assert (info["kernels_per_call"], info["long_rows"]) == ((1, 0) if fused else (2, 1))
        assert 5000 // (info["chunks_per_tile"] * info["items_per_chunk"]) > info["long_chain"]
        _check(orc, rp, col, None, B, got, info, 1, 1e-5)


def test_rows_spanning_thousands_of_tiles_take_the_second_kernel(mps, orc, cuda):
    rp, col = cases.from_lengths([3, 80000, 2, 0, 5], 90000, 21)
    rng = np.random.default_rng(6)
    val = rng.uniform(-1, 1, len(col)).astype(np.float32)
    B = rng.uniform(-1, 1, (90000, 64)).astype(np.float32)
    got, info = _run(mps, cuda, rp, col, val, B, 1, dict(chunks_per_unit=1))
    assert info["long_rows"] == 1 and info["kernels_per_call"] == 2  # 10,000+ tiles: one fix-up launch after the tile kernel, its first block for the long row
    assert 80000 // (info["chunks_per_tile"] * info["items_per_chunk"]) > info["very_long"]
    _check(orc, rp, col, val, B, got, info, 1, 1e-5)


@pytest.mark.parametrize("tune", [dict(chunks_per_unit=1), dict(chunks_per_unit=3), dict(chunks_per_unit=20, unroll=4),
                                  dict(unroll=8), dict(bulk_staging=False), dict(block_threads=128), dict(block_threads=256, unroll=4),
                                  dict(fused_fixup=0), dict(fused_fixup=1), dict(fused_fixup=0, chunks_per_unit=1)])
def test_tuning_knobs_keep_parity(mps, orc, graphs, cuda, tune):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 64, seed=1)
    got, info = _run(mps, cuda, rp, col, val, B, 8, tune)
    _check(orc, rp, col, val, B, got, info, 8, 1e-5)


def test_bulk_and_plain_staging_agree_and_unaligned_inputs_work(mps, orc, graphs, cuda):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    n, nnz = len(rp) - 1, len(col)
    B = graphs.dense_uniform(n, 32, seed=1)
    a, info = _run(mps, cuda, rp, col, val, B, 8)
    b, _ = _run(mps, cuda, rp, col, val, B, 8, dict(bulk_staging=False))
    assert np.array_equal(_bits(a), _bits(b))
    # col_idx / val / row_ptr that start 4 bytes into an allocation: 16-byte staging is not possible,
    # the plain-load path must take over and give the same bits
    d_B = _dev(B, cuda)
    pad = lambda x: torch.cat([torch.zeros(1, dtype=x.dtype, device=cuda), x])[1:]
    d_rp, d_col, d_val = pad(_dev(rp, cuda)), pad(_dev(col, cuda)), pad(_dev(val, cuda))
    assert d_col.data_ptr() % 16 == 4
    plan = mps.Plan(n, nnz, 32, mps.F32, 8, device=cuda)
    plan.partition(d_rp)
    c = plan.spmm(d_rp, d_col, d_val, d_B).cpu().numpy()
    plan.sync_check()
    assert np.array_equal(_bits(a), _bits(c))
    # B that is not 16-byte aligned cannot be gathered with 128-bit loads: a clear error, no fault
    with pytest.raises(mps.MpsError) as e:
        plan.spmm(d_rp, d_col, d_val, pad(d_B.reshape(-1))[: (n - 1) * 32].reshape(n - 1, 32))
    assert e.value.code == mps.capi.ERR_ALIGN
    plan.close()


def test_deterministic_and_repeat_safe(mps, graphs, cuda):
    """Two launches give the same bits and a second launch into the same C does not accumulate
    (the reference's atomics do both wrong: src/MergePathSpMM.cu:204,231-243)."""
    rp, col = graphs.rmat_csr(16, 32, seed=5)
    val = graphs.gcn_values(rp, col)
    n, nnz = len(rp) - 1, len(col)
    d_rp, d_col, d_val = _dev(rp, cuda), _dev(col, cuda), _dev(val, cuda)
    d_B = _dev(graphs.dense_uniform(n, 64, seed=6), cuda)
    plan = mps.Plan(n, nnz, 64, mps.F32, 8, device=cuda)
    plan.partition(d_rp)
    c1 = plan.spmm(d_rp, d_col, d_val, d_B)
    first = c1.clone()
    for _ in range(5):
        plan.spmm(d_rp, d_col, d_val, d_B, out=c1)
    c2 = plan.spmm(d_rp, d_col, d_val, d_B)
    plan.sync_check()
    assert torch.equal(first, c1) and torch.equal(first, c2)
    plan.close()


@pytest.mark.parametrize("which", ["small_fused", "mid_unfused"])
def test_launches_can_be_captured_in_a_cuda_graph(mps, graphs, cuda, which):
    """mps_spmm only enqueues kernels on the given stream, so a loop of multiplies can be captured once and
    replayed (launch-bound small graphs are where that pays).  Replays must reproduce the eager result."""
    rp, col = cases.c1_rmat() if which == "small_fused" else graphs.rmat_csr(17, 32, seed=9)
    val = graphs.gcn_values(rp, col)
    n, nnz = len(rp) - 1, len(col)
    d_rp, d_col, d_val = _dev(rp, cuda), _dev(col, cuda), _dev(val, cuda)
    d_B = _dev(graphs.dense_uniform(n, 32, seed=6), cuda)
    plan = mps.Plan(n, nnz, 32, mps.F32, 16, device=cuda)
    plan.partition(d_rp)
    assert plan.info()["kernels_per_call"] == (1 if which == "small_fused" else 2)
    eager = plan.spmm(d_rp, d_col, d_val, d_B).clone()
    plan.sync_check()
    out = torch.zeros_like(eager)
    side = torch.cuda.Stream(device=cuda)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(4):
                plan.spmm(d_rp, d_col, d_val, d_B, out=out, stream=side)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    plan.sync_check()
    plan.close()


def test_errors_are_codes_not_faults(mps, cuda):
    plan = mps.Plan(10, 20, 16, mps.F32, 8, device=cuda)
    z = torch.zeros(64, dtype=torch.int32, device=cuda)
    f = torch.zeros(10 * 16, dtype=torch.float32, device=cuda)
    with pytest.raises(mps.MpsError) as e:
        plan.spmm(z, z, None, f, out=f.clone())
    assert e.value.code == mps.capi.ERR_STATE  # partition not called yet
    with pytest.raises(mps.MpsError) as e:
        plan.tune(unroll=5)
    assert e.value.code == mps.capi.ERR_ARG
    plan.close()
    with pytest.raises(mps.MpsError) as e:
        mps.Plan(10, 20, 0, mps.F32, 8, device=cuda)
    assert e.value.code == mps.capi.ERR_ARG


def test_random_matrices_bit_exact_with_the_model(mps, orc, cuda):
    """Property test: random row lengths (empty rows, a few long rows, runs of short ones), random column indices and
    values, random dim (vector lanes, narrow fp16 lanes, scalar lanes, column slabs) / cost / dtype / layout knob - C is bit-equal to the CPU model of the summation order and
    within tolerance of the fp64 loop, whatever the shape."""
    from hypothesis import given, settings, strategies as st, HealthCheck
    lengths = st.lists(st.one_of(st.just(0), st.integers(0, 6), st.integers(0, 90), st.integers(200, 3000)), min_size=1, max_size=120)
    tunes = st.sampled_from([None, None, dict(fused_fixup=0), dict(chunks_per_unit=1), dict(unroll=4), dict(block_threads=128), dict(bulk_staging=False)])

    @settings(max_examples=150, deadline=None, suppress_health_check=list(HealthCheck))
    @given(lengths, st.sampled_from([3, 4, 6, 12, 16, 20, 30, 32, 50, 64, 100, 128]), st.sampled_from([1, 3, 8, 16, 600]), st.booleans(), st.booleans(), tunes,
           st.integers(0, 2 ** 31 - 1))
    def run(lens, dim, cost, half, with_values, tune, seed):
        rng = np.random.default_rng(seed)
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        n, nnz = len(rp) - 1, int(rp[-1])
        n_cols = n
        col = rng.integers(0, n_cols, nnz).astype(np.int32)
        dt = np.float16 if half else np.float32
        val = rng.uniform(-1, 1, nnz).astype(dt) if with_values else None
        B = rng.uniform(-1, 1, (n_cols, dim)).astype(dt)
        got, info = _run(mps, cuda, rp, col, val, B, cost, tune)
        _check(orc, rp, col, val, B, got, info, cost, 1e-2 if half else 1e-5)

    run()


def test_host_buffer_call_equals_device_path(mps, orc, graphs, cuda):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 64, seed=1)
    dev, info = _run(mps, cuda, rp, col, val, B, 8)
    host = mps.spmm_host(rp, col, val, B, cost=8)
    assert np.array_equal(_bits(dev), _bits(host))
    host2 = mps.spmm_host(rp, col, val, B, cost=8)   # workspace reuse
    assert np.array_equal(_bits(host), _bits(host2))
    Bh = B.astype(np.float16)
    vh = val.astype(np.float16)
    devh, _ = _run(mps, cuda, rp, col, vh, Bh, 8)
    assert np.array_equal(_bits(devh), _bits(mps.spmm_host(rp, col, vh, Bh, cost=8)))
    mps.capi.lib().mps_host_workspace_release()


def test_host_buffer_call_pipelines_large_inputs_over_row_slabs(mps, orc, graphs, cuda):
    """Above 4 Mi merge items the host call cuts A into row slabs (equal nnz + 4*rows) so that C flows back
    while later slabs of A still upload; each slab must equal the device path run on that slab alone."""
    rp, col = graphs.rmat_csr(19, 32, seed=3)
    val = graphs.gcn_values(rp, col)
    n, nnz = len(rp) - 1, len(col)
    n_slabs = min(16, (n + nnz) // (4 << 20))
    assert n_slabs >= 2
    B = graphs.dense_uniform(n, 32, seed=4)
    pinned = [torch.from_numpy(a).pin_memory() for a in (rp, col, val, B)]
    out = torch.empty((n, 32), dtype=torch.float32).pin_memory()
    for _ in range(2):   # second call reuses the workspace and the per-slab plans
        out.fill_(float("nan"))
        mps.spmm_host(*pinned, out=out, cost=16)
        host = out.numpy()
        b = mps.slab_bounds(rp, n_slabs, "items", 4)
        for s in range(n_slabs):
            r0, r1 = int(b[s]), int(b[s + 1])
            srp = mps.slab_rebase(rp, r0, r1)
            got, _ = _run(mps, cuda, srp, col[rp[r0]:rp[r1]], val[rp[r0]:rp[r1]], B, 16)
            assert np.array_equal(_bits(got), _bits(host[r0:r1])), s
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(host.astype(np.float64) - orc.spmm_f64(rp, col, val, B)) <= 1e-6 + 1e-5 * scale).all()
    mps.capi.lib().mps_host_workspace_release()


def test_scaled_host_call_equals_the_scaled_device_path(mps, orc, graphs, cuda):
    """mps_spmm_host_scaled: the factor vectors travel instead of a value per non-zero; one slab: bit-equal to
    mps_spmm_scaled on device buffers; several slabs: each slab bit-equal to the device path on that slab, the whole
    within tolerance of the fp64 product with values row_scale[i] * col_scale[j]."""
    rp, col = cases.c1_rmat()
    n, nnz = len(rp) - 1, len(col)
    rng = np.random.default_rng(5)
    rs = (1.0 / np.sqrt(np.maximum(np.diff(rp), 1).astype(np.float64))).astype(np.float32)
    cs = rng.uniform(0.5, 1.5, n).astype(np.float32)
    B = graphs.dense_uniform(n, 64, seed=1)

    def device_path(srp, scol, srs):
        plan = mps.Plan(len(srp) - 1, len(scol), B.shape[1], mps.F32, 16, device=cuda)
        d = [torch.from_numpy(a).to(cuda) if a is not None else None for a in (srp, scol, srs, cs, B)]
        plan.partition(d[0])
        out = plan.spmm_scaled(d[0], d[1], d[2], d[3], d[4])
        plan.sync_check()
        plan.close()
        return out.cpu().numpy()

    host = mps.spmm_host_scaled(rp, col, rs, cs, B, cost=16)
    assert np.array_equal(_bits(host), _bits(device_path(rp, col, rs)))
    only_cols = mps.spmm_host_scaled(rp, col, None, cs, B, cost=16)
    assert np.array_equal(_bits(only_cols), _bits(device_path(rp, col, None)))

    rp, col = graphs.rmat_csr(19, 32, seed=3)
    n, nnz = len(rp) - 1, len(col)
    n_slabs = min(16, (n + nnz) // (4 << 20))
    assert n_slabs >= 2
    rs = (1.0 / np.sqrt(np.maximum(np.diff(rp), 1).astype(np.float64))).astype(np.float32)
    cs = rs.copy()
    B = graphs.dense_uniform(n, 32, seed=4)
    pinned = [torch.from_numpy(a).pin_memory() for a in (rp, col, rs, cs, B)]
    out = torch.full((n, 32), float("nan"), dtype=torch.float32).pin_memory()
    mps.spmm_host_scaled(*pinned, out=out, cost=16)
    host = out.numpy()
    b = mps.slab_bounds(rp, n_slabs, "items", 4)
    for s in (0, n_slabs - 1):
        r0, r1 = int(b[s]), int(b[s + 1])
        got = device_path(mps.slab_rebase(rp, r0, r1), col[rp[r0]:rp[r1]], rs[r0:r1])
        assert np.array_equal(_bits(got), _bits(host[r0:r1])), s
    val = (np.repeat(rs, np.diff(rp)).astype(np.float64) * cs[col].astype(np.float64)).astype(np.float32)
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(host.astype(np.float64) - orc.spmm_f64(rp, col, val, B)) <= 1e-6 + 2e-5 * scale).all()
    mps.capi.lib().mps_host_workspace_release()


@pytest.mark.parametrize("dim,tune", [(16, None), (64, None), (64, dict(fused_fixup=0)), (20, None), (128, dict(chunks_per_unit=1, block_threads=128))])
def test_scaled_product_bit_exact_with_its_model(mps, orc, graphs, cuda, dim, tune):
    """mps_spmm_scaled: A's values are row_scale[i] * col_scale[j] (GCN: both = degree^-1/2), never stored."""
    rp, col = cases.c1_rmat()
    n, nnz = len(rp) - 1, len(col)
    rng = np.random.default_rng(11)
    rs = (1.0 / np.sqrt(np.diff(rp).astype(np.float64))).astype(np.float32)
    cs = rng.uniform(0.5, 1.5, n).astype(np.float32)
    B = graphs.dense_uniform(n, dim, seed=1)
    plan = mps.Plan(n, nnz, dim, mps.F32, 8, device=cuda)
    if tune:
        plan.tune(**tune)
    d_rp, d_col, d_rs, d_cs, d_B = (_dev(a, cuda) for a in (rp, col, rs, cs, B))
    plan.partition(d_rp)
    out = torch.full((n, dim), float("nan"), dtype=torch.float32, device=cuda)
    plan.spmm_scaled(d_rp, d_col, d_rs, d_cs, d_B, out=out)
    plan.sync_check()
    info = plan.info()
    got = out.cpu().numpy()
    model = orc.tile_model_scaled(rp, col, rs, cs, B, 8, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], unit_items=info["unit_items"])
    assert np.array_equal(_bits(got), _bits(model))
    rows = np.repeat(np.arange(n), np.diff(rp))
    val = (rs.astype(np.float64)[rows] * cs.astype(np.float64)[col]).astype(np.float32)
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(got.astype(np.float64) - orc.spmm_f64(rp, col, val, B)) <= 2e-6 + 2e-5 * scale).all()
    # the unscaled entry point still works on the same plan afterwards
    plain = plan.spmm(d_rp, d_col, None, d_B).cpu().numpy()
    assert np.array_equal(_bits(plain), _bits(orc.tile_model(rp, col, None, B, 8, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], unit_items=info["unit_items"])))
    plan.close()
    with pytest.raises(mps.MpsError) as e:
        ph = mps.Plan(n, nnz, 16, mps.F16, 8, device=cuda)
        ph.partition(d_rp)
        ph.spmm_scaled(d_rp, d_col, d_rs, d_cs, _dev(B[:, :16].astype(np.float16), cuda))
    assert e.value.code == mps.capi.ERR_UNSUPPORTED


def test_scaled_product_on_long_rows(mps, orc, cuda):
    rp, col = cases.from_lengths([3, 30000, 2, 0, 5], 40000, 21)
    rng = np.random.default_rng(6)
    rs = rng.uniform(0.5, 1.5, len(rp) - 1).astype(np.float32)
    cs = rng.uniform(-1, 1, 40000).astype(np.float32)
    B = rng.uniform(-1, 1, (40000, 32)).astype(np.float32)
    n, nnz = len(rp) - 1, len(col)
    for tune in (dict(chunks_per_unit=1), dict(chunks_per_unit=1, fused_fixup=1)):
        plan = mps.Plan(n, nnz, 32, mps.F32, 1, device=cuda)
        plan.tune(**tune)
        d = [_dev(a, cuda) for a in (rp, col, rs, cs, B)]
        plan.partition(d[0])
        got = plan.spmm_scaled(*d).cpu().numpy()
        plan.sync_check()
        info = plan.info()
        model = orc.tile_model_scaled(rp, col, rs, cs, B, 1, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], unit_items=info["unit_items"])
        assert np.array_equal(_bits(got), _bits(model)), tune
        plan.close()


def test_scaled_product_with_one_factor_only(mps, orc, graphs, cuda):
    """Either scale may be absent (= ones); the row-only form equals the full form on a B that already carries the
    column factor, which is how a caller avoids the per-non-zero gather of col_scale."""
    rp, col = cases.c1_rmat()
    n, nnz, dim = len(rp) - 1, len(col), 64
    rng = np.random.default_rng(12)
    rs = rng.uniform(0.5, 1.5, n).astype(np.float32)
    cs = rng.uniform(0.5, 1.5, n).astype(np.float32)
    B = graphs.dense_uniform(n, dim, seed=2)
    plan = mps.Plan(n, nnz, dim, mps.F32, 8, device=cuda)
    d_rp, d_col, d_rs, d_cs, d_B = (_dev(a, cuda) for a in (rp, col, rs, cs, B))
    plan.partition(d_rp)
    info = plan.info()
    shape = (8, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], info["unit_items"])
    for r, c, dr, dc in ((rs, None, d_rs, None), (None, cs, None, d_cs)):
        got = plan.spmm_scaled(d_rp, d_col, dr, dc, d_B).cpu().numpy()
        plan.sync_check()
        assert np.array_equal(_bits(got), _bits(orc.tile_model_scaled(rp, col, r, c, B, *shape)))
    Bs = (B * cs[:, None]).astype(np.float32)
    got = plan.spmm_scaled(d_rp, d_col, d_rs, None, _dev(Bs, cuda)).cpu().numpy()
    rows = np.repeat(np.arange(n), np.diff(rp))
    val = (rs.astype(np.float64)[rows] * cs.astype(np.float64)[col]).astype(np.float32)
    scale = orc.spmm_abs_f64(rp, col, val, B)
    assert (np.abs(got.astype(np.float64) - orc.spmm_f64(rp, col, val, B)) <= 2e-6 + 2e-5 * scale).all()
    with pytest.raises(mps.MpsError):
        plan.spmm_scaled(d_rp, d_col, None, None, d_B)
    plan.close()


def test_mid_size_graph_unfused_by_size_is_bit_exact_with_the_cpu_model(mps, orc, graphs, cuda):
    """Above 2048 tiles the cross-tile fix-up is the separate fixup_kernel (four columns per lane, its first blocks for
    the rows that span more than 32 tiles) - the form every large multiply takes.  R-MAT 2^17 reaches it by size alone."""
    rp, col = graphs.rmat_csr(17, 32, seed=9)
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    for dim, half in ((32, False), (64, False), (16, False), (128, True), (20, False)):
        if half:
            B, v = graphs.dense_normal_f16(n, dim, seed=6), val.astype(np.float16)
        else:
            B, v = graphs.dense_uniform(n, dim, seed=6), val
        got, info = _run(mps, cuda, rp, col, v, B, 16)
        assert info["n_tiles"] > 2048 and info["fused_fixup"] == 0 and info["kernels_per_call"] == 2, info
        _check(orc, rp, col, v, B, got, info, 16, 1e-2 if half else 1e-5)
    assert info["long_rows"] >= 0


@pytest.mark.parametrize("dim", [4, 16, 64, 128])
@pytest.mark.parametrize("cost", [1000, 10000, 10**7])
def test_costs_beyond_one_tile_are_cut_into_sub_chunk_units(mps, orc, graphs, cuda, dim, cost):
    """The reference's command line takes any cost; a chunk longer than a tile can stage is walked as several units."""
    rp, col = graphs.rmat_csr(17, 16, seed=4)
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, dim, seed=5)
    got, info = _run(mps, cuda, rp, col, val, B, cost)
    assert info["shared_bytes_per_block"] <= 64 * 1024
    if cost >= 10000:
        assert info["units_per_chunk"] > 1
    _check(orc, rp, col, val, B, got, info, cost, 1e-5)


def test_host_call_with_b_already_on_the_device(mps, graphs, cuda):
    """mps_spmm_host_resident_b: A and C are host buffers, B is a device buffer that another stream is still
    completing when the call starts; the result equals the all-host call bit for bit."""
    rp, col = graphs.rmat_csr(19, 32, seed=3)
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 32, seed=4)
    want = mps.spmm_host(rp, col, val, B, cost=16)
    side = torch.cuda.Stream(device=cuda)
    d_B = torch.empty((n, 32), dtype=torch.float32, device=cuda)
    hB = torch.from_numpy(B).pin_memory()
    pinned = [torch.from_numpy(a).pin_memory() for a in (rp, col, val)]
    out = torch.full((n, 32), float("nan"), dtype=torch.float32).pin_memory()
    for _ in range(2):
        d_B.zero_()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            d_B.copy_(hB, non_blocking=True)       # B arrives on another stream while A uploads
            mps.spmm_host_resident_b(*pinned, d_B, out, cost=16, stream=side)
        assert np.array_equal(_bits(out.numpy()), _bits(want))
        out.fill_(float("nan"))
    mps.capi.lib().mps_host_workspace_release()


@pytest.mark.parametrize("dim,half", [(16, False), (32, False), (64, False), (8, False), (12, False), (24, False), (32, True), (64, True), (128, True)])
def test_warp_per_unit_walk_is_bit_exact_with_its_model(mps, orc, graphs, cuda, dim, half):
    """mps_plan_set_walk(1): a warp walks one unit, its 32/lanes groups take consecutive non-zeros and their partial sums
    are combined with shuffles in a fixed tree at row ends.  Power-law graph (fused and unfused fix-up), the structured
    graph of short rows, and every edge-case shape."""
    def operands(n_cols, seed):
        if half:
            return graphs.dense_normal_f16(n_cols, dim, seed=seed)
        return graphs.dense_uniform(n_cols, dim, seed=seed)
    for rp, col in (cases.c1_rmat(), cases.c2_batched(400)):
        val = graphs.gcn_values(rp, col, "f16" if half else "f32")
        B = operands(len(rp) - 1, 1)
        for tune in (None, dict(fused_fixup=0), dict(chunks_per_unit=3)):
            got, info = _run(mps, cuda, rp, col, val, B, 8, tune, walk=1)
            assert info["groups_per_unit"] == 32 // info["lanes_per_chunk"] > 1 and info["units_per_tile"] == 2
            _check(orc, rp, col, val, B, got, info, 8, 1e-2 if half else 1e-5)
    rng = np.random.default_rng(3)
    for name, (rp, col) in sorted(cases.edge_cases().items()):
        n_cols = max(int(col.max()) + 1 if len(col) else 1, len(rp) - 1)
        val = rng.uniform(-1, 1, len(col)).astype(np.float16 if half else np.float32)
        B = operands(n_cols, 2)
        for cost in (1, 8):
            got, info = _run(mps, cuda, rp, col, val, B, cost, walk=1)
            _check(orc, rp, col, val, B, got, info, cost, 1e-2 if half else 1e-5)


def test_warp_per_unit_walk_on_a_mid_size_graph_and_where_it_does_not_apply(mps, orc, graphs, cuda):
    rp, col = graphs.rmat_csr(17, 32, seed=9)
    val = graphs.gcn_values(rp, col)
    B = graphs.dense_uniform(len(rp) - 1, 16, seed=6)
    got, info = _run(mps, cuda, rp, col, val, B, 16, walk=1)
    assert info["groups_per_unit"] == 8 and info["fused_fixup"] == 0
    _check(orc, rp, col, val, B, got, info, 16, 1e-5)
    # 32 lanes per row, generic dims and other block sizes keep the lane-group walk whatever is asked
    for dim, tune in ((128, None), (20, None), (16, dict(block_threads=128))):
        Bx = graphs.dense_uniform(len(rp) - 1, dim, seed=6)
        got, info = _run(mps, cuda, rp, col, val, Bx, 16, tune, walk=1)
        assert info["groups_per_unit"] == (1 if dim != 20 else info["groups_per_unit"])
        _check(orc, rp, col, val, Bx, got, info, 16, 1e-5)
    # narrow fp16 rows (four columns per lane) have no warp-per-unit kernel either
    Bh = graphs.dense_normal_f16(len(rp) - 1, 16, seed=6)
    got, info = _run(mps, cuda, rp, col, val.astype(np.float16), Bh, 16, walk=1)
    assert info["groups_per_unit"] == 1 and info["lanes_per_chunk"] == 4
    _check(orc, rp, col, val.astype(np.float16), Bh, got, info, 16, 1e-2)


def test_host_call_reports_a_bad_column_index_without_gathering_by_it(mps, graphs, cuda):
    """With a device the column indices are checked where they land (and replaced by 0 in the workspace copy before the
    multiply runs): the call returns MPS_ERR_ARG naming the first bad position, nothing faults, and the next call works."""
    rp, col = graphs.rmat_csr(19, 32, seed=3)       # large enough for several slabs
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 16, seed=4)
    good = mps.spmm_host(rp, col, val, B, cost=16)
    for where, value in ((len(col) - 5, n), (len(col) // 2, -3), (7, 2**31 - 1)):
        bad = col.copy()
        bad[where] = value
        bad[len(col) - 1] = n + 9                    # a later one as well: the first is reported
        with pytest.raises(mps.MpsError) as e:
            mps.spmm_host(rp, bad, val, B, cost=16)
        assert e.value.code == mps.capi.ERR_ARG and f"col_idx[{where}] = {value}" in str(e.value)
    again = mps.spmm_host(rp, col, val, B, cost=16)
    assert np.array_equal(_bits(again), _bits(good))
    mps.capi.lib().mps_host_workspace_release()


def test_gather_probe_reports_a_plausible_rate(mps, cuda):
    small = torch.zeros(32 << 20, dtype=torch.uint8, device=cuda)     # inside the L2
    rate = mps.gather_probe(small, 256, 1 << 24)
    assert 1000.0 < rate < 100000.0, rate                              # GB/s
    with pytest.raises(mps.MpsError):
        mps.gather_probe(small, 100, 1 << 20)
    idx = torch.randint(0, small.numel() // 256, (1 << 22,), dtype=torch.int32, device=cuda)
    rate = mps.gather_probe_stream(small, 256, idx)
    assert 1000.0 < rate < 100000.0, rate


# ------------------------------------------------------------------ slabs

def test_row_slabs_are_bit_identical_to_their_own_model_and_close_to_the_whole(mps, orc, graphs, cuda):
    rp, col = cases.c1_rmat()
    val = graphs.gcn_values(rp, col)
    n = len(rp) - 1
    B = graphs.dense_uniform(n, 32, seed=1)
    whole, _ = _run(mps, cuda, rp, col, val, B, 8)
    for g in (2, 3, 8):
        b = mps.slab_bounds(rp, g)
        parts = []
        for s in range(g):
            r0, r1 = int(b[s]), int(b[s + 1])
            srp = mps.slab_rebase(rp, r0, r1)
            scol, sval = col[rp[r0]:rp[r1]], val[rp[r0]:rp[r1]]
            got, info = _run(mps, cuda, srp, scol, sval, B, 8)
            model = orc.tile_model(srp, scol, sval, B, 8, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"], unit_items=info["unit_items"])
            assert np.array_equal(_bits(got), _bits(model))
            parts.append(got)
        cat = np.concatenate(parts)
        scale = orc.spmm_abs_f64(rp, col, val, B)
        assert (np.abs(cat.astype(np.float64) - whole) <= 1e-6 + 1e-5 * scale).all()


# ------------------------------------------------------------------ full size, size-independent properties

def test_full_size_rmat21_properties(mps, graphs, cuda):
    """Benchmark configuration 3 (2^21 nodes, ~67M nnz, dim 64), graph built on the device.
    Exact checks that need no oracle pass over 67M non-zeros:
      - unit values and B == 1: every C element equals its row's length (exact in fp32);
      - B = e_j columns (one-hot rows): C counts, per row, the neighbours in each residue class;
      - linearity: A(B1 + B2) == A B1 + A B2 to rounding; two runs are bit-identical."""
    rp, col = graphs.rmat_csr(21, 32, seed=0, device=cuda)
    n, nnz = rp.numel() - 1, col.numel()
    assert n == 1 << 21 and 55_000_000 < nnz <= 2 * (1 << 25) + n
    dim = 64
    plan = mps.Plan(n, nnz, dim, mps.F32, 8, device=cuda)
    plan.partition(rp)
    ones = torch.ones((n, dim), dtype=torch.float32, device=cuda)
    c = plan.spmm(rp, col, None, ones)
    plan.sync_check()
    lens = (rp[1:] - rp[:-1]).to(torch.float32)
    assert torch.equal(c, lens[:, None].expand(n, dim))
    onehot = torch.zeros((n, dim), dtype=torch.float32, device=cuda)
    onehot[torch.arange(n, device=cuda), torch.arange(n, device=cuda) % dim] = 1.0
    c = plan.spmm(rp, col, None, onehot)
    rows = torch.repeat_interleave(torch.arange(n, device=cuda), (rp[1:] - rp[:-1]).to(torch.int64))
    want = torch.zeros(n * dim, dtype=torch.float32, device=cuda)
    want.index_add_(0, rows * dim + (col.to(torch.int64) % dim), torch.ones(nnz, dtype=torch.float32, device=cuda))
    assert torch.equal(c, want.reshape(n, dim))
    del onehot, want, rows, ones
    val = graphs.gcn_values(rp, col)
    b1 = graphs.dense_uniform(n, dim, seed=1, device=cuda)
    b2 = graphs.dense_uniform(n, dim, seed=2, device=cuda)
    c1 = plan.spmm(rp, col, val, b1)
    c2 = plan.spmm(rp, col, val, b2)
    c12 = plan.spmm(rp, col, val, b1 + b2)
    again = plan.spmm(rp, col, val, b1)
    plan.sync_check()
    assert torch.equal(c1, again)
    # GCN values make every row an average-like sum with sum_k |a_ik| <= sqrt(deg_i); |b| < 2
    assert (c12 - (c1 + c2)).abs().max().item() < 1e-4
    plan.close()
    # configuration 4 on the same graph: fp16 storage, fp32 accumulation, dim 128.  Row lengths up to 2048 are
    # exact in fp16, longer ones round once; the one-hot product is exact wherever a count is <= 2048.
    del c1, c2, c12, again, b1, b2
    dim = 128
    plan = mps.Plan(n, nnz, dim, mps.F16, 16, device=cuda)
    plan.partition(rp)
    c = plan.spmm(rp, col, None, torch.ones((n, dim), dtype=torch.float16, device=cuda))
    plan.sync_check()
    assert torch.equal(c, lens.to(torch.float16)[:, None].expand(n, dim))  # one rounding of an exact fp32 sum
    v16 = val.to(torch.float16)
    b16 = graphs.dense_normal_f16(n, dim, seed=3, device=cuda)
    x = plan.spmm(rp, col, v16, b16)
    y = plan.spmm(rp, col, v16, b16)
    plan.sync_check()
    assert torch.equal(x, y) and torch.isfinite(x).all()
    plan.close()


def test_full_size_rmat24_properties(mps, graphs, cuda):
    """Benchmark configuration 5 on one GPU (2^24 nodes, ~1.04e9 nnz, dim 32): 64-bit offsets, a million tiles,
    hub rows of millions of non-zeros.  Unit values and B == 1 give every row's length exactly (< 2^24)."""
    rp, col = graphs.rmat_csr(24, 64, seed=0, device=cuda)
    n, nnz = rp.numel() - 1, col.numel()
    assert n == 1 << 24 and 900_000_000 < nnz < (1 << 30) + n
    torch.cuda.empty_cache()
    dim = 32
    plan = mps.Plan(n, nnz, dim, mps.F32, 16, device=cuda)
    plan.partition(rp)
    lens = (rp[1:] - rp[:-1]).to(torch.float32)
    assert lens.max().item() < 2 ** 24
    c = plan.spmm(rp, col, None, torch.ones((n, dim), dtype=torch.float32, device=cuda))
    plan.sync_check()
    assert torch.equal(c, lens[:, None].expand(n, dim))
    info = plan.info()
    assert info["n_tiles"] > 500_000 and info["long_rows"] > 0
    plan.close()
