"""Numeric parity at the sizes that are benchmarked (R-MAT 2^21 nodes / ~66M non-zeros, and one row slab of the
2^24-node graph), with real values:

  - the WHOLE C of configuration 3 (GCN fp32, cost 16, dim 64 and 16) bit for bit against the CPU model of the
    kernel's summation order, walked by all host threads;
  - sampled rows (>= 4096 random ones, every one of the longest rows, and rows cut by tile boundaries) against
    the fp64 loop on the host, with the scale-aware bound |d| <= 1e-6 + tol * sum_k |a_ik b_kj|
    (tol 1e-5 fp32, 1e-2 fp16);
  - the whole C with unit values against the reference's own kernel on the same graph (row 0 analytically: the
    reference loses chunk 0's share of it, src/MergePathSpMM.cu:365-369,467).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tile_cut_rows(rp, tile_items):
    """Rows that a tile boundary cuts: boundary d lies at x = #{r : rp[r] + r < d}; it cuts row x-1 when
    y = d - x lies strictly inside the row."""
    n = len(rp) - 1
    key = rp.astype(np.int64) + np.arange(n + 1, dtype=np.int64)
    total = n + 1 + int(rp[-1])
    d = np.arange(tile_items, total, tile_items, dtype=np.int64)
    x = np.minimum(np.searchsorted(key, d, "left"), n + 1)
    y = d - x
    ok = (x >= 1) & (x <= n)
    x, y = x[ok], y[ok]
    cut = y > rp[x - 1]
    return np.unique(x[cut] - 1)


def _pick_rows(rp, tile_items, seed, n_random=4096, n_long=64, n_cut=4096):
    rng = np.random.default_rng(seed)
    n = len(rp) - 1
    lens = np.diff(rp.astype(np.int64))
    cut = _tile_cut_rows(rp, tile_items)
    if len(cut) > n_cut:
        cut = rng.choice(cut, n_cut, replace=False)
    rows = np.unique(np.concatenate([rng.integers(0, n, n_random), np.argsort(lens)[-n_long:], cut, [0, n - 1]]))
    return rows, len(cut)


def _sub_csr(rp, col, val, rows):
    lens = (rp[rows + 1] - rp[rows]).astype(np.int64)
    sub_rp = np.zeros(len(rows) + 1, np.int64)
    np.cumsum(lens, out=sub_rp[1:])
    idx = np.concatenate([np.arange(rp[r], rp[r + 1], dtype=np.int64) for r in rows]) if len(rows) else np.zeros(0, np.int64)
    return sub_rp.astype(np.int32), col[idx], None if val is None else val[idx]


def _check_rows(orc, rp, col, val, B, got_rows, rows, tol, half=False):
    srp, scol, sval = _sub_csr(rp, col, val, rows)
    ref = orc.spmm_f64(srp, scol, sval, B, is_half=half)
    scale = orc.spmm_abs_f64(srp, scol, sval, B, is_half=half)
    if half:
        scale = np.maximum(scale, np.abs(ref))
    err = np.abs(got_rows.astype(np.float64) - ref)
    worst = float((err / (1e-6 + tol * scale)).max())
    assert worst <= 1.0, f"sampled rows: error reaches {worst:.3f} of the bound"
    return worst, float((err <= 1e-6 + tol * np.abs(ref)).mean())


def _reference_kernel(mps, cuda, half, d_rp, d_col, d_B, cost, tpw):
    """C of the reference's own kernel (unit values: degrees == 1), (n+1)-row operands as its indexing needs."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_mergepath_f16.so" if half else "libref_mergepath_f32.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref is not built (needs the reference tree at build time)")
    lib = C.CDLL(path)
    lib.refh_launch.argtypes = [C.c_void_p] * 5 + [C.POINTER(C.c_void_p)] + [C.c_int] * 4
    n, nnz, dim = d_rp.numel() - 1, d_col.numel(), d_B.shape[1]
    p, ipt = mps.chunk_count(n, nnz, cost)
    six = mps.schedule_device(d_rp, p)
    padded = torch.zeros((6, p + 64), dtype=torch.int32, device=cuda)
    padded[:, :p] = six
    deg = torch.ones(n + 1, dtype=torch.int32, device=cuda)
    B1 = torch.zeros((n + 1, dim), dtype=d_B.dtype, device=cuda)
    B1[:n] = d_B
    Cr = torch.zeros((n + 1, dim), dtype=d_B.dtype, device=cuda)
    ptrs = (C.c_void_p * 6)(*[padded[i].data_ptr() for i in range(6)])
    torch.cuda.synchronize()
    rc = lib.refh_launch(Cr.data_ptr(), B1.data_ptr(), d_rp.data_ptr(), d_col.data_ptr(), deg.data_ptr(), ptrs, n, dim, p, tpw)
    torch.cuda.synchronize()
    assert rc == 0, f"reference launch failed with CUDA error {rc}"
    return Cr[:n], ipt


@pytest.fixture(scope="module")
def c3(graphs, cuda):
    rp, col = graphs.rmat_csr(21, 32, seed=0, device=cuda)
    val = graphs.gcn_values(rp, col)
    host = dict(rp=rp.cpu().numpy(), col=col.cpu().numpy(), val=val.cpu().numpy())
    yield dict(rp=rp, col=col, val=val, host=host)


@pytest.mark.parametrize("dim", [64, 16])
def test_c3_whole_product_bit_exact_with_the_cpu_model_and_sampled_rows_in_fp64(mps, orc, graphs, cuda, c3, dim):
    rp, col, val, h = c3["rp"], c3["col"], c3["val"], c3["host"]
    n, nnz = rp.numel() - 1, col.numel()
    B = graphs.dense_uniform(n, dim, seed=1, device=cuda)
    plan = mps.Plan(n, nnz, dim, mps.F32, 16, device=cuda)
    plan.partition(rp)
    out = torch.full((n, dim), float("nan"), dtype=torch.float32, device=cuda)
    plan.spmm(rp, col, val, B, out=out)
    plan.sync_check()
    info = plan.info()
    plan.close()
    assert info["fused_fixup"] == 0 and info["kernels_per_call"] == 2 and info["long_rows"] > 0  # the benchmarked form
    got, hB = out.cpu().numpy(), B.cpu().numpy()
    assert not np.isnan(got).any()
    rows, n_cut = _pick_rows(h["rp"], info["tile_items"], seed=dim)
    assert n_cut >= 1000 and len(rows) >= 4096
    worst, literal = _check_rows(orc, h["rp"], h["col"], h["val"], hB, got[rows], rows, 1e-5)
    assert literal > 0.95
    model = orc.tile_model(h["rp"], h["col"], h["val"], hB, 16, info["chunks_per_tile"], info["chunks_per_unit"], info["long_chain"],
                           unit_items=info["unit_items"])
    same = got.view(np.uint32) == model.view(np.uint32)
    assert same.all(), f"{(~same).sum()} of {same.size} elements differ from the CPU model (first at {np.argwhere(~same)[0]})"


@pytest.mark.parametrize("dim", [64, 16])
def test_c3_unit_values_whole_product_against_the_reference_kernel(mps, graphs, cuda, c3, dim):
    rp, col = c3["rp"], c3["col"]
    n, nnz = rp.numel() - 1, col.numel()
    B = graphs.dense_uniform(n, dim, seed=1, device=cuda)
    ref, ipt = _reference_kernel(mps, cuda, False, rp, col, B, 32, 1)
    scale, _ = _reference_kernel(mps, cuda, False, rp, col, B.abs(), 32, 1)   # sum_k |b_kj|: all terms positive, no cancellation
    got = mps.spmm(rp, col, None, B, cost=16)
    err = (got.double() - ref.double()).abs()
    bound = 1e-6 + 1e-5 * scale.double()
    assert bool((err[1:] <= bound[1:]).all()), f"max error / bound = {float((err[1:] / bound[1:]).max()):.3f}"
    literal = float((err[1:] <= 1e-6 + 1e-5 * ref[1:].double().abs()).double().mean())
    assert literal > 0.95
    # row 0: the reference lacks exactly the first ipt - 1 contributions
    lost = B[col[: ipt - 1].long()].double().sum(0)
    assert torch.allclose(got[0].double() - ref[0].double(), lost, rtol=1e-4, atol=1e-3)


def test_c4_fp16_full_size_against_fp64_rows_an_fp32_product_and_the_reference_fp16_kernel(mps, orc, graphs, cuda, c3):
    rp, col, h = c3["rp"], c3["col"], c3["host"]
    n, nnz, dim = rp.numel() - 1, col.numel(), 128
    val = c3["val"].to(torch.float16)
    B = graphs.dense_normal_f16(n, dim, seed=3, device=cuda)
    plan = mps.Plan(n, nnz, dim, mps.F16, 16, device=cuda)
    plan.partition(rp)
    got = plan.spmm(rp, col, val, B)
    plan.sync_check()
    info = plan.info()
    plan.close()
    rows, _ = _pick_rows(h["rp"], info["tile_items"], seed=7)
    _check_rows(orc, h["rp"], h["col"], val.cpu().numpy(), B.cpu().numpy(), got[torch.from_numpy(rows).to(cuda)].cpu().numpy(), rows, 1e-2, half=True)
    # the same operands multiplied in fp32 storage: within 1e-2 relative of the row's scale everywhere
    v32, B32 = val.float(), B.float()
    c32 = mps.spmm(rp, col, v32, B32, cost=16)
    scale = mps.spmm(rp, col, v32.abs(), B32.abs(), cost=16)
    assert bool(((got.float() - c32).abs() <= 1e-6 + 1e-2 * torch.maximum(scale, c32.abs())).all())
    del c32, scale, v32, B32
    # the reference's fp16 kernel accumulates in fp16 and adds split rows with fp16 atomics: it is only meaningful on
    # short rows, and there the two must agree (unit values; row 0 excluded, see the module docstring)
    ref, _ = _reference_kernel(mps, cuda, True, rp, col, B, 32, 1)
    ours = mps.spmm(rp, col, None, B, cost=16)
    lens = rp[1:] - rp[:-1]
    short = lens <= 48
    short[0] = False
    sc = mps.spmm(rp, col, None, B.float().abs(), cost=16)
    d = (ours.float() - ref.float()).abs()
    assert bool((d[short] <= 1e-6 + 2e-2 * sc[short]).all())
    assert int(short.sum()) > n // 2


def test_c3_large_costs_use_sub_chunk_units_and_stay_bit_exact(mps, orc, graphs, cuda, c3):
    """cost = 5000 at dim 64 and cost = 2000 at dim 16 ask for chunks longer than a tile can stage (the reference's
    command line accepts any cost): a unit becomes a part of a chunk; sampled rows against fp64."""
    rp, col, val, h = c3["rp"], c3["col"], c3["val"], c3["host"]
    n, nnz = rp.numel() - 1, col.numel()
    for dim, cost in ((64, 5000), (16, 2000)):
        B = graphs.dense_uniform(n, dim, seed=2, device=cuda)
        plan = mps.Plan(n, nnz, dim, mps.F32, cost, device=cuda)
        plan.partition(rp)
        got = plan.spmm(rp, col, val, B)
        plan.sync_check()
        info = plan.info()
        plan.close()
        assert info["units_per_chunk"] > 1 and info["shared_bytes_per_block"] <= 48 * 1024
        rows, _ = _pick_rows(h["rp"], info["tile_items"], seed=cost)
        _check_rows(orc, h["rp"], h["col"], h["val"], B.cpu().numpy(), got[torch.from_numpy(rows).to(cuda)].cpu().numpy(), rows, 1e-5)


def test_c5_one_row_slab_of_the_2pow24_graph_against_fp64_rows(mps, orc, graphs, cuda):
    """Configuration 5 as a rank of an 8-GPU job sees it: the last of 8 item-balanced row slabs (many short rows)
    and the first (the hub rows), dim 32, B with all 2^24 rows."""
    rp, col = graphs.rmat_csr(24, 64, seed=0, device=cuda)
    n = rp.numel() - 1
    val = graphs.gcn_values(rp, col)
    dim = 32
    B = graphs.dense_uniform(n, dim, seed=1, device=cuda)
    hB = B.cpu().numpy()
    h_rp = rp.cpu().numpy()
    bounds = mps.slab_bounds(h_rp, 8, "items", 4)
    for g in (0, 7):
        r0, r1 = int(bounds[g]), int(bounds[g + 1])
        k0, k1 = int(h_rp[r0]), int(h_rp[r1])
        s_rp = (rp[r0:r1 + 1] - k0).contiguous()
        s_col, s_val = col[k0:k1].contiguous(), val[k0:k1].contiguous()
        if s_col.data_ptr() % 16:
            s_col, s_val = s_col.clone(), s_val.clone()
        plan = mps.Plan(r1 - r0, k1 - k0, dim, mps.F32, 16, device=cuda)
        plan.partition(s_rp)
        got = plan.spmm(s_rp, s_col, s_val, B)
        plan.sync_check()
        info = plan.info()
        plan.close()
        hs_rp = s_rp.cpu().numpy()
        rows, _ = _pick_rows(hs_rp, info["tile_items"], seed=g, n_long=32)
        worst, _ = _check_rows(orc, hs_rp, s_col.cpu().numpy(), s_val.cpu().numpy(), hB, got[torch.from_numpy(rows).to(cuda)].cpu().numpy(), rows, 1e-5)
        del got, s_rp, s_col, s_val
