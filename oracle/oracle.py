"""ctypes front end of the CPU oracle (oracle/mergepath_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
bench's CPU-baseline leg, never by the shipped package.

The C file restates the reference's host algorithm (src/MergePathSpMM.cu:
138-139, 280-385) and its kernels' arithmetic (:408-479); see its header for
what is pinned against the reference's own compiled host functions.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "mergepath_oracle.c")
_LIB = os.path.join(_HERE, "_build", "liboracle.so")

_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (AVX2+FMA so fmaf is one instruction)."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    os.makedirs(os.path.dirname(_LIB), exist_ok=True)
    cmd = ["gcc", "-O2", "-std=gnu11", "-fopenmp", "-mavx2", "-mfma", "-ffp-contract=off",
           "-fvisibility=hidden", "-shared", "-fPIC", "-o", _LIB, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        vp = C.c_void_p
        L.orc_chunk_count.restype = C.c_int
        L.orc_chunk_count.argtypes = [C.c_int, C.c_int, C.c_int]
        L.orc_items_per_chunk.restype = C.c_int
        L.orc_items_per_chunk.argtypes = [C.c_int, C.c_int, C.c_int]
        L.orc_merge_path_search.restype = None
        L.orc_merge_path_search.argtypes = [C.c_int64, _i32p, C.c_int, C.c_int,
                                            C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.orc_partition.restype = None
        L.orc_partition.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, _i32p]
        L.orc_schedule.restype = None
        L.orc_schedule.argtypes = [_i32p, C.c_int, C.c_int, C.c_int] + [_i32p] * 6
        L.orc_ref_kernel_emulate_f32.restype = None
        L.orc_ref_kernel_emulate_f32.argtypes = [_i32p, _i32p, _i32p, vp, vp, C.c_int, C.c_int, C.c_int] + [_i32p] * 6
        L.orc_spmm_f64.restype = None
        L.orc_spmm_f64.argtypes = [_i32p, _i32p, vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.orc_spmm_abs_f64.restype = None
        L.orc_spmm_abs_f64.argtypes = [_i32p, _i32p, vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.orc_spmm_f32_omp.restype = C.c_int
        L.orc_spmm_f32_omp.argtypes = [_i32p, _i32p, vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.orc_tile_model.restype = C.c_int
        L.orc_tile_model.argtypes = [_i32p, _i32p, vp, vp, vp] + [C.c_int] * 8 + [C.c_int64, C.c_int]
        L.orc_tile_model_scaled.restype = C.c_int
        L.orc_tile_model_scaled.argtypes = [_i32p, _i32p, vp, vp, vp, vp] + [C.c_int] * 7 + [C.c_int64]
        L.orc_slab_bounds.restype = None
        L.orc_slab_bounds.argtypes = [_i32p, C.c_int, C.c_int, _i32p]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def chunk_count(n_rows: int, nnz: int, cost: int) -> int:
    return lib().orc_chunk_count(n_rows, nnz, cost)


def items_per_chunk(n_rows: int, nnz: int, n_chunks: int) -> int:
    return lib().orc_items_per_chunk(n_rows, nnz, n_chunks)


def merge_path_search(diagonal: int, row_ptr) -> tuple[int, int]:
    rp = _i32(row_ptr)
    x, y = C.c_int(), C.c_int()
    lib().orc_merge_path_search(int(diagonal), rp, len(rp), int(rp[-1]), C.byref(x), C.byref(y))
    return x.value, y.value


def partition(row_ptr, n_chunks: int) -> np.ndarray:
    """(P+1, 2) int32 coordinates (x, y) in the reference's convention."""
    rp = _i32(row_ptr)
    xy = np.empty((n_chunks + 1, 2), np.int32)
    lib().orc_partition(rp, len(rp) - 1, int(rp[-1]), n_chunks, xy.reshape(-1))
    return xy


def schedule(row_ptr, n_chunks: int) -> np.ndarray:
    """(6, P) int32 in the reference's return order:
    feature_start, feature_start_num, feature_end, feature_end_num, start_row, end_row."""
    rp = _i32(row_ptr)
    out = np.zeros((6, n_chunks), np.int32)
    lib().orc_schedule(rp, len(rp) - 1, int(rp[-1]), n_chunks, *[out[i] for i in range(6)])
    return out


def ref_kernel_emulate_f32(row_ptr, col, deg, B, n_chunks: int, sched=None) -> np.ndarray:
    rp, ci, dg = _i32(row_ptr), _i32(col), _i32(deg)
    B = np.ascontiguousarray(B, np.float32)
    n, dim = len(rp) - 1, B.shape[1]
    if sched is None:
        sched = schedule(rp, n_chunks)
    Cm = np.zeros((n + 1, dim), np.float32)
    lib().orc_ref_kernel_emulate_f32(rp, ci, dg, _ptr(B), _ptr(Cm), n, dim, n_chunks,
                                     *[np.ascontiguousarray(sched[i]) for i in range(6)])
    return Cm[:n]


def _store(a, is_half):
    if a is None:
        return None
    return np.ascontiguousarray(a, np.float16 if is_half else np.float32)


def spmm_f64(row_ptr, col, val, B, is_half: bool = False) -> np.ndarray:
    rp, ci = _i32(row_ptr), _i32(col)
    v, Bm = _store(val, is_half), _store(B, is_half)
    n, dim = len(rp) - 1, Bm.shape[1]
    out = np.empty((n, dim), np.float64)
    lib().orc_spmm_f64(rp, ci, _ptr(v), _ptr(Bm), _ptr(out), n, dim, int(is_half))
    return out


def spmm_abs_f64(row_ptr, col, val, B, is_half: bool = False) -> np.ndarray:
    rp, ci = _i32(row_ptr), _i32(col)
    v, Bm = _store(val, is_half), _store(B, is_half)
    n, dim = len(rp) - 1, Bm.shape[1]
    out = np.empty((n, dim), np.float64)
    lib().orc_spmm_abs_f64(rp, ci, _ptr(v), _ptr(Bm), _ptr(out), n, dim, int(is_half))
    return out


def spmm_f32_omp(row_ptr, col, val, B, out=None, threads: int = 0):
    rp, ci = _i32(row_ptr), _i32(col)
    v, Bm = _store(val, False), _store(B, False)
    n, dim = len(rp) - 1, Bm.shape[1]
    if out is None:
        out = np.empty((n, dim), np.float32)
    used = lib().orc_spmm_f32_omp(rp, ci, _ptr(v), _ptr(Bm), _ptr(out), n, dim, threads)
    return out, used


def tile_model(row_ptr, col, val, B, cost: int, nch: int, cpu: int, long_chain: int, is_half: bool = False, unit_items: int = 0, groups: int = 1) -> np.ndarray:
    """nch = chunks per tile, cpu = chunks per unit (nch % cpu == 0); a unit holds cpu * items_per_chunk(cost) merge
    items unless unit_items > 0 names another count (sub-chunk units).  A tile is nch // cpu units.  groups > 1: that
    many lane groups share a unit (a warp walks it) and their partial sums are added in a fixed tree at row ends."""
    rp, ci = _i32(row_ptr), _i32(col)
    v, Bm = _store(val, is_half), _store(B, is_half)
    n, dim = len(rp) - 1, Bm.shape[1]
    out = np.zeros((n, dim), np.float16 if is_half else np.float32)
    rc = lib().orc_tile_model(rp, ci, _ptr(v), _ptr(Bm), _ptr(out), n, int(rp[-1]), dim, int(is_half),
                              cost, nch, cpu, long_chain, unit_items, groups)
    if rc != 0:
        raise ValueError("orc_tile_model: bad arguments")
    return out


def tile_model_scaled(row_ptr, col, row_scale, col_scale, B, cost: int, nch: int, cpu: int, long_chain: int, unit_items: int = 0) -> np.ndarray:
    """Model of mps_spmm_scaled: value(i, j) = row_scale[i] * col_scale[j], row factor applied to the finished row;
    a scale given as None is all ones."""
    rp, ci = _i32(row_ptr), _i32(col)
    rs, cs, Bm = (None if a is None else np.ascontiguousarray(a, np.float32) for a in (row_scale, col_scale, B))
    n, dim = len(rp) - 1, Bm.shape[1]
    out = np.zeros((n, dim), np.float32)
    rc = lib().orc_tile_model_scaled(rp, ci, _ptr(rs), _ptr(cs), _ptr(Bm), _ptr(out), n, int(rp[-1]), dim, cost, nch, cpu, long_chain, unit_items)
    if rc != 0:
        raise ValueError("orc_tile_model_scaled: bad arguments")
    return out


def slab_bounds(row_ptr, n_slabs: int) -> np.ndarray:
    rp = _i32(row_ptr)
    b = np.empty(n_slabs + 1, np.int32)
    lib().orc_slab_bounds(rp, len(rp) - 1, n_slabs, b)
    return b
