"""B200-native merge-path CSR SpMM: host-side mirror of the reference program's interface.

The reference (cag-uconn/MergePath-SpMM) is a command-line program: load `<graph>.csr`, build the
merge-path schedule for `<cost>`, multiply `<repeat>` times (src/MergePathSpMM.cu:110-277).  The
same steps are exposed here as functions over torch CUDA tensors (torch only owns the memory and
the stream), each a thin wrapper of one C-ABI entry point of libmps_b200.so (include/mps.h):

    load_csr / save_csr            the `.csr` text format                (ref :119-173)
    chunk_count                    P and items per chunk for a cost      (ref :138-139, :327-328)
    partition_device               MergePathSearch over all boundaries   (ref :280-297)
    schedule_device                generate_mp_sched's six arrays        (ref :300-385)
    Plan / spmm                    the kernels and their launch loops    (ref :223-264, :388-574)
    spmm_host                      the whole program body on host arrays (ref :187-267)
    slab_bounds                    nnz-balanced row slabs for several GPUs (new)

Nothing here computes on the CPU; without the CUDA library these calls raise.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .capi import F16, F32, MpsError  # noqa: F401

try:
    import torch
except Exception:  # pragma: no cover
    torch = None

__all__ = ["Plan", "MultiGpu", "layout_query", "coo_to_csr", "coo_to_csr_device", "npz_to_csr", "spmm", "spmm_host", "spmm_host_resident_b", "spmm_host_scaled", "gather_probe", "gather_probe_stream", "partition_host", "schedule_host", "load_csr_rect", "spmm_noalloc", "partition_device", "schedule_device", "chunk_count", "load_csr", "save_csr",
           "save_csr_bin", "load_csr_bin", "slab_bounds", "slab_rebase", "algorithmic_bytes", "F32", "F16", "MpsError"]


def _stream_ptr(stream=None):
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


def _dev_ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("expected CUDA tensors (there is no CPU path)")
        if t is not None and not t.is_contiguous():
            raise ValueError("expected contiguous tensors")


def chunk_count(n_rows: int, nnz: int, cost: int) -> tuple[int, int]:
    p, ipt = C.c_int32(), C.c_int32()
    capi.check(capi.lib().mps_chunk_count(n_rows, nnz, cost, C.byref(p), C.byref(ipt)))
    return p.value, ipt.value


def algorithmic_bytes(n_rows: int, nnz: int, dim: int, dtype=F32, has_val: bool = True) -> int:
    return int(capi.lib().mps_algorithmic_bytes(n_rows, nnz, dim, dtype, int(has_val)))


def partition_device(row_ptr, n_chunks: int, stream=None):
    """(n_chunks+1, 2) int32 CUDA tensor of (x, y) in the reference's convention."""
    _need_cuda(row_ptr)
    n_rows = row_ptr.numel() - 1
    nnz = int(row_ptr[-1].item())
    out = torch.empty((n_chunks + 1, 2), dtype=torch.int32, device=row_ptr.device)
    with torch.cuda.device(row_ptr.device):
        capi.check(capi.lib().mps_partition_device(_dev_ptr(row_ptr), n_rows, nnz, n_chunks, _dev_ptr(out), _stream_ptr(stream)))
    return out


def schedule_device(row_ptr, n_chunks: int, stream=None):
    """(6, n_chunks) int32 CUDA tensor in generate_mp_sched's return order."""
    _need_cuda(row_ptr)
    n_rows = row_ptr.numel() - 1
    nnz = int(row_ptr[-1].item())
    out = torch.empty((6, n_chunks), dtype=torch.int32, device=row_ptr.device)
    with torch.cuda.device(row_ptr.device):
        capi.check(capi.lib().mps_schedule_device(_dev_ptr(row_ptr), n_rows, nnz, n_chunks, _dev_ptr(out), _stream_ptr(stream)))
    return out


class Plan:
    """Shape-bound plan: create -> (tune) -> partition(row_ptr) -> spmm(...) any number of times."""

    INFO = ("n_chunks", "items_per_chunk", "chunks_per_tile", "n_tiles", "lanes_per_chunk", "elements_per_lane", "unroll",
            "shared_bytes", "long_rows", "threads_per_warp", "kernels_per_call", "long_chain", "chunks_per_unit", "units_per_tile", "block_threads", "very_long")

    def __init__(self, n_rows: int, nnz: int, dim: int, dtype=F32, cost: int = 8, threads_per_warp: int = 1, device=None):
        self._h = C.c_void_p()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.n_rows, self.nnz, self.dim, self.dtype, self.cost = n_rows, nnz, dim, dtype, cost
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_create(n_rows, nnz, dim, dtype, cost, threads_per_warp, C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            capi.lib().mps_plan_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def tune(self, chunks_per_unit: int = 0, unroll: int = 0, bulk_staging: bool = True, block_threads: int = 0, fused_fixup: int = -1):
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_tune(self._h, chunks_per_unit, unroll, int(bulk_staging), block_threads, fused_fixup))
        return self

    def set_walk(self, warp_per_unit: int = -1):
        """1: a whole warp walks a unit (lane groups combined with shuffles at row ends); 0: a lane group per unit; -1: automatic."""
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_set_walk(self._h, warp_per_unit))
        return self

    def partition(self, row_ptr, stream=None):
        _need_cuda(row_ptr)
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_partition(self._h, _dev_ptr(row_ptr), _stream_ptr(stream)))
        return self

    def spmm(self, row_ptr, col_idx, val, B, out=None, stream=None):
        _need_cuda(row_ptr, col_idx, val, B, out)
        if out is None:
            out = torch.empty((self.n_rows, self.dim), dtype=B.dtype, device=B.device)
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_spmm(self._h, _dev_ptr(row_ptr), _dev_ptr(col_idx), _dev_ptr(val), _dev_ptr(B), _dev_ptr(out),
                                           _stream_ptr(stream)))
        return out

    def spmm_scaled(self, row_ptr, col_idx, row_scale, col_scale, B, out=None, stream=None):
        """C[i] = row_scale[i] * sum_k col_scale[col[k]] * B[col[k]] (fp32): A's values are the outer product of two
        scale vectors, e.g. GCN normalisation, and are never stored."""
        _need_cuda(row_ptr, col_idx, row_scale, col_scale, B, out)
        if out is None:
            out = torch.empty((self.n_rows, self.dim), dtype=B.dtype, device=B.device)
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_spmm_scaled(self._h, _dev_ptr(row_ptr), _dev_ptr(col_idx), _dev_ptr(row_scale), _dev_ptr(col_scale),
                                                  _dev_ptr(B), _dev_ptr(out), _stream_ptr(stream)))
        return out

    def sync_check(self, stream=None):
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_sync_check(self._h, _stream_ptr(stream)))

    def profile(self, enable: bool = True):
        capi.check(capi.lib().mps_plan_profile(self._h, int(enable)))
        return self

    def profile_read(self, stream=None) -> tuple[float, int]:
        """(summed tile-kernel milliseconds, launches) since the last read."""
        ms, n = C.c_double(), C.c_int32()
        with torch.cuda.device(self.device):
            capi.check(capi.lib().mps_plan_profile_read(self._h, _stream_ptr(stream), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def info(self) -> dict:
        arr = (C.c_int64 * 16)()
        capi.check(capi.lib().mps_plan_info(self._h, arr))
        out = dict(zip(self.INFO, [int(v) for v in arr]))
        lay = (C.c_int64 * 12)()
        capi.check(capi.lib().mps_plan_layout(self._h, lay))
        out.update(zip(LAYOUT, [int(v) for v in lay]))
        return out


LAYOUT = ("unit_items", "units_per_tile", "tile_items", "n_tiles", "units_per_chunk", "shared_bytes_per_block", "column_slabs", "fused_fixup", "groups_per_unit")


def layout_query(n_rows: int, nnz: int, dim: int, dtype=F32, cost: int = 8) -> dict:
    """The automatic tile layout for a shape (mps_layout_query): no plan, no CUDA device needed."""
    lay = (C.c_int64 * 12)()
    capi.check(capi.lib().mps_layout_query(n_rows, nnz, dim, dtype, cost, lay))
    return dict(zip(LAYOUT, [int(v) for v in lay]))


def spmm(row_ptr, col_idx, val, B, cost: int = 8, threads_per_warp: int = 1):
    """One-shot C = A @ B on CUDA tensors (plans, partitions, multiplies, checks)."""
    n_rows = row_ptr.numel() - 1
    dtype = F16 if B.dtype == torch.float16 else F32
    plan = Plan(n_rows, col_idx.numel(), B.shape[1], dtype, cost, threads_per_warp, device=B.device)
    try:
        plan.partition(row_ptr)
        out = plan.spmm(row_ptr, col_idx, val, B)
        plan.sync_check()
    finally:
        plan.close()
    return out


def spmm_noalloc(row_ptr, col_idx, val, B, out, cost: int = 8, threads_per_warp: int = 1, stream=None):
    """C = A @ B into the caller's `out` without any device allocation by the library: the scratch
    is a fixed array inside libmps_b200.so (see mps_spmm_noalloc in include/mps.h for who needs this,
    the size limit, and why calls must not overlap).  Blocking; raises MpsError(ERR_UNSUPPORTED)
    when the problem's scratch does not fit."""
    _need_cuda(row_ptr, col_idx, val, B, out)
    dtype = F16 if B.dtype == torch.float16 else F32
    with torch.cuda.device(B.device):
        capi.check(capi.lib().mps_spmm_noalloc(row_ptr.numel() - 1, col_idx.numel(), B.shape[1], dtype, cost, threads_per_warp,
                                               _dev_ptr(row_ptr), _dev_ptr(col_idx), _dev_ptr(val), _dev_ptr(B), _dev_ptr(out),
                                               _stream_ptr(stream)))
    return out


def spmm_host(row_ptr, col_idx, val, B, out=None, cost: int = 8, threads_per_warp: int = 1):
    """The reference program's body on host (numpy or pinned torch CPU) arrays: upload, partition,
    multiply, download.  Returns C as a numpy array (or fills `out`)."""
    def host_ptr(a):
        if a is None:
            return None
        if torch is not None and isinstance(a, torch.Tensor):
            return C.c_void_p(a.data_ptr())
        return a.ctypes.data_as(C.c_void_p)

    n_rows = int(row_ptr.shape[0]) - 1
    nnz = int(col_idx.shape[0])
    dim = int(B.shape[1])
    is_half = str(B.dtype).endswith("float16")
    if out is None:
        out = np.empty((n_rows, dim), np.float16 if is_half else np.float32)
    capi.check(capi.lib().mps_spmm_host(n_rows, int(B.shape[0]), nnz, dim, F16 if is_half else F32, cost, threads_per_warp, host_ptr(row_ptr),
                                        host_ptr(col_idx), host_ptr(val), host_ptr(B), host_ptr(out)))
    return out


def spmm_host_scaled(row_ptr, col_idx, row_scale, col_scale, B, out=None, cost: int = 8, threads_per_warp: int = 1):
    """mps_spmm_host_scaled: C[i] = row_scale[i] * sum_k col_scale[col[k]] * B[col[k]] on host (numpy or pinned torch CPU)
    arrays, fp32; either scale may be None (all ones), not both.  Returns C as a numpy array (or fills `out`)."""
    def host_ptr(a):
        if a is None:
            return None
        if torch is not None and isinstance(a, torch.Tensor):
            return C.c_void_p(a.data_ptr())
        return a.ctypes.data_as(C.c_void_p)

    n_rows, dim = int(row_ptr.shape[0]) - 1, int(B.shape[1])
    if out is None:
        out = np.empty((n_rows, dim), np.float32)
    capi.check(capi.lib().mps_spmm_host_scaled(n_rows, int(B.shape[0]), int(col_idx.shape[0]), dim, cost, threads_per_warp, host_ptr(row_ptr),
                                               host_ptr(col_idx), host_ptr(row_scale), host_ptr(col_scale), host_ptr(B), host_ptr(out)))
    return out


def spmm_host_resident_b(row_ptr, col_idx, val, d_B, out, cost: int = 8, threads_per_warp: int = 1, stream=None):
    """mps_spmm_host with B already on the device (a CUDA tensor, complete once the work queued on `stream` -
    default: torch's current stream - has run): A and `out` are host arrays (numpy, or pinned torch CPU tensors).
    The call of a rank whose share of B arrives over NVLink (see multi.replicate_b)."""
    def host_ptr(a):
        if a is None:
            return None
        if isinstance(a, torch.Tensor):
            return C.c_void_p(a.data_ptr())
        return a.ctypes.data_as(C.c_void_p)

    _need_cuda(d_B)
    is_half = d_B.dtype == torch.float16
    with torch.cuda.device(d_B.device):
        capi.check(capi.lib().mps_spmm_host_resident_b(int(row_ptr.shape[0]) - 1, int(d_B.shape[0]), int(col_idx.shape[0]), int(d_B.shape[1]),
                                                       F16 if is_half else F32, cost, threads_per_warp, host_ptr(row_ptr), host_ptr(col_idx),
                                                       host_ptr(val), _dev_ptr(d_B), _stream_ptr(stream), host_ptr(out)))
    return out


def gather_probe_stream(table, row_bytes: int, index, stream=None) -> float:
    """GB/s at which this GPU delivers the rows of `table` named by `index` (int32 CUDA tensor, e.g. the multiply's col_idx
    with table = B) to a kernel that only fetches them, each group of threads taking a contiguous run in order
    (mps_gather_probe_stream)."""
    _need_cuda(table, index)
    rows = table.numel() * table.element_size() // row_bytes
    sink = torch.empty(1 << 20, dtype=torch.int32, device=table.device)
    ms, nbytes = C.c_float(), C.c_int64()
    with torch.cuda.device(table.device):
        capi.check(capi.lib().mps_gather_probe_stream(_dev_ptr(table), rows, row_bytes, _dev_ptr(index), index.numel(), _dev_ptr(sink), sink.numel() * 4,
                                                      _stream_ptr(stream), C.byref(ms), C.byref(nbytes)))
    return nbytes.value / (ms.value * 1e-3) / 1e9


def gather_probe(table, row_bytes: int, gathers: int, stream=None) -> float:
    """GB/s at which this GPU fetches random whole rows of `row_bytes` from `table` (any CUDA tensor; its bytes are
    the table) with 128-bit loads - mps_gather_probe.  A table inside the L2 gives the L2 -> SM gather rate, one far
    larger than the L2 the random-row rate of HBM."""
    _need_cuda(table)
    rows = table.numel() * table.element_size() // row_bytes
    sink = torch.empty(1 << 20, dtype=torch.int32, device=table.device)
    ms, nbytes = C.c_float(), C.c_int64()
    with torch.cuda.device(table.device):
        capi.check(capi.lib().mps_gather_probe(_dev_ptr(table), rows, row_bytes, gathers, _dev_ptr(sink), sink.numel() * 4, _stream_ptr(stream),
                                               C.byref(ms), C.byref(nbytes)))
    return nbytes.value / (ms.value * 1e-3) / 1e9


def partition_host(row_ptr, n_chunks: int, threads: int = 0):
    """(n_chunks+1, 2) int32 numpy array of (x, y): mps_partition_device's result computed on the host."""
    rp = np.ascontiguousarray(row_ptr, np.int32)
    out = np.empty((n_chunks + 1, 2), np.int32)
    capi.check(capi.lib().mps_partition_host(rp.ctypes.data_as(C.c_void_p), len(rp) - 1, n_chunks, out.ctypes.data_as(C.c_void_p), threads))
    return out


def schedule_host(row_ptr, n_chunks: int, threads: int = 0):
    """(6, n_chunks) int32 numpy array in generate_mp_sched's return order, computed on the host."""
    rp = np.ascontiguousarray(row_ptr, np.int32)
    out = np.empty((6, n_chunks), np.int32)
    capi.check(capi.lib().mps_schedule_host(rp.ctypes.data_as(C.c_void_p), len(rp) - 1, n_chunks, out.ctypes.data_as(C.c_void_p), threads))
    return out


class MultiGpu:
    """Single-process driver over several GPUs of one node (mps_multi_*): A in row slabs of equal
    nnz + 4*rows, B replicated, each device writes its own rows of C; gather_c makes C complete on
    every device with NCCL.  Host (numpy) arrays in, host arrays out."""

    def __init__(self, row_ptr, col_idx, val, n_cols: int, dim: int, dtype=F32, cost: int = 16, threads_per_warp: int = 1,
                 n_gpus: int = 1, devices=None):
        self._keep = [np.ascontiguousarray(row_ptr, np.int32), np.ascontiguousarray(col_idx, np.int32),
                      None if val is None else np.ascontiguousarray(val, np.float16 if dtype == F16 else np.float32)]
        self.n_rows, self.n_cols, self.dim, self.dtype, self.n_gpus = len(self._keep[0]) - 1, n_cols, dim, dtype, n_gpus
        dev = None if devices is None else np.ascontiguousarray(devices, np.int32)
        ptr = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
        self._h = C.c_void_p()
        capi.check(capi.lib().mps_multi_create(n_gpus, ptr(dev), self.n_rows, n_cols, dim, dtype, cost, threads_per_warp,
                                               ptr(self._keep[0]), ptr(self._keep[1]), ptr(self._keep[2]), C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            capi.lib().mps_multi_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def slab(self, g: int) -> dict:
        dev, r0, r1, nz = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        capi.check(capi.lib().mps_multi_slab(self._h, g, C.byref(dev), C.byref(r0), C.byref(r1), C.byref(nz), None))
        return {"device": dev.value, "row0": r0.value, "row1": r1.value, "nnz": nz.value}

    def set_b(self, B):
        B = np.ascontiguousarray(B, np.float16 if self.dtype == F16 else np.float32)
        assert B.shape == (self.n_cols, self.dim)
        capi.check(capi.lib().mps_multi_set_b(self._h, B.ctypes.data_as(C.c_void_p)))
        return self

    def spmm(self, repeat: int = 1, gather_c: bool = False) -> tuple[float, float]:
        """(ms per multiply, ms of the gather), each the maximum over devices."""
        a, b = C.c_float(), C.c_float()
        capi.check(capi.lib().mps_multi_spmm(self._h, repeat, int(gather_c), C.byref(a), C.byref(b)))
        return a.value, b.value

    def get_c(self, from_gpu: int = -1):
        out = np.empty((self.n_rows, self.dim), np.float16 if self.dtype == F16 else np.float32)
        capi.check(capi.lib().mps_multi_get_c(self._h, out.ctypes.data_as(C.c_void_p), from_gpu))
        return out


def load_csr(path: str, threads: int = 0):
    """Reads a `.csr` text file; returns (row_ptr, col_idx) as int32 numpy arrays."""
    csr = capi.Csr()
    capi.check(capi.lib().mps_csr_load(path.encode(), threads, C.byref(csr)))
    try:
        rp = np.ctypeslib.as_array(csr.row_ptr, shape=(csr.n_rows + 1,)).copy()
        col = np.ctypeslib.as_array(csr.col_idx, shape=(csr.nnz,)).copy() if csr.nnz else np.empty(0, np.int32)
    finally:
        capi.lib().mps_csr_free(C.byref(csr))
    return rp, col


def load_csr_rect(path: str, threads: int = 0):
    """As load_csr for a file whose column indices reach beyond its rows; returns (row_ptr, col_idx, n_cols)."""
    csr, n_cols = capi.Csr(), C.c_int32()
    capi.check(capi.lib().mps_csr_load_rect(path.encode(), threads, C.byref(csr), C.byref(n_cols)))
    rp, col = _take_csr(csr)
    return rp, col, n_cols.value


def _take_csr(csr):
    try:
        rp = np.ctypeslib.as_array(csr.row_ptr, shape=(csr.n_rows + 1,)).copy()
        col = np.ctypeslib.as_array(csr.col_idx, shape=(csr.nnz,)).copy() if csr.nnz else np.empty(0, np.int32)
    finally:
        capi.lib().mps_csr_free(C.byref(csr))
    return rp, col


def coo_to_csr(src, dst, n_nodes: int = 0, threads: int = 0):
    """Edge list -> (row_ptr, col_idx): duplicates collapsed, columns sorted per row, as scipy's
    coo_matrix(...).tocsr() leaves them in the reference's converters."""
    s = np.ascontiguousarray(src, np.int64)
    d = np.ascontiguousarray(dst, np.int64)
    csr = capi.Csr()
    capi.check(capi.lib().mps_coo_to_csr(n_nodes, len(s), s.ctypes.data_as(C.c_void_p), d.ctypes.data_as(C.c_void_p), threads, C.byref(csr)))
    return _take_csr(csr)


def coo_to_csr_device(src, dst, n_nodes: int, stream=None):
    """Edge list (int64 CUDA tensors) -> (row_ptr, col_idx) int32 CUDA tensors, same result as coo_to_csr."""
    _need_cuda(src, dst)
    e = src.numel()
    rp = torch.empty(n_nodes + 1, dtype=torch.int32, device=src.device)
    col = torch.empty(max(e, 1), dtype=torch.int32, device=src.device)
    nnz = C.c_int32()
    with torch.cuda.device(src.device):
        capi.check(capi.lib().mps_coo_to_csr_device(n_nodes, e, _dev_ptr(src), _dev_ptr(dst), _dev_ptr(rp), _dev_ptr(col), C.byref(nnz),
                                                    _stream_ptr(stream)))
    return rp, col[: nnz.value]


def csr_transpose_device(row_ptr, col_idx, val, n_cols: int, stream=None):
    """CSR of the transpose of an (n_rows x n_cols) matrix given as int32 CUDA tensors (val: fp32 / fp16 tensor or None).
    Returns (row_ptr_t, col_idx_t, val_t); each transposed row's columns are ascending."""
    _need_cuda(row_ptr, col_idx, val)
    n_rows, nnz = row_ptr.numel() - 1, col_idx.numel()
    dtype = F16 if (val is not None and val.dtype == torch.float16) else F32
    if val is not None and val.dtype not in (torch.float16, torch.float32):
        raise ValueError("values must be float32 or float16")
    rp_t = torch.empty(n_cols + 1, dtype=torch.int32, device=row_ptr.device)
    col_t = torch.empty(nnz, dtype=torch.int32, device=row_ptr.device)
    val_t = None if val is None else torch.empty_like(val)
    with torch.cuda.device(row_ptr.device):
        capi.check(capi.lib().mps_csr_transpose_device(n_rows, n_cols, nnz, dtype, _dev_ptr(row_ptr), _dev_ptr(col_idx), _dev_ptr(val),
                                                       _dev_ptr(rp_t), _dev_ptr(col_t), _dev_ptr(val_t), _stream_ptr(stream)))
    return rp_t, col_t, val_t


def npz_to_csr(path: str, threads: int = 0):
    """(row_ptr, col_idx) from a `.npz` with members src_li / dst_li (scripts/npz_to_csr.py's input)."""
    csr = capi.Csr()
    capi.check(capi.lib().mps_npz_to_csr(path.encode(), threads, C.byref(csr)))
    return _take_csr(csr)


def save_csr(path: str, row_ptr, col_idx) -> None:
    rp = np.ascontiguousarray(row_ptr, np.int32)
    col = np.ascontiguousarray(col_idx, np.int32)
    capi.check(capi.lib().mps_csr_save(path.encode(), len(rp) - 1, rp.ctypes.data_as(C.c_void_p), col.ctypes.data_as(C.c_void_p)))


def save_csr_bin(path: str, row_ptr, col_idx, val=None) -> None:
    rp = np.ascontiguousarray(row_ptr, np.int32)
    col = np.ascontiguousarray(col_idx, np.int32)
    vb, vp = 0, None
    if val is not None:
        val = np.ascontiguousarray(val)
        vb, vp = val.dtype.itemsize, val.ctypes.data_as(C.c_void_p)
    capi.check(capi.lib().mps_csr_save_bin(path.encode(), len(rp) - 1, rp.ctypes.data_as(C.c_void_p), col.ctypes.data_as(C.c_void_p), vp, vb))


def load_csr_bin(path: str):
    csr, val, vb = capi.Csr(), C.c_void_p(), C.c_int()
    capi.check(capi.lib().mps_csr_load_bin(path.encode(), C.byref(csr), C.byref(val), C.byref(vb)))
    libc = C.CDLL(None)
    libc.free.argtypes = [C.c_void_p]
    try:
        rp = np.ctypeslib.as_array(csr.row_ptr, shape=(csr.n_rows + 1,)).copy()
        col = np.ctypeslib.as_array(csr.col_idx, shape=(csr.nnz,)).copy() if csr.nnz else np.empty(0, np.int32)
        v = None
        if val.value and vb.value:
            dt = np.float16 if vb.value == 2 else np.float32
            v = np.frombuffer((C.c_char * (vb.value * csr.nnz)).from_address(val.value), dtype=dt).copy()
    finally:
        capi.lib().mps_csr_free(C.byref(csr))
        if val.value:
            libc.free(val)
    return rp, col, v


def slab_bounds(row_ptr, n_slabs: int, balance: str = "nnz", row_weight: int = 1):
    """Row slab boundaries for n_slabs devices; balance = "nnz" (equal non-zeros) or "items"
    (equal non-zeros + row_weight * rows; row_weight 1 is the merge path's own cost measure)."""
    rp = np.ascontiguousarray(row_ptr, np.int32)
    b = np.empty(n_slabs + 1, np.int32)
    rpp, bp = rp.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p)
    if balance == "items":
        capi.check(capi.lib().mps_slab_bounds_items(rpp, len(rp) - 1, n_slabs, row_weight, bp))
    else:
        capi.check(capi.lib().mps_slab_bounds(rpp, len(rp) - 1, n_slabs, bp))
    return b


def slab_rebase(row_ptr, row0: int, row1: int):
    rp = np.ascontiguousarray(row_ptr, np.int32)
    out = np.empty(row1 - row0 + 1, np.int32)
    capi.check(capi.lib().mps_slab_rebase(rp.ctypes.data_as(C.c_void_p), row0, row1, out.ctypes.data_as(C.c_void_p)))
    return out
