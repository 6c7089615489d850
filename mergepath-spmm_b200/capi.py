"""ctypes bindings of libmps_b200.so - one Python function per symbol of include/mps.h.

There is no CPU fallback: if the shared library cannot be loaded (and cannot be built with nvcc)
importing this module's `lib()` raises, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

OK = 0
ERR_ARG, ERR_IO, ERR_FORMAT, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM, ERR_DEVICE, ERR_ALIGN, ERR_STATE = range(-1, -10, -1)
F32, F16 = 0, 1

SYMBOLS = [
    "mps_last_error", "mps_version", "mps_csr_load", "mps_csr_load_rect", "mps_csr_free", "mps_csr_save", "mps_csr_save_bin",
    "mps_csr_load_bin", "mps_coo_to_csr", "mps_coo_to_csr_device", "mps_csr_transpose_device", "mps_npz_to_csr", "mps_chunk_count", "mps_partition_device", "mps_schedule_device", "mps_plan_create",
    "mps_plan_destroy", "mps_plan_tune", "mps_plan_partition", "mps_spmm", "mps_spmm_scaled", "mps_plan_sync_check", "mps_plan_info", "mps_plan_set_walk", "mps_plan_layout", "mps_layout_query", "mps_plan_profile", "mps_plan_profile_read",
    "mps_algorithmic_bytes", "mps_gather_probe", "mps_gather_probe_stream", "mps_spmm_host", "mps_spmm_host_resident_b", "mps_spmm_host_scaled", "mps_partition_host", "mps_schedule_host", "mps_host_workspace_release", "mps_spmm_noalloc", "mps_slab_bounds", "mps_slab_bounds_items", "mps_slab_rebase", "mps_multi_create", "mps_multi_destroy", "mps_multi_slab",
    "mps_multi_set_b", "mps_multi_spmm", "mps_multi_get_c",
]


class MpsError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"mps error {code}: {message}")
        self.code = code


class Csr(C.Structure):
    _fields_ = [("n_rows", C.c_int32), ("nnz", C.c_int32),
                ("row_ptr", C.POINTER(C.c_int32)), ("col_idx", C.POINTER(C.c_int32))]


_lib = None


def lib():
    """The loaded library; builds it in-tree first if the .so is absent."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("MPS_B200_LIB") or _build.LIB  # MPS_B200_LIB: use a library built elsewhere
    if not os.path.exists(path):
        path = _build.build_library()
    L = C.CDLL(path)
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    L.mps_last_error.restype = C.c_char_p
    L.mps_version.restype = C.c_char_p
    L.mps_csr_load.argtypes = [C.c_char_p, C.c_int, C.POINTER(Csr)]
    L.mps_csr_load_rect.argtypes = [C.c_char_p, C.c_int, C.POINTER(Csr), C.POINTER(i32)]
    L.mps_csr_free.argtypes = [C.POINTER(Csr)]
    L.mps_csr_free.restype = None
    L.mps_csr_save.argtypes = [C.c_char_p, i32, vp, vp]
    L.mps_csr_save_bin.argtypes = [C.c_char_p, i32, vp, vp, vp, C.c_int]
    L.mps_csr_load_bin.argtypes = [C.c_char_p, C.POINTER(Csr), C.POINTER(vp), C.POINTER(C.c_int)]
    L.mps_coo_to_csr.argtypes = [i32, i64, vp, vp, C.c_int, C.POINTER(Csr)]
    L.mps_coo_to_csr_device.argtypes = [i32, i64, vp, vp, vp, vp, C.POINTER(i32), vp]
    L.mps_csr_transpose_device.argtypes = [i32, i32, i32, C.c_int, vp, vp, vp, vp, vp, vp, vp]
    L.mps_npz_to_csr.argtypes = [C.c_char_p, C.c_int, C.POINTER(Csr)]
    L.mps_chunk_count.argtypes = [i32, i32, i32, C.POINTER(i32), C.POINTER(i32)]
    L.mps_partition_device.argtypes = [vp, i32, i32, i32, vp, vp]
    L.mps_schedule_device.argtypes = [vp, i32, i32, i32, vp, vp]
    L.mps_plan_create.argtypes = [i32, i32, i32, C.c_int, i32, i32, C.POINTER(vp)]
    L.mps_plan_destroy.argtypes = [vp]
    L.mps_plan_destroy.restype = None
    L.mps_plan_tune.argtypes = [vp, i32, i32, i32, i32, i32]
    L.mps_plan_partition.argtypes = [vp, vp, vp]
    L.mps_spmm.argtypes = [vp, vp, vp, vp, vp, vp, vp]
    L.mps_spmm_scaled.argtypes = [vp] * 8
    L.mps_plan_sync_check.argtypes = [vp, vp]
    L.mps_plan_info.argtypes = [vp, C.POINTER(i64)]
    L.mps_plan_layout.argtypes = [vp, C.POINTER(i64)]
    L.mps_plan_set_walk.argtypes = [vp, i32]
    L.mps_layout_query.argtypes = [i32, i32, i32, C.c_int, i32, C.POINTER(i64)]
    L.mps_plan_profile.argtypes = [vp, C.c_int]
    L.mps_plan_profile_read.argtypes = [vp, vp, C.POINTER(C.c_double), C.POINTER(i32)]
    L.mps_algorithmic_bytes.argtypes = [i32, i32, i32, C.c_int, C.c_int]
    L.mps_algorithmic_bytes.restype = i64
    L.mps_spmm_host.argtypes = [i32, i32, i32, i32, C.c_int, i32, i32, vp, vp, vp, vp, vp]
    L.mps_spmm_host_resident_b.argtypes = [i32, i32, i32, i32, C.c_int, i32, i32, vp, vp, vp, vp, vp, vp]
    L.mps_spmm_host_scaled.argtypes = [i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp]
    L.mps_partition_host.argtypes = [vp, i32, i32, vp, C.c_int]
    L.mps_schedule_host.argtypes = [vp, i32, i32, vp, C.c_int]
    L.mps_gather_probe.argtypes = [vp, i64, i32, i64, vp, i64, vp, C.POINTER(C.c_float), C.POINTER(i64)]
    L.mps_gather_probe_stream.argtypes = [vp, i64, i32, vp, i64, vp, i64, vp, C.POINTER(C.c_float), C.POINTER(i64)]
    L.mps_host_workspace_release.restype = None
    L.mps_spmm_noalloc.argtypes = [i32, i32, i32, C.c_int, i32, i32, vp, vp, vp, vp, vp, vp]
    L.mps_slab_bounds.argtypes = [vp, i32, i32, vp]
    L.mps_slab_bounds_items.argtypes = [vp, i32, i32, i32, vp]
    L.mps_slab_rebase.argtypes = [vp, i32, i32, vp]
    L.mps_multi_create.argtypes = [i32, vp, i32, i32, i32, C.c_int, i32, i32, vp, vp, vp, C.POINTER(vp)]
    L.mps_multi_destroy.argtypes = [vp]
    L.mps_multi_destroy.restype = None
    L.mps_multi_slab.argtypes = [vp, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(vp)]
    L.mps_multi_set_b.argtypes = [vp, vp]
    L.mps_multi_spmm.argtypes = [vp, i32, i32, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    L.mps_multi_get_c.argtypes = [vp, vp, i32]
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != OK:
        raise MpsError(rc, lib().mps_last_error().decode("utf-8", "replace"))
