"""Generates tests/golden/reference_partition.npz from the REFERENCE's own host functions.

Run in a container that has the reference tree and the harness built from it
(`make -C oracle REF=<reference tree>` -> oracle/_ref/libref_mergepath_f32.so):

    python tests/golden/make_golden.py

For each case the file holds row_ptr, the chunk count the reference's main() derives for the
cost (src/MergePathSpMM.cu:138-139), the (x, y) coordinates MergePathSearch returns on every
chunk boundary (:280-297, called as generate_mp_sched calls it) and the six arrays of
generate_mp_sched (:300-385).  The GPU box has no reference tree; the tests read the .npz.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402


def main():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_mergepath_f32.so"))
    i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
    lib.refh_chunk_count.argtypes = [C.c_int] * 3
    lib.refh_search_many.argtypes = [i32p, C.c_int, C.c_int, i32p, C.c_int, i32p]
    lib.refh_schedule.argtypes = [i32p, C.c_int, C.c_int, C.c_int, i32p]

    todo = {"c1_rmat": (cases.c1_rmat(), (4, 8, 32)), "c2_batched_60": (cases.c2_batched(60), (8,))}
    for name, g in cases.edge_cases().items():
        todo[name] = (g, (1, 3, 8))
    out = {}
    for name, ((rp, _col), costs) in todo.items():
        rp = np.ascontiguousarray(rp, np.int32)
        n, nnz = len(rp) - 1, int(rp[-1])
        out[f"{name}/row_ptr"] = rp
        for cost in costs:
            p = lib.refh_chunk_count(n, nnz, cost)
            total = n + 1 + nnz
            ipt = (total + p - 1) // p
            diags = np.minimum(np.arange(p + 1, dtype=np.int64) * ipt, total).astype(np.int32)
            xy = np.zeros((p + 1, 2), np.int32)
            lib.refh_search_many(rp, n, nnz, diags, p + 1, xy.reshape(-1))
            six = np.zeros((6, p), np.int32)
            lib.refh_schedule(rp, n, nnz, p, six.reshape(-1))
            out[f"{name}/cost{cost}/n_chunks"] = np.int32(p)
            out[f"{name}/cost{cost}/xy"] = xy
            out[f"{name}/cost{cost}/six"] = six
    path = os.path.join(HERE, "reference_partition.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(todo), "graphs")


if __name__ == "__main__":
    main()
