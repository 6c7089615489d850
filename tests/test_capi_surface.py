"""The shared library loads on a machine without a GPU and exports every symbol the header declares;
host-only entry points behave; compute entry points refuse to run without a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mps.h")).read()
    return sorted(set(re.findall(r"MPS_API[^;(]*?\b(mps_\w+)\s*\(", text)))


def test_header_and_binding_list_agree(mps):
    assert _declared() == sorted(mps.capi.SYMBOLS)


def test_every_declared_symbol_is_exported(mps):
    lib = mps.capi.lib()
    for name in _declared():
        assert getattr(lib, name) is not None, name


def test_every_declaration_cites_the_reference_or_says_new():
    text = open(os.path.join(ROOT, "include", "mps.h")).read()
    assert text.count("src/MergePathSpMM.cu:") >= 10


def test_chunk_count_is_the_reference_arithmetic(mps, orc):
    for n, nnz, cost in [(4096, 118000, 8), (10, 5, 8), (0, 0, 1), (2097152, 67000000, 4), (16777216, 1070000000, 32), (1000, 99999, 7)]:
        p, ipt = mps.chunk_count(n, nnz, cost)
        assert p == orc.chunk_count(n, nnz, cost)
        assert ipt == orc.items_per_chunk(n, nnz, p)


def test_bad_arguments_return_codes(mps):
    with pytest.raises(mps.MpsError) as e:
        mps.chunk_count(10, 10, 0)
    assert e.value.code == mps.capi.ERR_ARG
    with pytest.raises(mps.MpsError) as e:
        mps.chunk_count(2**30, 2**30, 8)
    assert e.value.code == mps.capi.ERR_UNSUPPORTED
    assert "31 bits" in str(e.value)


def test_algorithmic_bytes_formula(mps):
    n, nnz, dim = 2097152, 67_000_000, 64
    assert mps.algorithmic_bytes(n, nnz, dim, mps.F32) == 4 * (n + 1) + nnz * 8 + nnz * dim * 4 + n * dim * 4
    assert mps.algorithmic_bytes(n, nnz, dim, mps.F16) == 4 * (n + 1) + nnz * 6 + nnz * dim * 2 + n * dim * 2
    assert mps.algorithmic_bytes(n, nnz, dim, mps.F32, False) == 4 * (n + 1) + nnz * 4 + nnz * dim * 4 + n * dim * 4


def test_no_cpu_fallback_without_a_device(mps):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present; the refusal path is for machines without one")
    h = C.c_void_p()
    rc = mps.capi.lib().mps_plan_create(100, 100, 16, 0, 8, 1, C.byref(h))
    assert rc == mps.capi.ERR_CUDA
    rp = np.zeros(3, np.int32); col = np.zeros(0, np.int32); B = np.zeros((2, 4), np.float32)
    with pytest.raises(mps.MpsError) as e:
        mps.spmm_host(rp, col, None, B)
    assert e.value.code == mps.capi.ERR_CUDA


def test_slab_bounds_match_oracle_and_balance(mps, orc):
    import cases
    rp, _ = cases.c1_rmat()
    nnz = int(rp[-1])
    for g in (1, 2, 3, 4, 8):
        b = mps.slab_bounds(rp, g)
        assert np.array_equal(b, orc.slab_bounds(rp, g))
        assert b[0] == 0 and b[-1] == len(rp) - 1 and (np.diff(b) >= 0).all()
        per = np.diff(rp[b].astype(np.int64))
        assert per.sum() == nnz
        biggest_row = int(np.diff(rp).max())
        assert per.max() <= nnz / g + biggest_row
    n = len(rp) - 1
    for g in (2, 4, 8):
        for w in (1, 4):
            bi = mps.slab_bounds(rp, g, "items", w)
            assert bi[0] == 0 and bi[-1] == n and (np.diff(bi) >= 0).all()
            items = np.diff(rp[bi].astype(np.int64) + w * bi.astype(np.int64))
            assert items.sum() == nnz + w * n and items.max() <= (nnz + w * n) / g + biggest_row + w
        assert np.array_equal(mps.slab_bounds(rp, g, "items", 0), mps.slab_bounds(rp, g))
    sl = mps.slab_rebase(rp, int(b[1]), int(b[2]))
    assert sl[0] == 0 and sl[-1] == rp[b[2]] - rp[b[1]]


def test_header_is_plain_c_and_links_from_a_c_program(mps, tmp_path):
    """The boundary is a C ABI: include/mps.h compiles as C99 and a C program links against the library."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "use_mps.c"
    src.write_text('#include <stdio.h>\n#include "mps.h"\n'
                   'int main(void) {\n'
                   '    int32_t p = 0, ipt = 0;\n'
                   '    if (mps_chunk_count(4096, 100882, 8, &p, &ipt) != MPS_OK) return 1;\n'
                   '    printf("%d %d %s\\n", (int)p, (int)ipt, mps_version());\n'
                   '    return mps_csr_load("/nonexistent.csr", 1, (mps_csr *)0) == MPS_OK;\n'
                   '}\n')
    libdir = os.path.join(root, "mergepath-spmm_b200", "lib")
    exe = tmp_path / "use_mps"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I" + os.path.join(root, "include"), "-o", str(exe), str(src),
                    "-L" + libdir, "-lmps_b200", "-Wl,-rpath," + libdir], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    n_chunks, ipt, _ = r.stdout.split(None, 2)
    assert (int(n_chunks), int(ipt)) == mps.chunk_count(4096, 100882, 8)
