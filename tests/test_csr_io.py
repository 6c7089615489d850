"""The `.csr` text loader/writer and the binary sidecar (host code of the C ABI; no GPU needed).
Grammar facts come from the reference's loader (src/MergePathSpMM.cu:130-173) and writers
(scripts/npz_to_csr.py:21-28)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import cases


def _write(path, text):
    with open(path, "w", newline="") as f:
        f.write(text)


def test_reads_the_writers_format(tmp_path, mps):
    p = str(tmp_path / "g.csr")
    _write(p, "0,2,3,3,5,\n1,2,0,0,3,")  # trailing commas, no final newline
    rp, col = mps.load_csr(p)
    assert rp.tolist() == [0, 2, 3, 3, 5] and col.tolist() == [1, 2, 0, 0, 3]
    assert rp.dtype == np.int32 and col.dtype == np.int32


@pytest.mark.parametrize("text", [
    "0,2,3,3,5\n1,2,0,0,3",        # no trailing commas
    "0,2,3,3,5,\n1,2,0,0,3,\n",    # final newline
    " 0, 2,\t3,3, 5,\n 1,2, 0,0,3,\nignored third line",  # blanks before numbers, extra line
    "0 ,2\t,3,3,5 ,\n1,2 ,0,0,3 ",                        # blanks after numbers (stoi stops at them)
    "+0,2,3,3,5,\n1,2,0,0,3,",
])
def test_accepted_variants(tmp_path, mps, text):
    p = str(tmp_path / "g.csr")
    _write(p, text)
    rp, col = mps.load_csr(p)
    assert rp.tolist() == [0, 2, 3, 3, 5] and col.tolist() == [1, 2, 0, 0, 3]


@pytest.mark.parametrize("text,code", [
    ("0,2,3,3,5,\r\n1,2,0,0,3,", "FORMAT"),   # CRLF: the reference's stoi throws on the "\r" cell
    ("0,2,,3,5,\n1,2,0,0,3,", "FORMAT"),      # empty cell
    ("0,2,x,3,5,\n1,2,0,0,3,", "FORMAT"),
    ("0,2,3,3,5,\n1,2,0,0,", "FORMAT"),       # nnz disagrees with line 2
    ("0,2,1,3,5,\n1,2,0,0,3,", "FORMAT"),     # row_ptr decreases
    ("0,2,3,3,5,\n1,2,0,0,4,", "FORMAT"),     # column out of range
    ("1,2,3,3,5,\n1,2,0,0,3,", "FORMAT"),     # row_ptr[0] != 0
    ("0,99999999999,\n1,", "FORMAT"),         # does not fit int32
    ("", "FORMAT"),
])
def test_rejected_inputs(tmp_path, mps, text, code):
    p = str(tmp_path / "g.csr")
    _write(p, text)
    with pytest.raises(mps.MpsError) as e:
        mps.load_csr(p)
    assert e.value.code == getattr(mps.capi, "ERR_" + code)


def test_missing_file_is_an_error_not_minus_one_rows(tmp_path, mps):
    with pytest.raises(mps.MpsError) as e:
        mps.load_csr(str(tmp_path / "absent.csr"))
    assert e.value.code == mps.capi.ERR_IO


def test_empty_graph_and_no_nonzeros(tmp_path, mps):
    p = str(tmp_path / "g.csr")
    _write(p, "0,0,0,\n")
    rp, col = mps.load_csr(p)
    assert rp.tolist() == [0, 0, 0] and len(col) == 0


def test_round_trip_and_writer_bytes(tmp_path, mps):
    rp, col = cases.c1_rmat()
    p = str(tmp_path / "c1.csr")
    mps.save_csr(p, rp, col)
    raw = open(p, "rb").read()
    assert raw.count(b"\n") == 1 and raw.endswith(b",") and b"\r" not in raw
    first, second = raw.split(b"\n")
    assert first == (",".join(map(str, rp.tolist())) + ",").encode()   # what the reference's writers emit
    assert second == (",".join(map(str, col.tolist())) + ",").encode()
    for threads in (1, 3, 8):
        rp2, col2 = mps.load_csr(p, threads)
        assert np.array_equal(rp, rp2) and np.array_equal(col, col2)


def test_parallel_parse_matches_single_thread_on_a_larger_file(tmp_path, mps, graphs):
    rp, col = graphs.rmat_csr(15, 16, seed=4)   # ~0.5M nnz, several MB of text => many pieces
    p = str(tmp_path / "big.csr")
    mps.save_csr(p, rp, col)
    a = mps.load_csr(p, 1)
    b = mps.load_csr(p, 8)
    assert np.array_equal(a[0], rp) and np.array_equal(a[1], col)
    assert np.array_equal(b[0], rp) and np.array_equal(b[1], col)


def _long_file(cells2, n_rows=40, seed=3):
    """Two long lines: a monotone row_ptr whose last cell is len(cells2), then the given cells of line 2."""
    rng = np.random.default_rng(seed)
    inner = np.sort(rng.integers(0, len(cells2) + 1, n_rows - 1))
    rp = [0] + inner.tolist() + [len(cells2)]
    return ",".join(map(str, rp)) + ",\n" + ",".join(cells2) + ","


def test_cells_of_every_shape_in_long_lines(tmp_path, mps):
    """Long lines go through the eight-bytes-at-a-time path; cells it must hand to the byte-wise loop (blanks, signs,
    nine and ten digits, leading zeros) are mixed with plain ones of one to eight digits."""
    rng = np.random.default_rng(8)
    want, cells = [], []
    for i in range(3000):
        digits = int(rng.integers(1, 11))
        lo, hi = 10 ** (digits - 1) if digits > 1 else 0, min(10 ** digits - 1, 2 ** 31 - 2)
        v = int(rng.integers(lo, hi + 1))
        text = str(v)
        shape = int(rng.integers(0, 8))
        text = {0: " " + text, 1: text + " ", 2: "+" + text, 3: "00" + text, 4: "\t" + text + "\t"}.get(shape, text)
        want.append(v)
        cells.append(text)
    p = str(tmp_path / "mixed.csr")
    _write(p, _long_file(cells))
    for threads in (1, 4):
        rp, col, n_cols = mps.load_csr_rect(p, threads)
        assert col.tolist() == want and n_cols == max(want) + 1 and rp[-1] == len(want)


@pytest.mark.parametrize("bad", ["12a4", "", "1/2", "1:2", "12 3", "99999999999", "2147483648", "-", "1+", "١٢"])
def test_a_bad_cell_in_the_middle_of_a_long_line_is_a_format_error(tmp_path, mps, bad):
    cells = [str(i % 977) for i in range(4000)]
    for at in (0, 1999, 3999):
        mixed = list(cells)
        mixed[at] = bad
        p = str(tmp_path / f"bad{at}.csr")
        _write(p, _long_file(mixed))
        for threads in (1, 4):
            with pytest.raises(mps.MpsError) as e:
                mps.load_csr_rect(p, threads)
            assert e.value.code == mps.capi.ERR_FORMAT, (bad, at)


def _cell_model(text):
    """The loader's grammar for one cell: blanks, an optional sign, digits, blanks; the value must fit int32.
    Returns the value, or None for a cell the loader must refuse."""
    import re
    m = re.fullmatch(r"[ \t]*([+-]?)([0-9]+)[ \t]*", text)
    if not m:
        return None
    v = int(m.group(2)) * (-1 if m.group(1) == "-" else 1)
    return v if -2 ** 31 <= v < 2 ** 31 else None


def test_loader_against_a_model_of_its_grammar_on_random_cells(tmp_path, mps):
    """Property test: lines of random cells - plain, decorated and malformed, of every length - parse to what a
    regular-expression model of the grammar says, or are refused where the model refuses (or a column is negative)."""
    from hypothesis import given, settings, strategies as st, HealthCheck
    plain = st.integers(0, 2 ** 31 - 2).map(str)
    decorated = st.tuples(st.sampled_from(["", " ", "\t", "  "]), st.sampled_from(["", "+", "-"]), st.integers(0, 2 ** 33).map(str),
                          st.sampled_from(["", " ", "\t "])).map("".join)
    zeros = st.tuples(st.sampled_from(["0", "00", "0000000"]), st.integers(0, 99999999).map(str)).map("".join)
    junk = st.text(alphabet="0123456789+- \t./:;abcxyz", min_size=0, max_size=12)
    cell = st.one_of(plain, plain, plain, decorated, zeros, junk)
    path = str(tmp_path / "fuzz.csr")

    @settings(max_examples=150, deadline=None, suppress_health_check=list(HealthCheck))
    @given(st.lists(cell, min_size=1, max_size=40), st.integers(0, 3), st.integers(1, 4))
    def run(odd, where, threads):
        cells = [str(i % 9973) for i in range(300)]
        at = (0, 100, 299, 150)[where]
        cells[at:at] = odd                       # the random cells sit at the start, in the middle or at the end
        want = [_cell_model(c) for c in cells]
        _write(path, _long_file(cells))
        if any(v is None or v < 0 for v in want):
            with pytest.raises(mps.MpsError) as e:
                mps.load_csr_rect(path, threads)
            assert e.value.code == mps.capi.ERR_FORMAT
        else:
            rp, col, n_cols = mps.load_csr_rect(path, threads)
            assert col.tolist() == want

    run()


def test_reads_the_reference_converter_output(tmp_path, mps):
    """The independent writer: scipy's coo->csr plus the cell-by-cell text of the reference's
    scripts/npz_to_csr.py:13-28, restated here (the script itself is not shipped)."""
    import scipy.sparse as sp
    rng = np.random.default_rng(0)
    src, dst = rng.integers(0, 300, 4000), rng.integers(0, 300, 4000)
    m = sp.coo_matrix((np.ones(len(src)), (src, dst)), shape=(300, 300)).tocsr()
    p = str(tmp_path / "conv.csr")
    with open(p, "w") as f:
        for e in m.indptr:
            f.write(str(e) + ",")
        f.write("\n")
        for e in m.indices:
            f.write(str(e) + ",")
    rp, col = mps.load_csr(p)
    assert np.array_equal(rp, m.indptr) and np.array_equal(col, m.indices)


def test_binary_sidecar_round_trip(tmp_path, mps, graphs):
    rp, col = cases.c2_batched(50)
    val = graphs.gcn_values(rp, col)
    p = str(tmp_path / "g.csr.bin")
    mps.save_csr_bin(p, rp, col, val)
    rp2, col2, val2 = mps.load_csr_bin(p)
    assert np.array_equal(rp, rp2) and np.array_equal(col, col2) and np.array_equal(val, val2)
    mps.save_csr_bin(p, rp, col, val.astype(np.float16))
    assert mps.load_csr_bin(p)[2].dtype == np.float16
    mps.save_csr_bin(p, rp, col, None)
    assert mps.load_csr_bin(p)[2] is None
    with open(p, "r+b") as f:
        f.truncate(100)
    with pytest.raises(mps.MpsError):
        mps.load_csr_bin(p)


def test_columns_beyond_the_rows_need_the_rect_loader(tmp_path, mps):
    """scripts/npz_to_csr.py builds its matrix without a shape: a destination above every source gives columns >= N."""
    p = str(tmp_path / "wide.csr")
    _write(p, "0,2,3,\n1,7,0,")
    with pytest.raises(mps.MpsError) as e:
        mps.load_csr(p)
    assert e.value.code == mps.capi.ERR_FORMAT
    rp, col, n_cols = mps.load_csr_rect(p)
    assert rp.tolist() == [0, 2, 3] and col.tolist() == [1, 7, 0] and n_cols == 8
    _write(p, "0,2,3,\n1,-7,0,")
    with pytest.raises(mps.MpsError):
        mps.load_csr_rect(p)
    q = str(tmp_path / "square.csr")
    _write(q, "0,2,3,\n1,0,0,")
    assert mps.load_csr_rect(q)[2] == 2


def test_a_damaged_sidecar_is_rejected_like_a_damaged_text_file(tmp_path, mps):
    rp = np.array([0, 2, 3, 3, 5], np.int32)
    col = np.array([1, 2, 0, 0, 3], np.int32)
    p = str(tmp_path / "g.bin")
    mps.save_csr_bin(p, rp, col)
    raw = bytearray(open(p, "rb").read())
    good = bytes(raw)
    at_col = 32 + 4 * len(rp)
    raw[at_col + 4: at_col + 8] = np.int32(4).tobytes()            # col_idx[1] = 4 with 4 rows
    open(p, "wb").write(raw)
    with pytest.raises(mps.MpsError) as e:
        mps.load_csr_bin(p)
    assert e.value.code == mps.capi.ERR_FORMAT and "col_idx[1]" in str(e.value)
    raw = bytearray(good)
    raw[32 + 8: 32 + 12] = np.int32(1).tobytes()                   # row_ptr = 0,2,1,...
    open(p, "wb").write(raw)
    with pytest.raises(mps.MpsError) as e:
        mps.load_csr_bin(p)
    assert e.value.code == mps.capi.ERR_FORMAT and "row_ptr decreases" in str(e.value)
    open(p, "wb").write(good)
    assert mps.load_csr_bin(p)[0].tolist() == rp.tolist()
