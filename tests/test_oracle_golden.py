"""The oracle's restatement of the reference's host algorithm against vectors the reference's own
compiled functions produced (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_partition.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _cases(golden):
    names = sorted({k.split("/")[0] for k in golden.files})
    for name in names:
        costs = sorted({int(k.split("/")[1][4:]) for k in golden.files if k.startswith(name + "/cost")})
        for c in costs:
            yield name, c


def test_golden_file_covers_edge_cases(golden):
    names = {k.split("/")[0] for k in golden.files}
    for need in ("c1_rmat", "all_empty", "one_giant_row", "tiny_below_floor", "single_empty_row"):
        assert need in names


def test_chunk_count_matches_reference(golden, orc):
    for name, cost in _cases(golden):
        rp = golden[f"{name}/row_ptr"]
        assert orc.chunk_count(len(rp) - 1, int(rp[-1]), cost) == int(golden[f"{name}/cost{cost}/n_chunks"]), (name, cost)


def test_partition_matches_reference_bit_exact(golden, orc):
    for name, cost in _cases(golden):
        rp = golden[f"{name}/row_ptr"]
        p = int(golden[f"{name}/cost{cost}/n_chunks"])
        assert np.array_equal(orc.partition(rp, p), golden[f"{name}/cost{cost}/xy"]), (name, cost)


def test_schedule_matches_reference_bit_exact(golden, orc):
    for name, cost in _cases(golden):
        rp = golden[f"{name}/row_ptr"]
        p = int(golden[f"{name}/cost{cost}/n_chunks"])
        assert np.array_equal(orc.schedule(rp, p), golden[f"{name}/cost{cost}/six"]), (name, cost)


def test_golden_graphs_are_the_seeded_cases(golden):
    """The fixtures were made from tests/cases.py; the generators must still give the same graphs."""
    import cases
    rp, _ = cases.c1_rmat()
    assert np.array_equal(rp, golden["c1_rmat/row_ptr"])
    for name, (rp, _col) in cases.edge_cases().items():
        assert np.array_equal(rp, golden[f"{name}/row_ptr"]), name
