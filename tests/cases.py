"""Small seeded graphs shared by the CPU and GPU tests (row_ptr, col_idx as int32 numpy arrays)."""
import numpy as np

import __graft_entry__ as entry

entry.load_package()
from mergepath_spmm_b200 import graphs  # noqa: E402


def c1_rmat():
    """Benchmark configuration 1: R-MAT, 4,096 nodes, 65,536 sampled edges, seed 0."""
    return graphs.rmat_csr(12, 32, seed=0, n_edges=65536)


def c2_batched(n_components=1100):
    """Benchmark configuration 2: block-diagonal random geometric components."""
    return graphs.batched_geometric_csr(seed=0, n_components=n_components)


def from_lengths(lens, n_cols=None, seed=0):
    lens = np.asarray(lens, dtype=np.int64)
    n = len(lens)
    return graphs.random_csr(n, n_cols or max(n, 1), lens, seed)


def edge_cases():
    """name -> (row_ptr, col_idx): shapes the merge path has to get right."""
    rng = np.random.default_rng(1)
    out = {}
    out["empty_rows_everywhere"] = from_lengths(np.where(rng.random(700) < 0.6, 0, rng.integers(1, 9, 700)), 700, 2)
    out["one_giant_row"] = from_lengths([0, 3, 5000, 1, 0, 2] + [1] * 50, 6000, 3)
    out["giant_first_row"] = from_lengths([4000] + [2] * 300, 4200, 4)
    out["giant_last_row"] = from_lengths([2] * 300 + [4000], 4200, 5)
    out["all_empty"] = from_lengths([0] * 300, 300, 6)
    out["single_row"] = from_lengths([37], 64, 7)
    out["single_empty_row"] = from_lengths([0], 1, 8)
    out["tiny_below_floor"] = from_lengths(rng.integers(0, 4, 40), 40, 9)
    out["dense_rows"] = from_lengths([64] * 64, 64, 10)
    out["leading_and_trailing_empty"] = from_lengths([0] * 100 + list(rng.integers(1, 30, 200)) + [0] * 100, 400, 11)
    out["two_giants_adjacent"] = from_lengths([1] * 10 + [3000, 3500] + [1] * 10, 4000, 12)
    out["above_floor_irregular"] = from_lengths(rng.integers(0, 40, 3000), 3000, 13)
    return out
