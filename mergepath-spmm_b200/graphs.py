"""Seeded synthetic inputs: graphs, values and dense operands.

The reference measures on a suite of public graphs fetched from the network
(README.md:18-23, scripts/fetch_dataset.py:10); these generators stand in for it
with the suite's two shape classes - power-law (R-MAT) and batched small structured
graphs (random geometric components, block diagonal).

Every random draw is a pure function hash(seed, stream, index) on 64-bit integers,
so a graph does not depend on thread count, batch size or on whether it is built
with numpy on the host or with torch on a GPU: both give the same bits.
"""
from __future__ import annotations

import math

import numpy as np

try:  # torch is only needed for device-side generation
    import torch
except Exception:  # pragma: no cover
    torch = None

_M64 = (1 << 64) - 1


def _s64(c: int) -> int:
    """Two's-complement view of an unsigned 64-bit constant."""
    c &= _M64
    return c - (1 << 64) if c >= (1 << 63) else c


_K_STREAM = _s64(0x9E3779B97F4A7C15)
_K_SEED = _s64(0xD6E8FEB86659FD93)
_K_MIX1 = _s64(0xBF58476D1CE4E5B9)
_K_MIX2 = _s64(0x94D049BB133111EB)


def _lsr(z, s: int):
    """Logical shift right on int64 arrays/tensors."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def hash64(index, seed: int, stream: int):
    """splitmix64 finaliser over (index + stream*K1 + seed*K2); int64 in, int64 out (wrapping)."""
    off = _s64(stream * 0x9E3779B97F4A7C15 + seed * 0xD6E8FEB86659FD93)
    if isinstance(index, np.ndarray):
        with np.errstate(over="ignore"):
            z = index + np.int64(off)
            z = (z ^ _lsr(z, 30)) * np.int64(_K_MIX1)
            z = (z ^ _lsr(z, 27)) * np.int64(_K_MIX2)
            return z ^ _lsr(z, 31)
    z = index + off
    z = (z ^ _lsr(z, 30)) * _K_MIX1
    z = (z ^ _lsr(z, 27)) * _K_MIX2
    return z ^ _lsr(z, 31)


def _arange(n: int, device=None, start: int = 0):
    if device is None:
        return np.arange(start, start + n, dtype=np.int64)
    return torch.arange(start, start + n, dtype=torch.int64, device=device)


# --------------------------------------------------------------------------- R-MAT

def rmat_edges(scale: int, n_edges: int, seed: int, abc=(0.57, 0.19, 0.19), device=None, batch: int = 1 << 27):
    """n_edges directed R-MAT edges on 2**scale nodes; `scale` quadrant picks per edge, no noise.
    Returns (u, v) int64."""
    ta = int(abc[0] * 4294967296.0)
    tb = ta + int(abc[1] * 4294967296.0)
    tc = tb + int(abc[2] * 4294967296.0)
    us, vs = [], []
    for e0 in range(0, n_edges, batch):
        m = min(batch, n_edges - e0)
        idx = _arange(m, device, e0)
        u = idx * 0
        v = idx * 0
        for level in range(scale):
            r = _lsr(hash64(idx, seed, level + 1), 32)
            right = ((r >= ta) & (r < tb)) | (r >= tc)   # quadrants b and d set the column bit
            down = r >= tb                               # quadrants c and d set the row bit
            if device is None:
                u = u * 2 + down.astype(np.int64)
                v = v * 2 + right.astype(np.int64)
            else:
                u = u * 2 + down.to(torch.int64)
                v = v * 2 + right.to(torch.int64)
        us.append(u)
        vs.append(v)
    if device is None:
        return np.concatenate(us), np.concatenate(vs)
    return torch.cat(us), torch.cat(vs)


def csr_from_edges(u, v, n_nodes: int, symmetrise: bool = True, self_loops: bool = True):
    """Undirected simple graph in CSR (int32 row_ptr, int32 col_idx, columns sorted per row):
    both directions kept, self-loops and duplicates dropped, then every self-loop added."""
    on_host = isinstance(u, np.ndarray)
    xp = np if on_host else torch
    keep = u != v
    u, v = u[keep], v[keep]
    parts = [u * n_nodes + v]
    if symmetrise:
        parts.append(v * n_nodes + u)
    if self_loops:
        d = _arange(n_nodes, None if on_host else u.device)
        parts.append(d * n_nodes + d)
    keys = xp.concatenate(parts) if on_host else torch.cat(parts)
    del parts, u, v
    keys = xp.unique(keys)
    rows = keys // n_nodes
    cols = keys - rows * n_nodes
    if on_host:
        counts = np.bincount(rows, minlength=n_nodes)
        row_ptr = np.zeros(n_nodes + 1, np.int64)
        np.cumsum(counts, out=row_ptr[1:])
        return row_ptr.astype(np.int32), cols.astype(np.int32)
    counts = torch.bincount(rows, minlength=n_nodes)
    row_ptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr.to(torch.int32), cols.to(torch.int32)


def rmat_csr(scale: int, avg_degree: int, seed: int, device=None, n_edges: int | None = None):
    """R-MAT graph as the benchmark configurations define it: N = 2**scale nodes,
    N*avg_degree/2 sampled directed edges (or n_edges), a/b/c/d = .57/.19/.19/.05,
    symmetrised, deduplicated, self-loops added."""
    n = 1 << scale
    e = n * avg_degree // 2 if n_edges is None else n_edges
    u, v = rmat_edges(scale, e, seed, device=device)
    return csr_from_edges(u, v, n)


# --------------------------------------------------------------------------- batched geometric

def batched_geometric_csr(seed: int, n_components: int = 1100, lo: int = 20, hi: int = 60, mean_degree: float = 4.0):
    """Block-diagonal union of random geometric graphs in the unit square (host only):
    component sizes uniform in [lo, hi], edge iff distance < sqrt(mean_degree/((n-1)*pi)),
    self-loops added."""
    comp = np.arange(n_components, dtype=np.int64)
    sizes = lo + (_lsr(hash64(comp, seed, 1), 11) % (hi - lo + 1))
    starts = np.concatenate([[0], np.cumsum(sizes)])
    n = int(starts[-1])
    node = np.arange(n, dtype=np.int64)
    px = _lsr(hash64(node, seed, 2), 11).astype(np.float64) * 2.0 ** -53
    py = _lsr(hash64(node, seed, 3), 11).astype(np.float64) * 2.0 ** -53
    us, vs = [], []
    for c in range(n_components):
        a, b = int(starts[c]), int(starts[c + 1])
        m = b - a
        r2 = mean_degree / ((m - 1) * math.pi)
        dx = px[a:b, None] - px[None, a:b]
        dy = py[a:b, None] - py[None, a:b]
        i, j = np.nonzero((dx * dx + dy * dy < r2) & ~np.eye(m, dtype=bool))
        us.append(i + a)
        vs.append(j + a)
    u = np.concatenate(us).astype(np.int64)
    v = np.concatenate(vs).astype(np.int64)
    return csr_from_edges(u, v, n, symmetrise=False)


# --------------------------------------------------------------------------- values and dense operands

def gcn_values(row_ptr, col_idx, dtype="f32"):
    """D^-1/2 (A+I) D^-1/2 with d = row length (self-loop included), computed in fp64."""
    on_host = isinstance(row_ptr, np.ndarray)
    if on_host:
        deg = np.diff(row_ptr.astype(np.int64)).astype(np.float64)
        rows = np.repeat(np.arange(len(deg)), np.diff(row_ptr.astype(np.int64)))
        val = 1.0 / np.sqrt(deg[rows] * deg[col_idx.astype(np.int64)])
        return val.astype(np.float16 if dtype == "f16" else np.float32)
    rp = row_ptr.to(torch.int64)
    lens = rp[1:] - rp[:-1]
    deg = lens.to(torch.float64)
    rows = torch.repeat_interleave(torch.arange(len(lens), device=rp.device), lens)
    val = 1.0 / torch.sqrt(deg[rows] * deg[col_idx.to(torch.int64)])
    return val.to(torch.float16 if dtype == "f16" else torch.float32)


def dense_uniform(n_rows: int, dim: int, seed: int, device=None):
    """n_rows x dim fp32, uniform on [-1, 1) with 24-bit resolution (exact in fp32)."""
    idx = _arange(n_rows * dim, device)
    m = _lsr(hash64(idx, seed, 7), 40)
    if device is None:
        return (m.astype(np.float32) * np.float32(2.0 ** -23) - np.float32(1.0)).reshape(n_rows, dim)
    return (m.to(torch.float32) * (2.0 ** -23) - 1.0).reshape(n_rows, dim)


def dense_normal_f16(n_rows: int, dim: int, seed: int, device=None, clip: float = 4.0):
    """n_rows x dim fp16, N(0,1) by Box-Muller on the counter hash, clipped to +-clip."""
    idx = _arange(n_rows * dim, device)
    a = _lsr(hash64(idx, seed, 8), 11)
    b = _lsr(hash64(idx, seed, 9), 11)
    if device is None:
        u1 = (a.astype(np.float64) + 1.0) * 2.0 ** -53
        u2 = b.astype(np.float64) * 2.0 ** -53
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * math.pi * u2)
        return np.clip(z, -clip, clip).astype(np.float16).reshape(n_rows, dim)
    u1 = (a.to(torch.float64) + 1.0) * 2.0 ** -53
    u2 = b.to(torch.float64) * 2.0 ** -53
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
    return z.clamp(-clip, clip).to(torch.float16).reshape(n_rows, dim)


def random_csr(n_rows: int, n_cols: int, density_rows, seed: int):
    """Small irregular CSR for edge-case tests: density_rows[i] = length of row i (host only);
    columns are distinct and sorted inside a row."""
    rng = np.random.default_rng(seed)
    lens = np.asarray(density_rows, dtype=np.int64)
    assert len(lens) == n_rows and (lens <= n_cols).all()
    row_ptr = np.zeros(n_rows + 1, np.int64)
    np.cumsum(lens, out=row_ptr[1:])
    col = np.empty(int(row_ptr[-1]), np.int32)
    for i, m in enumerate(lens):
        if m:
            if m * 4 > n_cols:
                pick = rng.permutation(n_cols)[:m]
            else:
                pick = np.unique(rng.integers(0, n_cols, size=int(m * 2) + 8))
                while len(pick) < m:
                    pick = np.unique(np.concatenate([pick, rng.integers(0, n_cols, size=int(m) + 8)]))
                pick = rng.permutation(pick)[:m]
            col[row_ptr[i]:row_ptr[i + 1]] = np.sort(pick)
    return row_ptr.astype(np.int32), col
