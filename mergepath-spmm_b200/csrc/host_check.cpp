// Validation of a caller's CSR arrays on host threads, shared by the loaders, the host-buffer call and the
// multi-GPU driver: a non-monotone row_ptr or a column index outside [0, n_cols) must come back as a status
// code, never reach a kernel that gathers rows of B by it.  (The reference checks nothing: its bounds helper
// src/MergePathSpMM.cu:41-52 is never called.)
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <thread>
#include <vector>

#include "mps_internal.h"

namespace mps {

namespace {

int threads_for(long long n, int requested) {
    int t = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
    if (t < 1) t = 1;
    if (t > 32) t = 32;
    const long long by_size = n / (1 << 18) + 1;  // a thread per 256 Ki entries at most
    if (t > by_size) t = (int)by_size;
    return t;
}

// Runs fn(begin, end) -> first bad index or -1 over [0, n) on several threads; returns the smallest bad index.
template <typename F>
long long first_bad(long long n, int requested_threads, F fn) {
    if (n <= 0) return -1;
    const int t = threads_for(n, requested_threads);
    if (t == 1) return fn(0, n);
    std::vector<long long> found((size_t)t, -1);
    std::vector<std::thread> th;
    for (int i = 0; i < t; ++i) {
        const long long b = n * i / t, e = n * (i + 1) / t;
        th.emplace_back([&, i, b, e] { found[(size_t)i] = fn(b, e); });
    }
    for (auto &x : th) x.join();
    for (long long v : found)
        if (v >= 0) return v;
    return -1;
}

}  // namespace

long long first_decreasing_row(const int32_t *rp, long long n_rows, int threads) {
    return first_bad(n_rows, threads, [rp](long long b, long long e) -> long long {
        for (long long i = b; i < e; ++i)
            if (rp[i + 1] < rp[i]) return i;
        return -1;
    });
}

long long first_bad_column(const int32_t *col, long long nnz, int32_t n_cols, int threads) {
    const uint32_t limit = n_cols < 0 ? 0u : (uint32_t)n_cols;  // a negative index is a huge unsigned one
    return first_bad(nnz, threads, [col, limit](long long b, long long e) -> long long {
        const long long kBlock = 1 << 14;
        for (long long i = b; i < e; i += kBlock) {
            const long long stop = std::min(e, i + kBlock);
            uint32_t top = 0;
            for (long long k = i; k < stop; ++k) top = std::max(top, (uint32_t)col[k]);  // vectorises
            if (top >= limit)
                for (long long k = i; k < stop; ++k)
                    if ((uint32_t)col[k] >= limit) return k;
        }
        return -1;
    });
}

int32_t max_column(const int32_t *col, long long nnz, int threads) {
    if (nnz <= 0) return -1;
    const int t = threads_for(nnz, threads);
    std::vector<int32_t> top((size_t)t, -1);
    std::vector<std::thread> th;
    for (int i = 0; i < t; ++i) {
        const long long b = nnz * i / t, e = nnz * (i + 1) / t;
        th.emplace_back([&, i, b, e] { int32_t m = -1; for (long long k = b; k < e; ++k) m = std::max(m, col[k]); top[(size_t)i] = m; });
    }
    for (auto &x : th) x.join();
    return *std::max_element(top.begin(), top.end());
}

int check_csr_host(const char *who, int32_t n_rows, int32_t n_cols, const int32_t *row_ptr, const int32_t *col_idx, int threads) {
    if (row_ptr[0] != 0) return fail(MPS_ERR_ARG, "%s: row_ptr[0] is %d, expected 0", who, row_ptr[0]);
    const long long bad_row = first_decreasing_row(row_ptr, n_rows, threads);
    if (bad_row >= 0) return fail(MPS_ERR_ARG, "%s: row_ptr decreases at row %lld (%d -> %d)", who, bad_row, row_ptr[bad_row], row_ptr[bad_row + 1]);
    if (!col_idx) return MPS_OK;
    const long long bad = first_bad_column(col_idx, row_ptr[n_rows], n_cols, threads);
    if (bad >= 0) return fail(MPS_ERR_ARG, "%s: col_idx[%lld] = %d outside [0, %d)", who, bad, col_idx[bad], n_cols);
    return MPS_OK;
}

}  // namespace mps
