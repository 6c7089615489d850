// Host versions of the two partition entry points, for callers that want the reference's schedule without a
// device (a loader that pre-computes it, a test on a machine without a GPU).  Same results as
// mps_partition_device / mps_schedule_device, which are what the multiply itself uses.
//
// Replaces MergePathSearch (src/MergePathSpMM.cu:280-297) and generate_mp_sched (:300-385): the reference
// materialises list B = 0..nnz-1 as an array and searches every diagonal on one thread; here list B is
// implicit and the chunk boundaries are searched by all cores.
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

#include "mps.h"
#include "mps_internal.h"

using mps::fail;

namespace {

struct Coord { int32_t x, y; };

// Diagonal `diag` of the merge of row_ptr[0..n_rows] (ties first) with 0..nnz-1: x = row_ptr entries taken.
inline Coord search(long long diag, const int32_t *rp, long long n_list_a, long long nnz) {
    long long lo = std::max<long long>(diag - nnz, 0), hi = std::min(diag, n_list_a);
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)rp[mid] <= diag - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    lo = std::min(lo, n_list_a);
    return {(int32_t)lo, (int32_t)(diag - lo)};
}

template <typename F>
void parallel_for(long long n, int n_threads, F fn) {
    int t = n_threads > 0 ? n_threads : (int)std::thread::hardware_concurrency();
    t = (int)std::max<long long>(1, std::min<long long>(t, n / 4096 + 1));
    if (t == 1) { fn(0, n); return; }
    std::vector<std::thread> th;
    for (int i = 0; i < t; ++i) th.emplace_back(fn, n * i / t, n * (i + 1) / t);
    for (auto &x : th) x.join();
}

int check(const char *who, const int32_t *rp, int32_t n_rows, int32_t n_chunks, const void *out) {
    if (!rp || !out || n_rows < 0 || n_chunks < 1) return fail(MPS_ERR_ARG, "%s: bad argument", who);
    const long long nnz = rp[n_rows];
    if (nnz < 0 || (long long)n_rows + 1 + nnz >= 1ll << 31) return fail(MPS_ERR_UNSUPPORTED, "%s: N+1+nnz does not fit 31 bits", who);
    return MPS_OK;
}

}  // namespace

extern "C" int mps_partition_host(const int32_t *row_ptr, int32_t n_rows, int32_t n_chunks, int32_t *xy, int n_threads) {
    if (int rc = check("mps_partition_host", row_ptr, n_rows, n_chunks, xy)) return rc;
    const long long nnz = row_ptr[n_rows], total = (long long)n_rows + 1 + nnz, ipt = (total + n_chunks - 1) / n_chunks;
    parallel_for((long long)n_chunks + 1, n_threads, [=](long long b, long long e) {
        for (long long t = b; t < e; ++t) {
            const Coord c = search(std::min(ipt * t, total), row_ptr, (long long)n_rows + 1, nnz);
            xy[2 * t] = c.x;
            xy[2 * t + 1] = c.y;
        }
    });
    return MPS_OK;
}

extern "C" int mps_schedule_host(const int32_t *row_ptr, int32_t n_rows, int32_t n_chunks, int32_t *six, int n_threads) {
    if (int rc = check("mps_schedule_host", row_ptr, n_rows, n_chunks, six)) return rc;
    const long long nnz = row_ptr[n_rows], total = (long long)n_rows + 1 + nnz, ipt = (total + n_chunks - 1) / n_chunks;
    const size_t p = (size_t)n_chunks;
    parallel_for(n_chunks, n_threads, [=](long long b, long long e) {
        for (long long t = b; t < e; ++t) {
            const long long d0 = std::min(ipt * t, total), d1 = std::min(d0 + ipt, total);
            const Coord a = search(d0, row_ptr, (long long)n_rows + 1, nnz), z = search(d1, row_ptr, (long long)n_rows + 1, nnz);
            const int32_t first = a.x > 0 ? a.x - 1 : 0, last = z.x - 1;
            // a chunk that starts inside a row owns a "head" (the row's remaining share), one that ends inside a row a
            // "tail"; offset 0 doubles as the reference's "none" mark (:365-369), so a share that starts at non-zero 0 is lost
            int32_t head_at = (row_ptr[first] == a.y || t == 0) ? 0 : a.y;
            int32_t tail_at = (row_ptr[last] == z.y) ? 0 : z.y;
            int32_t head_len = 0, tail_len = 0;
            if (head_at != 0) {
                if (first == last && tail_at != 0) { head_len = tail_at - head_at; tail_at = 0; }
                else head_len = row_ptr[first + 1] - head_at;
            }
            if (tail_at != 0) { tail_len = tail_at - row_ptr[last]; tail_at = row_ptr[last]; }
            six[t] = head_at; six[p + t] = head_len; six[2 * p + t] = tail_at;
            six[3 * p + t] = tail_len; six[4 * p + t] = first; six[5 * p + t] = last;
        }
    });
    return MPS_OK;
}
