// mps_plan_mark_hot_columns: which rows of B should the L2 keep?  (No reference counterpart.)
//
// The gather of B is served by the L2 wherever a row was fetched recently; on a power-law graph a few percent of the
// columns receive most of the non-zeros.  When B is many times larger than the L2 (a rank of a multi-GPU job holds all
// of a B that grows with the job) the default replacement lets rarely used rows push those hub rows out.  This call
// counts how often each column occurs in the plan's col_idx, takes the most frequent columns until their rows of B fill
// the given budget, and keeps a copy of col_idx in the plan with bit 31 set on those columns; mps_spmm then gathers
// marked rows with an L2 evict-last policy and all others with evict-first.
#include <cuda_runtime.h>

#include "mps.h"
#include "mps_internal.h"
#include "mps_plan.h"

using mps::fail;

namespace {

constexpr int kBuckets = 2048;  // occurrences 0..2046 counted exactly, 2047 = that many or more

__global__ void count_columns(const int *__restrict__ col, long long nnz, int *__restrict__ count) {
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x)
        atomicAdd(count + col[k], 1);
}
__global__ void bucket_counts(const int *__restrict__ count, int n_cols, unsigned long long *__restrict__ columns_with, unsigned long long *__restrict__ nnz_with) {
    __shared__ unsigned long long sc[kBuckets], sn[kBuckets];
    for (int i = threadIdx.x; i < kBuckets; i += blockDim.x) sc[i] = sn[i] = 0;
    __syncthreads();
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_cols; c += (long long)gridDim.x * blockDim.x) {
        const int v = count[c];
        const int b = v < kBuckets - 1 ? v : kBuckets - 1;
        atomicAdd(&sc[b], 1ull);
        atomicAdd(&sn[b], (unsigned long long)v);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBuckets; i += blockDim.x) {
        if (sc[i]) atomicAdd(columns_with + i, sc[i]);
        if (sn[i]) atomicAdd(nnz_with + i, sn[i]);
    }
}
__global__ void mark_columns(const int *__restrict__ col, long long nnz, const int *__restrict__ count, int at_least, int *__restrict__ out) {
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < nnz; k += (long long)gridDim.x * blockDim.x) {
        const int c = col[k];
        out[k] = count[c] >= at_least ? (int)((unsigned)c | 0x80000000u) : c;
    }
}

}  // namespace

extern "C" int mps_plan_mark_hot_columns(mps_plan *p, const int32_t *d_col_idx, int32_t n_cols, int64_t budget_bytes, void *stream,
                                         int64_t *hot_columns, int64_t *hot_nnz) {
    if (!p) return fail(MPS_ERR_ARG, "mps_plan_mark_hot_columns: plan is NULL");
    cudaFree(p->d_col_hot);
    p->d_col_hot = nullptr;
    p->hot_columns = p->hot_nnz = 0;
    if (hot_columns) *hot_columns = 0;
    if (hot_nnz) *hot_nnz = 0;
    if (budget_bytes <= 0 || p->nnz == 0) return MPS_OK;  // marking switched off
    if (!d_col_idx || n_cols < 1) return fail(MPS_ERR_ARG, "mps_plan_mark_hot_columns: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const long long row_bytes = (long long)p->dim * (p->dtype == MPS_F16 ? 2 : 4);
    const long long max_rows = budget_bytes / row_bytes;
    int *count = nullptr;
    unsigned long long *hist = nullptr;
    cudaError_t e = cudaMalloc(&count, sizeof(int) * (size_t)n_cols);
    if (e == cudaSuccess) e = cudaMalloc(&hist, sizeof(unsigned long long) * 2 * kBuckets);
    if (e == cudaSuccess) e = cudaMalloc(&p->d_col_hot, sizeof(int) * (size_t)p->nnz);
    if (e == cudaSuccess) e = cudaMemsetAsync(count, 0, sizeof(int) * (size_t)n_cols, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(hist, 0, sizeof(unsigned long long) * 2 * kBuckets, st);
    unsigned long long h[2 * kBuckets];
    if (e == cudaSuccess) {
        count_columns<<<2048, 256, 0, st>>>(d_col_idx, p->nnz, count);
        bucket_counts<<<296, 256, 0, st>>>(count, n_cols, hist, hist + kBuckets);
        e = cudaMemcpyAsync(h, hist, sizeof h, cudaMemcpyDeviceToHost, st);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    int at_least = kBuckets;  // nothing marked
    long long rows = 0, nnz_hot = 0;
    if (e == cudaSuccess) {
        for (int b = kBuckets - 1; b >= 1; --b) {  // most frequent first, whole buckets, while the rows fit the budget
            if (rows + (long long)h[b] > max_rows) break;
            rows += (long long)h[b];
            nnz_hot += (long long)h[kBuckets + b];
            at_least = b;
        }
        mark_columns<<<2048, 256, 0, st>>>(d_col_idx, p->nnz, count, at_least, p->d_col_hot);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    }
    cudaFree(count);
    cudaFree(hist);
    if (e != cudaSuccess || rows == 0) {
        cudaFree(p->d_col_hot);
        p->d_col_hot = nullptr;
        if (e != cudaSuccess) return fail(MPS_ERR_CUDA, "mps_plan_mark_hot_columns: %s", cudaGetErrorString(e));
        return MPS_OK;  // no column is frequent enough to fit: nothing marked, the plain kernel runs
    }
    p->hot_columns = rows;
    p->hot_nnz = nnz_hot;
    if (hot_columns) *hot_columns = rows;
    if (hot_nnz) *hot_nnz = nnz_hot;
    return MPS_OK;
}
