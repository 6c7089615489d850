// Device-side structure conversions.
//
// (1) Edge list -> CSR (no reference counterpart; the reference converts on the host in Python,
// scripts/npz_to_csr.py:13-19).  Same result as mps_coo_to_csr: duplicates collapsed, columns sorted.
//   keys = src * n + dst  ->  radix sort  ->  drop repeats  ->  row_ptr[r] = first key >= r * n
// Sort, select and scan come from CUB (shipped with the CUDA toolkit); this is set-up work before the
// multiply, not part of it.
//
// (2) CSR -> CSR of the transpose (no reference counterpart): what the backward pass of the reference's use
// case multiplies with, dB = A^T dC.  A stable radix sort of the non-zeros by column keeps each transposed
// row's entries in ascending source-row order:
//   perm = argsort(col, stable)  ->  col_t[k'] = row_of(perm[k']),  val_t[k'] = val[perm[k']],
//   row_ptr_t[c] = first k' whose column >= c.
#include "mps.h"

#include <cuda_runtime.h>

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>

#include "mps_internal.h"

using mps::fail;

namespace {

#define CD_CUDA(call)                                                                                \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess) { rc = fail(MPS_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); goto done; } \
    } while (0)

__global__ void make_keys(const long long *__restrict__ src, const long long *__restrict__ dst, long long n_edges, long long n,
                          unsigned long long *__restrict__ keys, int *__restrict__ bad) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_edges) return;
    const long long s = src[i], d = dst[i];
    if (s < 0 || d < 0 || s >= n || d >= n) { atomicExch(bad, 1); keys[i] = 0; return; }
    keys[i] = (unsigned long long)s * (unsigned long long)n + (unsigned long long)d;
}

// row_ptr[r] = number of unique keys below r * n (lower bound), r = 0..n; col[k] = key mod n
__global__ void keys_to_csr(const unsigned long long *__restrict__ keys, const int *__restrict__ n_unique, long long n,
                            int *__restrict__ row_ptr, int *__restrict__ col) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int m = *n_unique;
    if (i <= n) {
        const unsigned long long want = (unsigned long long)i * (unsigned long long)n;
        int lo = 0, hi = m;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (keys[mid] < want) lo = mid + 1;
            else hi = mid;
        }
        row_ptr[i] = lo;
    }
    if (i < m) col[i] = (int)(keys[i] % (unsigned long long)n);
}

}  // namespace

extern "C" int mps_coo_to_csr_device(int32_t n_nodes, int64_t n_edges, const int64_t *d_src, const int64_t *d_dst, int32_t *d_row_ptr,
                                     int32_t *d_col_idx, int32_t *nnz_out, void *stream) {
    if (n_nodes < 1 || n_edges < 0 || !d_row_ptr || !nnz_out || (n_edges > 0 && (!d_src || !d_dst || !d_col_idx)))
        return fail(MPS_ERR_ARG, "mps_coo_to_csr_device: bad argument");
    if ((long long)n_nodes + 1 + n_edges >= 1LL << 31) return fail(MPS_ERR_UNSUPPORTED, "mps_coo_to_csr_device: N+1+edges does not fit 31 bits");
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MPS_OK;
    unsigned long long *keys = nullptr, *sorted = nullptr;
    void *tmp = nullptr;
    int *d_count = nullptr;  // [0] = unique keys, [1] = bad-index flag
    int h_count[2] = {0, 0};
    size_t tmp_sort = 0, tmp_sel = 0;
    const size_t m = (size_t)(n_edges ? n_edges : 1);
    int bits = 1;
    while (bits < 64 && ((unsigned long long)n_nodes * (unsigned long long)n_nodes - 1) >> bits) ++bits;  // key width
    CD_CUDA(cudaMalloc(&keys, 8 * m));
    CD_CUDA(cudaMalloc(&sorted, 8 * m));
    CD_CUDA(cudaMalloc(&d_count, 2 * sizeof(int)));
    CD_CUDA(cudaMemsetAsync(d_count, 0, 2 * sizeof(int), st));
    CD_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, tmp_sort, keys, sorted, (int)n_edges, 0, bits, st));
    CD_CUDA(cub::DeviceSelect::Unique(nullptr, tmp_sel, sorted, keys, d_count, (int)n_edges, st));
    CD_CUDA(cudaMalloc(&tmp, (tmp_sort > tmp_sel ? tmp_sort : tmp_sel) + 16));
    if (n_edges > 0) {
        make_keys<<<(unsigned)((n_edges + 255) / 256), 256, 0, st>>>((const long long *)d_src, (const long long *)d_dst, n_edges, n_nodes, keys, d_count + 1);
        CD_CUDA(cudaGetLastError());
        CD_CUDA(cub::DeviceRadixSort::SortKeys(tmp, tmp_sort, keys, sorted, (int)n_edges, 0, bits, st));
        CD_CUDA(cub::DeviceSelect::Unique(tmp, tmp_sel, sorted, keys, d_count, (int)n_edges, st));  // unique keys back into `keys`
    }
    {
        const long long threads = (long long)n_nodes + 1 > n_edges ? (long long)n_nodes + 1 : n_edges;
        keys_to_csr<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(keys, d_count, n_nodes, d_row_ptr, d_col_idx);
        CD_CUDA(cudaGetLastError());
    }
    CD_CUDA(cudaMemcpyAsync(h_count, d_count, 2 * sizeof(int), cudaMemcpyDeviceToHost, st));
    CD_CUDA(cudaStreamSynchronize(st));
    if (h_count[1]) rc = fail(MPS_ERR_ARG, "mps_coo_to_csr_device: a node index lies outside [0, %d)", n_nodes);
    else *nnz_out = h_count[0];
done:
    cudaFree(keys); cudaFree(sorted); cudaFree(tmp); cudaFree(d_count);
    return rc;
}

namespace {

__global__ void iota_and_check(const int *__restrict__ col, int nnz, int n_cols, int *__restrict__ perm, int *__restrict__ bad) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    perm[i] = i;
    if ((unsigned)col[i] >= (unsigned)n_cols) atomicExch(bad, 1);
}

// k' -> source non-zero k = perm[k']; its row is the last i with row_ptr[i] <= k
template <typename V>
__global__ void transpose_fill(const int *__restrict__ rp, int n_rows, const int *__restrict__ perm, int nnz, const V *__restrict__ val,
                               int *__restrict__ col_t, V *__restrict__ val_t) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const int k = perm[i];
    int lo = 0, hi = n_rows + 1;  // first index with row_ptr > k
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (rp[mid] <= k) lo = mid + 1;
        else hi = mid;
    }
    col_t[i] = lo - 1;
    if (val) val_t[i] = val[k];
}

__global__ void row_ptr_of_sorted(const int *__restrict__ keys, int nnz, int n_cols, int *__restrict__ rp_t) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c > n_cols) return;
    int lo = 0, hi = nnz;  // first k' with keys[k'] >= c
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (keys[mid] < c) lo = mid + 1;
        else hi = mid;
    }
    rp_t[c] = lo;
}

}  // namespace

extern "C" int mps_csr_transpose_device(int32_t n_rows, int32_t n_cols, int32_t nnz, int dtype, const int32_t *d_row_ptr,
                                        const int32_t *d_col_idx, const void *d_val, int32_t *d_row_ptr_t, int32_t *d_col_idx_t,
                                        void *d_val_t, void *stream) {
    if (n_rows < 0 || n_cols < 1 || nnz < 0 || !d_row_ptr || !d_row_ptr_t || (nnz > 0 && (!d_col_idx || !d_col_idx_t)) ||
        ((d_val != nullptr) != (d_val_t != nullptr)))
        return fail(MPS_ERR_ARG, "mps_csr_transpose_device: bad argument");
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "mps_csr_transpose_device: unknown dtype %d", dtype);
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MPS_OK;
    int *perm = nullptr, *perm_sorted = nullptr, *keys_sorted = nullptr, *d_bad = nullptr;
    void *tmp = nullptr;
    size_t tmp_bytes = 0;
    int h_bad = 0;
    const size_t m = (size_t)(nnz ? nnz : 1);
    int bits = 1;
    while (bits < 31 && ((unsigned)(n_cols - 1) >> bits)) ++bits;
    CD_CUDA(cudaMalloc(&perm, 4 * m));
    CD_CUDA(cudaMalloc(&perm_sorted, 4 * m));
    CD_CUDA(cudaMalloc(&keys_sorted, 4 * m));
    CD_CUDA(cudaMalloc(&d_bad, sizeof(int)));
    CD_CUDA(cudaMemsetAsync(d_bad, 0, sizeof(int), st));
    CD_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_col_idx, keys_sorted, perm, perm_sorted, nnz, 0, bits, st));
    CD_CUDA(cudaMalloc(&tmp, tmp_bytes + 16));
    if (nnz > 0) {
        const unsigned blocks = (unsigned)((nnz + 255) / 256);
        iota_and_check<<<blocks, 256, 0, st>>>(d_col_idx, nnz, n_cols, perm, d_bad);
        CD_CUDA(cudaGetLastError());
        CD_CUDA(cudaMemcpyAsync(&h_bad, d_bad, sizeof(int), cudaMemcpyDeviceToHost, st));
        CD_CUDA(cudaStreamSynchronize(st));
        if (h_bad) { rc = fail(MPS_ERR_ARG, "mps_csr_transpose_device: a column index lies outside [0, %d)", n_cols); goto done; }
        CD_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, d_col_idx, keys_sorted, perm, perm_sorted, nnz, 0, bits, st));
        if (dtype == MPS_F16)
            transpose_fill<unsigned short><<<blocks, 256, 0, st>>>(d_row_ptr, n_rows, perm_sorted, nnz, (const unsigned short *)d_val, d_col_idx_t,
                                                                   (unsigned short *)d_val_t);
        else
            transpose_fill<unsigned int><<<blocks, 256, 0, st>>>(d_row_ptr, n_rows, perm_sorted, nnz, (const unsigned int *)d_val, d_col_idx_t,
                                                                 (unsigned int *)d_val_t);
        CD_CUDA(cudaGetLastError());
    }
    row_ptr_of_sorted<<<(unsigned)((n_cols + 1 + 255) / 256), 256, 0, st>>>(keys_sorted, nnz, n_cols, d_row_ptr_t);
    CD_CUDA(cudaGetLastError());
    CD_CUDA(cudaStreamSynchronize(st));
done:
    cudaFree(perm); cudaFree(perm_sorted); cudaFree(keys_sorted); cudaFree(tmp); cudaFree(d_bad);
    return rc;
}
