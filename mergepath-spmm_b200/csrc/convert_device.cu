// Edge list -> CSR on the device (no reference counterpart; the reference converts on the host in Python,
// scripts/npz_to_csr.py:13-19).  Same result as mps_coo_to_csr: duplicates collapsed, columns sorted.
//   keys = src * n + dst  ->  radix sort  ->  drop repeats  ->  row_ptr[r] = first key >= r * n
// Sort, select and scan come from CUB (shipped with the CUDA toolkit); this is set-up work before the
// multiply, not part of it.
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
