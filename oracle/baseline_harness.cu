// Harness around the reference's comparison programs row_wise.cu and nz_splitting.cu, UNMODIFIED.
//
// TEST / MEASUREMENT INFRASTRUCTURE ONLY (reported baselines, never shipped).  Built by
// oracle/Makefile into oracle/_ref/; the reference file is pulled in by #include from where it lies
// with its main() renamed and never called.  BASE_ROW_WISE selects src/row_wise.cu, BASE_NZ_SPLIT
// selects src/nz_splitting.cu (one per shared object: both define the same globals).
#define main baseline_reference_main_unused
#if defined(BASE_ROW_WISE)
#include "row_wise.cu"
#elif defined(BASE_NZ_SPLIT)
#include "nz_splitting.cu"
#else
#error "define BASE_ROW_WISE or BASE_NZ_SPLIT"
#endif
#undef main

#define BASEH_API extern "C" __attribute__((visibility("default")))

#if defined(BASE_ROW_WISE)
// One launch as run_spmm_row_wise issues it (src/row_wise.cu:184-190): `num_warps` blocks of 256
// threads, of which the first num_warps warps each take a contiguous range of rows; dim <= 32 only
// (one column per lane, :222).  Device pointers; returns the cudaError_t of launch + sync.
BASEH_API int baseh_row_wise(float *C, const float *B, const int *rp, const int *col, const int *deg, int n_rows, int dim,
                             int num_warps) {
    if (dim > WARP_SIZE) return -1;
    spmm_row_wise<<<num_warps, BLOCK>>>(C, (float *)B, (int *)rp, (int *)col, (int *)deg, n_rows, dim, WARP_SIZE, num_warps);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaDeviceSynchronize();
}
#endif

#if defined(BASE_NZ_SPLIT)
// Host part (src/nz_splitting.cu:256-316): number of neighbour groups of at most part_size
// non-zeros, then their start offsets (num_parts + 1 ints) and owning rows (num_parts ints).
BASEH_API int baseh_nz_count(const int *rp, int n_rows, int part_size) { return calculate_part_num(part_size, (int *)rp, n_rows); }
BASEH_API void baseh_nz_build(const int *rp, int n_rows, int part_size, int num_parts, int *part_ptr, int *part_to_node) {
    std::vector<int *> p = build_part(part_size, (int *)rp, n_rows);
    memcpy(part_ptr, p[0], sizeof(int) * ((size_t)num_parts + 1));
    memcpy(part_to_node, p[1], sizeof(int) * (size_t)num_parts);
    delete[] p[0]; delete[] p[1]; delete[] p[2];
}
// One launch with main()'s grid and shared-memory formulas (:212-240).  d_part_ptr must hold
// num_parts + 1 ints (the kernels read part_pointers[id + 1], :346,424).  C zeroed by the caller.
BASEH_API int baseh_nz_launch(float *C, const float *B, const int *rp, const int *col, const int *deg, const int *d_part_ptr,
                              const int *d_part_to_node, int n_rows, int dim, int num_parts, int part_size) {
    if (dim > 32) {
        const int grid = (num_parts * WARP_SIZE + BLOCK - 1) / (BLOCK);
        int shared_memory = (part_size * WARPS_PER_BLOCK * sizeof(int)) + (WARPS_PER_BLOCK * dim * sizeof(float));
        spmm_forward_cuda_kernel_64<<<grid, BLOCK, shared_memory>>>(C, (float *)B, (int *)rp, (int *)col, (int *)deg, (int *)d_part_ptr,
                                                                    (int *)d_part_to_node, n_rows, dim, num_parts, part_size, WARP_SIZE,
                                                                    WARPS_PER_BLOCK);
    } else {
        const int ngs = WARP_SIZE / dim;
        const int updated_dim = ngs * dim;
        int shared_memory = ngs * part_size * WARPS_PER_BLOCK * sizeof(int);
        const int grid = (num_parts * WARP_SIZE + BLOCK - 1) / (BLOCK * ngs);
        spmm_forward_cuda_kernel<<<grid, BLOCK, shared_memory>>>(C, (float *)B, (int *)rp, (int *)col, (int *)deg, (int *)d_part_ptr,
                                                                 (int *)d_part_to_node, n_rows, dim, num_parts, part_size, WARP_SIZE,
                                                                 WARPS_PER_BLOCK, updated_dim, ngs);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaDeviceSynchronize();
}
#endif
