// Harness around the UNMODIFIED reference translation unit.
//
// TEST INFRASTRUCTURE ONLY.  Built by oracle/Makefile into oracle/_ref/ (which is
// never committed); the reference source is pulled in by #include from where it
// lies (-I<reference>/src), nothing of it is copied into this repository.
//
// REF_TU selects the reference file: "MergePathSpMM.cu" (fp32, default) or
// "MergePathSpMM_fp16.cu" (define REF_HALF as well).  Its main() is renamed and
// never called; the harness drives the reference's own functions:
//   MergePathSearch, generate_mp_sched   (host, src/MergePathSpMM.cu:280-385)
//   spmm_merge_path, spmm_merge_path_64  (device, :388-574)
// with the launch shapes main() uses (:223-264).
#ifndef REF_TU
#define REF_TU "MergePathSpMM.cu"
#endif
#define main mergepath_reference_main_unused
#include REF_TU
#undef main

#ifdef REF_HALF
typedef __half ref_scalar;
#else
typedef float ref_scalar;
#endif

#define REFH_API extern "C" __attribute__((visibility("default")))

// The reference reads its graph from file-scope globals (:26-35).
static void refh_bind_graph(const int *rp, int n_rows, int nnz) {
    NODE_NUM = n_rows;
    NODE_ACT_NUM = n_rows + 1;
    FEATURE_TOTAL = nnz;
    row_ptr = const_cast<int *>(rp);
}

// Chunk count exactly as main() derives it (:138-139).
REFH_API int refh_chunk_count(int n_rows, int nnz, int cost) {
    int n_act = n_rows + 1;
    int p = (n_act + nnz - 1) / cost;
    if (p < 1024) p = 1024;
    return p;
}

// Coordinates of `count` diagonals through the reference's MergePathSearch, called the way
// generate_mp_sched calls it: num_rows = N+1 and an identity array as list B.
REFH_API void refh_search_many(const int *rp, int n_rows, int nnz, const int *diagonals, int count, int *xy) {
    int *identity = new int[nnz > 0 ? nnz : 1];
    for (int i = 0; i < nnz; ++i) identity[i] = i;
    for (int i = 0; i < count; ++i) {
        CoordinateT c = MergePathSearch(diagonals[i], const_cast<int *>(rp), identity, n_rows + 1, nnz);
        xy[2 * i] = c.x;
        xy[2 * i + 1] = c.y;
    }
    delete[] identity;
}

// The six schedule arrays in the reference's return order (:380-383), copied out.
REFH_API void refh_schedule(const int *rp, int n_rows, int nnz, int n_chunks, int *six_by_p) {
    refh_bind_graph(rp, n_rows, nnz);
    std::vector<int *> s = generate_mp_sched(n_chunks);
    for (int a = 0; a < 6; ++a) {
        memcpy(six_by_p + (size_t)a * n_chunks, s[a], sizeof(int) * (size_t)n_chunks);
        delete[] s[a];
    }
}

// One launch of the reference kernel on caller-owned DEVICE buffers.  sched is six device arrays
// of at least n_chunks + pad ints each (the dim<=32 kernel may read up to tpw-1 slots past
// n_chunks, see the grid formula at :230), in the order of refh_schedule.  C must be zeroed by the
// caller (partial rows are added with atomics).  Returns the cudaError_t of launch + sync.
REFH_API int refh_launch(void *C, const void *B, const int *d_rp, const int *d_col, const int *d_deg,
                         int *const *d_sched, int n_rows, int dim, int n_chunks, int tpw) {
    int *fs = d_sched[0], *fsn = d_sched[1], *fe = d_sched[2], *fen = d_sched[3], *rs = d_sched[4], *re = d_sched[5];
    if (dim <= WARP_SIZE) {
        if (tpw > WARP_SIZE / dim) return -1;  // main() exits here (:224-228)
        const int grid = (n_chunks * WARP_SIZE + BLOCK - 1) / (BLOCK * tpw);
        spmm_merge_path<<<grid, BLOCK>>>((ref_scalar *)C, (ref_scalar *)B, (int *)d_rp, (int *)d_col, (int *)d_deg,
                                         fs, fe, fsn, fen, rs, re, n_rows, dim, WARP_SIZE, WARPS_PER_BLOCK,
                                         n_chunks, tpw);
    } else {
        int factor = ceil(dim / WARP_SIZE);
        int n_warps = n_chunks * factor;
        int grid = (n_warps * WARP_SIZE + BLOCK - 1) / BLOCK;
        spmm_merge_path_64<<<grid, BLOCK>>>((ref_scalar *)C, (ref_scalar *)B, (int *)d_rp, (int *)d_col, (int *)d_deg,
                                            fs, fe, fsn, fen, rs, re, n_rows, dim, WARP_SIZE, WARPS_PER_BLOCK,
                                            n_warps, factor);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaDeviceSynchronize();
}

REFH_API int refh_scalar_bytes(void) { return (int)sizeof(ref_scalar); }
