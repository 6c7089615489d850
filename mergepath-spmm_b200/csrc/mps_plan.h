// The plan object behind the opaque mps_plan of the public header.  Internal: shared by the .cu
// translation units of libmps_b200.so only.
#pragma once
#include <cuda_runtime.h>

static const int kProfSlots = 256;  // event pairs kept between two profile reads

struct mps_plan {
    int n_rows, nnz, dim, dtype, cost, tpw_requested, tpw_effective;
    int n_chunks, ipt;
    int vec, gl, unroll, slab_cols, n_col_slabs;
    int block;                          // threads per tile block (64, 128 or 256)
    int nch, cpu, n_tiles, smem_bytes;  // chunks per tile, chunks per unit (whole-chunk layouts; 1 unit = 1 "chunk" otherwise)
    int unit_items, tile_items;         // merge items one lane group walks, merge items per tile (= units per tile x unit_items)
    int sub_chunk;                      // units per reference chunk when a chunk is too long for one unit (1 = whole chunks)
    int bulk;
    int long_chain, very_long, n_long, long_capacity;  // chain lengths (tiles): strand order above long_chain, own kernel above very_long
    int device, sm_count;
    bool user_cpu, user_unroll, user_block, user_fused, user_walk;
    int walk;  // 0: one lane group walks a unit; 1: a whole warp walks a unit, its groups combined with shuffles at row ends
    int fused;  // cross-tile fix-up inside the tile kernel (small problems) or as a kernel of its own
    bool partitioned;
    int2 *d_tile_xy;
    float *d_tcarry, *d_thead;
    int *d_status, *d_long_list, *d_long_count;
    int *d_consumer, *d_need, *d_cnt;  // per tile: who ends my carry's row, contributions awaited, arrivals (x column slabs)
    bool profiling;
    int prof_used;
    cudaEvent_t prof_ev[2 * kProfSlots];
};

namespace mps {
// Fills every shape-derived field (chunking, lanes, column slabs, defaults); no CUDA call.
void plan_init_shape(mps_plan *p, int n_rows, int nnz, int dim, int dtype, int cost, int threads_per_warp);
// Chooses chunks per tile / unroll, computes shared-memory size and the tile count.
int plan_finish_layout(mps_plan *p);
}  // namespace mps
