// C ABI of the B200 merge-path CSR SpMM library: plans, launches, the host-buffer call.
// Declarations and the reference interface each entry point replaces: include/mps.h.
#include "mps.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <new>
#include <string>

#include "mps_internal.h"
#include "mps_kernels.cuh"
#include "mps_plan.h"

namespace mps {

static thread_local std::string g_error;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

#define MPS_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess) return fail(MPS_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

static int check_shape(int64_t n_rows, int64_t nnz) {
    if (n_rows < 0 || nnz < 0) return fail(MPS_ERR_ARG, "negative size (n_rows=%lld nnz=%lld)", (long long)n_rows, (long long)nnz);
    if (n_rows + 1 + nnz >= (int64_t)1 << 31)
        return fail(MPS_ERR_UNSUPPORTED, "N+1+nnz = %lld does not fit 31 bits", (long long)(n_rows + 1 + nnz));
    return MPS_OK;
}

static void chunking(int n_rows, int nnz, int cost, int *n_chunks, int *ipt) {
    const long long total = (long long)n_rows + 1 + nnz;
    long long p = (total - 1) / cost;  // the reference's (N+1 + nnz - 1) / cost
    if (p < 1024) p = 1024;
    *n_chunks = (int)p;
    *ipt = (int)((total + p - 1) / p);
}

}  // namespace mps

using namespace mps;

extern "C" const char *mps_last_error(void) { return g_error.c_str(); }
extern "C" const char *mps_version(void) { return "mps_b200 0.1 (sm_100a)"; }

extern "C" int mps_chunk_count(int32_t n_rows, int32_t nnz, int32_t cost, int32_t *n_chunks, int32_t *items_per_chunk) {
    if (cost < 1 || !n_chunks || !items_per_chunk) return fail(MPS_ERR_ARG, "mps_chunk_count: cost must be >= 1 and outputs non-NULL");
    if (int rc = check_shape(n_rows, nnz)) return rc;
    chunking(n_rows, nnz, cost, n_chunks, items_per_chunk);
    return MPS_OK;
}

extern "C" int64_t mps_algorithmic_bytes(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int has_val) {
    const int64_t s = dtype == MPS_F16 ? 2 : 4;
    return 4 * ((int64_t)n_rows + 1) + (int64_t)nnz * (4 + (has_val ? s : 0)) + (int64_t)nnz * dim * s + (int64_t)n_rows * dim * s;
}

extern "C" int mps_partition_device(const int32_t *d_row_ptr, int32_t n_rows, int32_t nnz, int32_t n_chunks, int32_t *d_xy,
                                    void *stream) {
    if (!d_row_ptr || !d_xy || n_chunks < 1) return fail(MPS_ERR_ARG, "mps_partition_device: bad argument");
    if (int rc = check_shape(n_rows, nnz)) return rc;
    if (((uintptr_t)d_xy & 7) != 0) return fail(MPS_ERR_ALIGN, "mps_partition_device: d_xy must be 8-byte aligned");
    const long long total = (long long)n_rows + 1 + nnz;
    const long long ipt = (total + n_chunks - 1) / n_chunks;
    const int count = n_chunks + 1;
    partition_kernel<<<(count + 255) / 256, 256, 0, (cudaStream_t)stream>>>(d_row_ptr, n_rows, nnz, ipt, total, count,
                                                                           reinterpret_cast<int2 *>(d_xy));
    MPS_CUDA(cudaGetLastError());
    return MPS_OK;
}

extern "C" int mps_schedule_device(const int32_t *d_row_ptr, int32_t n_rows, int32_t nnz, int32_t n_chunks, int32_t *d_six,
                                   void *stream) {
    if (!d_row_ptr || !d_six || n_chunks < 1) return fail(MPS_ERR_ARG, "mps_schedule_device: bad argument");
    if (int rc = check_shape(n_rows, nnz)) return rc;
    const long long total = (long long)n_rows + 1 + nnz;
    const long long ipt = (total + n_chunks - 1) / n_chunks;
    schedule_kernel<<<(n_chunks + 255) / 256, 256, 0, (cudaStream_t)stream>>>(d_row_ptr, n_rows, nnz, ipt, total, n_chunks, d_six);
    MPS_CUDA(cudaGetLastError());
    return MPS_OK;
}

// ------------------------------------------------------------------------------------- plan

static int pow2_at_least(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

// Shared memory a tile may use.  The resident blocks of an SM (768 threads' worth: the registers allow no more) must fit a
// 196 KiB shared-memory carve-out, each with the 1 KiB the runtime reserves per block: one step more (228 KiB) leaves
// 28 KiB of L1, and the gathers in flight then wait for L1 lines - measured 1.9 ms against 1.2 ms per multiply at dim 64.
static const int kCarveoutBytes = 196 * 1024;
static const int kVeryLongFused = 8192;       // chain length (tiles) above which even the fused form hands a row to a block of fixup_kernel
static const int kFuseMaxTiles = 2048;       // up to here a second launch costs more than the fence the fused fix-up needs
static const int kTilesPerSm = 6;            // smaller tiles rather than idle SMs on small problems
static const int kUnitItems = 272;           // merge items one lane group walks per tile, at most
static const int kTileItemsPerThread = 17;          // merge items per tile the automatic layout aims for
static const int kSmemLimit = 200 * 1024;

static const int kWalkWarpMaxLanes = 0;  // lanes per group up to which a whole warp walks a unit by default (0: never)

static int plan_layout(mps_plan *p) {
    const int elem = p->dtype == MPS_F16 ? 2 : 4;
    if (!p->user_block) p->block = 64;  // small blocks wait least at the three block barriers of a tile; 12 of them fit an SM
    if (p->block < p->gl) p->block = p->gl;
    // a warp per unit exists for full-width lanes, 64-thread blocks and batches of eight; it pays where a warp holds
    // several lane groups (see kWalkWarpMaxLanes)
    const bool can_spread = p->vec == (p->dtype == MPS_F16 ? 8 : 4) && p->gl < 32 && p->block == 64 && (!p->user_unroll || p->unroll == 8);
    // ten gathers in flight per thread: the most that 80 registers hold (12 resident blocks); 12 and 16 lose warps
    if (!p->user_walk) p->walk = (can_spread && p->gl <= kWalkWarpMaxLanes) ? 1 : 0;
    if (!can_spread) p->walk = 0;
    const int groups = p->walk ? 32 / p->gl : 1;          // lane groups that share a unit
    const int gpc = p->block / (p->gl * groups);          // units per tile
    const int kSmemTarget = kCarveoutBytes / (kWarpsPerSm * 32 / p->block) - 1024 - 64, kTileItems = kTileItemsPerThread * p->block;
    if (!p->user_unroll) p->unroll = 10;
    if (p->walk) p->unroll = 8;  // the warp-per-unit kernel exists for batches of eight
    if (p->vec == 1) p->unroll = 4;
    auto smem_of = [&](long long unit) -> long long {  // shared memory of a tile whose units hold `unit` merge items (64-bit: no wrap)
        const long long items = (long long)gpc * unit;
        if (items > (1ll << 24)) return 1ll << 40;
        return TileSmem(gpc, (int)items, p->slab_cols, elem).bytes;
    };
    const long long total = (long long)p->n_rows + 1 + p->nnz;
    long long unit;
    p->sub_chunk = 1;
    if (p->user_cpu) {
        unit = (long long)p->cpu * p->ipt;
    } else {
        // about kTileItems merge items per tile, fewer when the whole problem would otherwise leave SMs without
        // a tile (at least kTilesPerSm tiles per SM), as long as the windows fit the shared-memory target
        if (p->sm_count <= 0) {
            int dev = 0, sms = 0;
            if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) p->sm_count = sms;
            if (p->sm_count <= 0) p->sm_count = 148;
        }
        long long items = total / ((long long)p->sm_count * kTilesPerSm);
        if (items > kTileItems) items = kTileItems;
        if (items > (long long)gpc * groups * kUnitItems) items = (long long)gpc * groups * kUnitItems;  // wide rows: few units, keep each walk short
        int cpu = (int)(items / ((long long)gpc * p->ipt));
        if (cpu < 1) cpu = 1;
        if (cpu > 64) cpu = 64;
        while (cpu > 1 && smem_of((long long)cpu * p->ipt) > kSmemTarget) --cpu;
        p->cpu = cpu;
        unit = (long long)cpu * p->ipt;
        const long long unit_cap = (long long)groups * kUnitItems;  // the same "keep each walk short" as above
        if (cpu == 1 && (smem_of(unit) > kSmemTarget || unit > unit_cap)) {
            // `cost` asks for chunks longer than a unit should be: a unit becomes the k-th part of a chunk (the merge
            // path is cut at multiples of ceil(ipt / k) instead of ipt; the partition search takes any step)
            long long goal = items / gpc;  // what a unit of the automatic layout holds: at most the cap, less on small problems
            if (goal > unit_cap) goal = unit_cap;
            if (goal < 1) goal = 1;
            long long k = (p->ipt + goal - 1) / goal;
            if (k < 2) k = 2;
            while ((p->ipt + k - 1) / k > 1 && smem_of((p->ipt + k - 1) / k) > kSmemTarget) ++k;
            unit = (p->ipt + k - 1) / k;
            p->sub_chunk = (int)k;
        }
    }
    if (smem_of(unit) > kSmemLimit)
        return fail(MPS_ERR_UNSUPPORTED, "a tile of %d units x %lld merge items needs %lld bytes of shared memory (chunks_per_unit %d x %d items per chunk)",
                    gpc, unit, smem_of(unit), p->cpu, p->ipt);
    p->unit_items = (int)unit;
    p->tile_items = (int)(gpc * unit);
    p->nch = gpc * p->cpu;
    p->smem_bytes = (int)smem_of(unit);
    const long long tiles = (total + p->tile_items - 1) / p->tile_items;
    p->n_tiles = (int)(tiles < 1 ? 1 : tiles);
    if (!p->user_fused) p->fused = (long long)p->n_tiles * p->n_col_slabs <= kFuseMaxTiles ? 1 : 0;
    // a tile block sums chains of any realistic length itself; a lone lane group of fixup_kernel should not:
    // there every strand-order chain goes to a whole block of fixup_kernel (512 threads per row)
    p->very_long = p->fused ? kVeryLongFused : p->long_chain;
    return MPS_OK;
}

// Shape-dependent fields of a plan (no CUDA call, no allocation); the caller validated the arguments.
void mps::plan_init_shape(mps_plan *p, int n_rows, int nnz, int dim, int dtype, int cost, int threads_per_warp) {
    memset(p, 0, sizeof *p);
    p->n_rows = n_rows; p->nnz = nnz; p->dim = dim; p->dtype = dtype; p->cost = cost;
    p->tpw_requested = threads_per_warp;
    // the reference exits when tpw > 32/dim (src/MergePathSpMM.cu:224-228) and ignores it for dim > 32
    const int tpw_max = dim <= 32 ? 32 / dim : 1;
    p->tpw_effective = threads_per_warp < 1 ? 1 : (threads_per_warp > tpw_max ? tpw_max : threads_per_warp);
    chunking(n_rows, nnz, cost, &p->n_chunks, &p->ipt);
    const int full_vec = dtype == MPS_F16 ? 8 : 4;
    if (dtype == MPS_F16 && dim % 4 == 0 && dim <= 32 && (dim % 8 != 0 || dim / 8 < 4)) {
        // narrow fp16 rows: four columns per lane (64-bit loads), so that a warp holds at most eight lane groups (dim 16:
        // groups of 4 lanes as for fp32) and widths that are multiples of 4 but not of 8 need no scalar lanes
        p->vec = 4;
        p->gl = pow2_at_least(dim / 4 < 2 ? 2 : dim / 4);
    } else if (dim % full_vec == 0) {
        p->vec = full_vec;
        int lanes = dim / full_vec;
        p->gl = lanes >= 32 ? 32 : pow2_at_least(lanes < 2 ? 2 : lanes);
    } else {
        p->vec = 1;
        p->gl = 32;
    }
    p->slab_cols = p->gl * p->vec;
    p->n_col_slabs = (dim + p->slab_cols - 1) / p->slab_cols;
    p->bulk = 1;
    p->long_chain = 32;
    p->very_long = kVeryLongFused;
}

int mps::plan_finish_layout(mps_plan *p) { return plan_layout(p); }

static void plan_free_scratch(mps_plan *p) {
    cudaFree(p->d_tile_xy); cudaFree(p->d_tcarry); cudaFree(p->d_thead);
    cudaFree(p->d_status); cudaFree(p->d_long_list); cudaFree(p->d_long_count);
    cudaFree(p->d_consumer); cudaFree(p->d_need); cudaFree(p->d_cnt);
    p->d_tile_xy = nullptr; p->d_tcarry = p->d_thead = nullptr;
    p->d_status = p->d_long_list = p->d_long_count = nullptr;
    p->d_consumer = p->d_need = p->d_cnt = nullptr;
}

static int plan_alloc_scratch(mps_plan *p) {
    plan_free_scratch(p);
    p->long_capacity = p->n_tiles / p->long_chain + 2;
    const size_t rows = (size_t)p->n_tiles * p->dim * sizeof(float);
    MPS_CUDA(cudaMalloc(&p->d_tile_xy, sizeof(int2) * ((size_t)p->n_tiles + 1)));
    MPS_CUDA(cudaMalloc(&p->d_tcarry, rows ? rows : 4));
    MPS_CUDA(cudaMalloc(&p->d_thead, rows ? rows : 4));
    MPS_CUDA(cudaMalloc(&p->d_status, sizeof(int)));
    MPS_CUDA(cudaMalloc(&p->d_long_list, sizeof(int) * (size_t)p->long_capacity));
    MPS_CUDA(cudaMalloc(&p->d_long_count, sizeof(int)));
    MPS_CUDA(cudaMalloc(&p->d_consumer, sizeof(int) * (size_t)p->n_tiles));
    MPS_CUDA(cudaMalloc(&p->d_need, sizeof(int) * (size_t)p->n_tiles));
    MPS_CUDA(cudaMalloc(&p->d_cnt, sizeof(int) * (size_t)p->n_tiles * p->n_col_slabs));
    MPS_CUDA(cudaMemset(p->d_status, 0, sizeof(int)));
    return MPS_OK;
}

extern "C" int mps_plan_create(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost, int32_t threads_per_warp,
                               mps_plan **out) {
    if (!out) return fail(MPS_ERR_ARG, "mps_plan_create: out is NULL");
    *out = nullptr;
    if (dim < 1 || cost < 1) return fail(MPS_ERR_ARG, "mps_plan_create: dim and cost must be >= 1 (dim=%d cost=%d)", dim, cost);
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "mps_plan_create: unknown dtype %d", dtype);
    if (int rc = check_shape(n_rows, nnz)) return rc;
    mps_plan *p = new (std::nothrow) mps_plan();
    if (!p) return fail(MPS_ERR_NOMEM, "mps_plan_create: out of host memory");
    plan_init_shape(p, n_rows, nnz, dim, dtype, cost, threads_per_warp);
    if (cudaError_t e = cudaGetDevice(&p->device)) {
        delete p;
        return fail(MPS_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    }
    int rc = plan_layout(p);
    if (rc == MPS_OK) rc = plan_alloc_scratch(p);
    if (rc != MPS_OK) { plan_free_scratch(p); delete p; return rc; }
    *out = p;
    return MPS_OK;
}

extern "C" void mps_plan_destroy(mps_plan *plan) {
    if (!plan) return;
    for (cudaEvent_t e : plan->prof_ev)
        if (e) cudaEventDestroy(e);
    plan_free_scratch(plan);
    delete plan;
}

extern "C" int mps_plan_tune(mps_plan *p, int32_t chunks_per_unit, int32_t unroll, int32_t bulk_staging, int32_t block_threads,
                             int32_t fused_fixup) {
    if (!p) return fail(MPS_ERR_ARG, "mps_plan_tune: plan is NULL");
    if (unroll != 0 && unroll != 4 && unroll != 8 && unroll != 10) return fail(MPS_ERR_ARG, "mps_plan_tune: unroll must be 0, 4, 8 or 10");
    if (chunks_per_unit < 0 || chunks_per_unit > 4096) return fail(MPS_ERR_ARG, "mps_plan_tune: chunks_per_unit out of range");
    if (block_threads != 0 && block_threads != 64 && block_threads != 128 && block_threads != 256)
        return fail(MPS_ERR_ARG, "mps_plan_tune: block_threads must be 0, 64, 128 or 256");
    if (block_threads != 0 && block_threads < p->gl) return fail(MPS_ERR_ARG, "mps_plan_tune: a block must hold at least one group of %d lanes", p->gl);
    if (fused_fixup < -1 || fused_fixup > 1) return fail(MPS_ERR_ARG, "mps_plan_tune: fused_fixup must be -1 (automatic), 0 or 1");
    p->user_fused = fused_fixup >= 0;
    if (p->user_fused) p->fused = fused_fixup;
    p->user_block = block_threads != 0;
    if (p->user_block) p->block = block_threads;
    const int old_tiles = p->n_tiles;
    p->user_cpu = chunks_per_unit > 0;
    if (p->user_cpu) p->cpu = chunks_per_unit;
    p->user_unroll = unroll != 0;
    if (p->user_unroll) p->unroll = unroll;
    p->bulk = bulk_staging ? 1 : 0;
    if (int rc = plan_layout(p)) return rc;
    p->partitioned = false;
    if (p->n_tiles != old_tiles) return plan_alloc_scratch(p);
    return MPS_OK;
}

extern "C" int mps_plan_set_walk(mps_plan *p, int32_t warp_per_unit) {
    if (!p) return fail(MPS_ERR_ARG, "mps_plan_set_walk: plan is NULL");
    if (warp_per_unit < -1 || warp_per_unit > 1) return fail(MPS_ERR_ARG, "mps_plan_set_walk: -1 (automatic), 0 or 1");
    const int old_tiles = p->n_tiles;
    p->user_walk = warp_per_unit >= 0;
    if (p->user_walk) p->walk = warp_per_unit;
    if (int rc = plan_layout(p)) return rc;
    p->partitioned = false;
    if (p->n_tiles != old_tiles) return plan_alloc_scratch(p);
    return MPS_OK;
}

extern "C" int mps_plan_partition(mps_plan *p, const int32_t *d_row_ptr, void *stream) {
    if (!p || !d_row_ptr) return fail(MPS_ERR_ARG, "mps_plan_partition: NULL argument");
    cudaStream_t st = (cudaStream_t)stream;
    const long long total = (long long)p->n_rows + 1 + p->nnz;
    const int count = p->n_tiles + 1;
    partition_kernel<<<(count + 255) / 256, 256, 0, st>>>(d_row_ptr, p->n_rows, p->nnz, (long long)p->tile_items, total, count,
                                                         p->d_tile_xy);
    MPS_CUDA(cudaGetLastError());
    MPS_CUDA(cudaMemsetAsync(p->d_long_count, 0, sizeof(int), st));
    MPS_CUDA(cudaMemsetAsync(p->d_cnt, 0, sizeof(int) * (size_t)p->n_tiles * p->n_col_slabs, st));
    fixup_plan_kernel<<<(p->n_tiles + 255) / 256, 256, 0, st>>>(p->d_tile_xy, d_row_ptr, p->n_tiles, p->very_long, p->d_consumer, p->d_need,
                                                                p->d_long_list, p->d_long_count, p->long_capacity);
    MPS_CUDA(cudaGetLastError());
    int n_long = 0;
    MPS_CUDA(cudaMemcpyAsync(&n_long, p->d_long_count, sizeof(int), cudaMemcpyDeviceToHost, st));
    MPS_CUDA(cudaStreamSynchronize(st));
    if (n_long > p->long_capacity) return fail(MPS_ERR_STATE, "mps_plan_partition: %d long rows exceed the list capacity %d", n_long, p->long_capacity);
    p->n_long = n_long;
    p->partitioned = true;
    return MPS_OK;
}

namespace mps {
// one multiply on a partitioned plan, defined in mps_spmm_f32.cu / mps_spmm_f32_scaled.cu / mps_spmm_f16.cu
int spmm_f32(mps_plan *p, const TileParams &tp, cudaStream_t st);
int spmm_f32_scaled(mps_plan *p, const TileParams &tp, cudaStream_t st);
int spmm_f16(mps_plan *p, const TileParams &tp, cudaStream_t st);
}  // namespace mps

static int spmm_launch(mps_plan *p, const int32_t *d_row_ptr, const int32_t *d_col_idx, const void *d_val, const float *d_row_scale,
                       const float *d_col_scale, const void *d_B, void *d_C, void *stream) {
    if (!p || !d_row_ptr || !d_B || !d_C || (!d_col_idx && p->nnz > 0)) return fail(MPS_ERR_ARG, "mps_spmm: NULL argument");
    if (!p->partitioned) return fail(MPS_ERR_STATE, "mps_spmm: call mps_plan_partition first");
    const uintptr_t elem = p->dtype == MPS_F16 ? 2 : 4;
    const uintptr_t need = p->vec > 1 ? (uintptr_t)p->vec * elem : elem;  // one lane's load: 16 bytes, 8 for narrow fp16 rows
    if (((uintptr_t)d_B % need) || ((uintptr_t)d_C % need))
        return fail(MPS_ERR_ALIGN, "mps_spmm: B and C must be %d-byte aligned for dim=%d", (int)need, p->dim);
    if (((uintptr_t)d_row_ptr % 4) || ((uintptr_t)d_col_idx % 4) || ((uintptr_t)d_val % elem))
        return fail(MPS_ERR_ALIGN, "mps_spmm: row_ptr/col_idx/val not aligned to their element size");
    TileParams tp;
    tp.rp = d_row_ptr; tp.col = d_col_idx; tp.val = d_val; tp.B = d_B; tp.C = d_C;
    tp.row_scale = d_row_scale; tp.col_scale = d_col_scale;
    tp.tile_xy = p->d_tile_xy; tp.tcarry = p->d_tcarry; tp.thead = p->d_thead; tp.status = p->d_status;
    tp.consumer = p->d_consumer; tp.need = p->d_need; tp.cnt = p->d_cnt; tp.long_chain = p->long_chain; tp.very_long = p->very_long; tp.fused = p->fused;
    tp.total = (long long)p->n_rows + 1 + p->nnz;
    tp.n_rows = p->n_rows; tp.nnz = p->nnz; tp.dim = p->dim;
    tp.unit_items = p->unit_items; tp.tile_items = p->tile_items; tp.n_tiles = p->n_tiles;
    // a product without stored values (unit values, or the scaled form) stages no value window: a third less shared memory
    tp.smem_bytes = d_val ? p->smem_bytes : TileSmem(p->tile_items / p->unit_items, p->tile_items, p->slab_cols, 0).bytes;
    const bool aligned16 = !((uintptr_t)d_row_ptr % 16) && !((uintptr_t)d_col_idx % 16) && !((uintptr_t)d_val % 16);
    tp.bulk = (p->bulk && aligned16) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (p->dtype == MPS_F16) return spmm_f16(p, tp, st);
    return (d_row_scale || d_col_scale) ? spmm_f32_scaled(p, tp, st) : spmm_f32(p, tp, st);
}

extern "C" int mps_spmm(mps_plan *p, const int32_t *d_row_ptr, const int32_t *d_col_idx, const void *d_val, const void *d_B,
                        void *d_C, void *stream) {
    return spmm_launch(p, d_row_ptr, d_col_idx, d_val, nullptr, nullptr, d_B, d_C, stream);
}

extern "C" int mps_spmm_scaled(mps_plan *p, const int32_t *d_row_ptr, const int32_t *d_col_idx, const float *d_row_scale,
                               const float *d_col_scale, const void *d_B, void *d_C, void *stream) {
    if (!d_row_scale && !d_col_scale) return fail(MPS_ERR_ARG, "mps_spmm_scaled: both scale arrays are NULL (use mps_spmm)");
    if (p && p->dtype != MPS_F32) return fail(MPS_ERR_UNSUPPORTED, "mps_spmm_scaled: fp32 plans only");
    if (((uintptr_t)d_row_scale % 4) || ((uintptr_t)d_col_scale % 4)) return fail(MPS_ERR_ALIGN, "mps_spmm_scaled: scale arrays must be 4-byte aligned");
    return spmm_launch(p, d_row_ptr, d_col_idx, nullptr, d_row_scale, d_col_scale, d_B, d_C, stream);
}

extern "C" int mps_plan_sync_check(mps_plan *p, void *stream) {
    if (!p) return fail(MPS_ERR_ARG, "mps_plan_sync_check: plan is NULL");
    int status = 0;
    MPS_CUDA(cudaMemcpyAsync(&status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MPS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (status != kDevOk) {
        cudaMemsetAsync(p->d_status, 0, sizeof(int), (cudaStream_t)stream);
        cudaMemsetAsync(p->d_cnt, 0, sizeof(int) * (size_t)p->n_tiles * p->n_col_slabs, (cudaStream_t)stream);  // a block that gave up left its count short
        return fail(MPS_ERR_DEVICE, "a tile block gave up waiting for its staged window (status %d)", status);
    }
    return MPS_OK;
}

extern "C" int mps_plan_profile(mps_plan *p, int enable) {
    if (!p) return fail(MPS_ERR_ARG, "mps_plan_profile: plan is NULL");
    if (enable)
        for (cudaEvent_t &e : p->prof_ev)
            if (!e) MPS_CUDA(cudaEventCreate(&e));
    p->profiling = enable != 0;
    p->prof_used = 0;
    return MPS_OK;
}

extern "C" int mps_plan_profile_read(mps_plan *p, void *stream, double *tile_ms, int32_t *launches) {
    if (!p || !tile_ms || !launches) return fail(MPS_ERR_ARG, "mps_plan_profile_read: NULL argument");
    MPS_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    double sum = 0.0;
    for (int i = 0; i < p->prof_used; ++i) {
        float ms = 0.0f;
        MPS_CUDA(cudaEventElapsedTime(&ms, p->prof_ev[2 * i], p->prof_ev[2 * i + 1]));
        sum += ms;
    }
    *tile_ms = sum;
    *launches = p->prof_used;
    p->prof_used = 0;
    return MPS_OK;
}

extern "C" int mps_plan_info(const mps_plan *p, int64_t what[16]) {
    if (!p || !what) return fail(MPS_ERR_ARG, "mps_plan_info: NULL argument");
    for (int i = 0; i < 16; ++i) what[i] = 0;
    what[0] = p->n_chunks; what[1] = p->ipt; what[2] = p->nch; what[3] = p->n_tiles;
    what[4] = p->gl; what[5] = p->vec; what[6] = p->unroll; what[7] = p->smem_bytes;
    what[8] = p->n_long; what[9] = p->tpw_effective;
    what[10] = 1 + (((!p->fused && p->n_tiles > 1) || p->n_long > 0) ? 1 : 0);
    what[11] = p->long_chain; what[12] = p->cpu; what[13] = p->tile_items / p->unit_items; what[14] = p->block; what[15] = p->very_long;
    return MPS_OK;
}

extern "C" int mps_plan_layout(const mps_plan *p, int64_t what[12]) {
    if (!p || !what) return fail(MPS_ERR_ARG, "mps_plan_layout: NULL argument");
    for (int i = 0; i < 12; ++i) what[i] = 0;
    what[0] = p->unit_items; what[1] = p->tile_items / p->unit_items; what[2] = p->tile_items; what[3] = p->n_tiles;
    what[4] = p->sub_chunk; what[5] = p->smem_bytes; what[6] = p->n_col_slabs; what[7] = p->fused;
    what[8] = p->walk ? 32 / p->gl : 1;
    return MPS_OK;
}

extern "C" int mps_layout_query(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost, int64_t what[12]) {
    if (!what) return fail(MPS_ERR_ARG, "mps_layout_query: what is NULL");
    if (dim < 1 || cost < 1) return fail(MPS_ERR_ARG, "mps_layout_query: dim and cost must be >= 1 (dim=%d cost=%d)", dim, cost);
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "mps_layout_query: unknown dtype %d", dtype);
    if (int rc = check_shape(n_rows, nnz)) return rc;
    mps_plan plan;
    plan_init_shape(&plan, n_rows, nnz, dim, dtype, cost, 1);
    plan.sm_count = 148;  // the layout of a B200, whatever machine asks
    if (int rc = plan_layout(&plan)) return rc;
    return mps_plan_layout(&plan, what);
}

// ------------------------------------------------------------------------------------- host-buffer call
//
// The call is cut into row slabs (equal nnz + 4*rows) so that PCIe runs in both directions at once:
//   upload stream  : all of B first (no row of C can be formed before it is whole), then col_idx/val slab by slab;
//   plan stream    : row_ptr, rebasing + partition of every slab, beside the upload of B;
//   work stream    : waits for slab s, multiplies it;
//   download stream: copies slab s of C back as soon as it is multiplied
// so the download of C starts right after B and the first slab of A have landed and overlaps the upload of
// the later slabs.  Device buffers and the per-slab plans live in a per-thread workspace that only grows /
// is rebuilt when shapes change.

// out[i] = rp[row0 + i] - rp[row0], i = 0..rows
__global__ void rebase_kernel(const int *__restrict__ rp, int row0, int rows, int *__restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= rows) out[i] = rp[row0 + i] - rp[row0];
}

// Column indices of a slab in the workspace copy: an index outside [0, n_cols) is replaced by 0 and the smallest such
// position recorded, so that the multiply that follows can only gather rows of B that exist; the host turns the record
// into MPS_ERR_ARG.  Reads 4 bytes per non-zero out of device memory - nothing beside the upload it follows.
__global__ void clamp_columns_kernel(int *__restrict__ col, long long n, unsigned n_cols, long long base, unsigned long long *__restrict__ first_bad) {
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (long long)gridDim.x * blockDim.x)
        if ((unsigned)col[k] >= n_cols) {
            atomicMin(first_bad, (unsigned long long)(base + k));
            col[k] = 0;
        }
}

namespace {
const int kMaxHostSlabs = 16;  // measured on a 2^21-node graph: 8 and 12 slabs 0.1-0.7 ms slower per call, 24 and 32 slower still
const long long kHostSlabMinItems = 4ll << 20;  // below this the call is one slab

struct HostWorkspace {
    static const int kBuffers = 8;
    void *buf[kBuffers] = {};  // rp, col, val, B, C, rebased rp slabs, row scale, column scale
    size_t cap[kBuffers] = {};
    mps_plan *plan[kMaxHostSlabs] = {};
    cudaStream_t s_in = nullptr, s_b = nullptr, s_work = nullptr, s_out = nullptr;  // plan, upload, work, download
    cudaEvent_t ev_b = nullptr, ev_slab[kMaxHostSlabs] = {}, ev_done[kMaxHostSlabs] = {};
    unsigned long long *d_bad = nullptr;  // smallest position of a column index outside [0, n_cols) seen by this call
    int device = -1;
    void release() {
        cudaFree(d_bad); d_bad = nullptr;
        for (int i = 0; i < kBuffers; ++i) { cudaFree(buf[i]); buf[i] = nullptr; cap[i] = 0; }
        for (int i = 0; i < kMaxHostSlabs; ++i) {
            mps_plan_destroy(plan[i]); plan[i] = nullptr;
            if (ev_slab[i]) cudaEventDestroy(ev_slab[i]);
            if (ev_done[i]) cudaEventDestroy(ev_done[i]);
            ev_slab[i] = ev_done[i] = nullptr;
        }
        if (ev_b) cudaEventDestroy(ev_b);
        if (s_in) cudaStreamDestroy(s_in);
        if (s_b) cudaStreamDestroy(s_b);
        if (s_work) cudaStreamDestroy(s_work);
        if (s_out) cudaStreamDestroy(s_out);
        ev_b = nullptr; s_in = s_b = s_work = s_out = nullptr; device = -1;
    }
};
thread_local HostWorkspace g_ws;
}  // namespace

static int ws_reserve(int i, size_t bytes) {
    if (g_ws.cap[i] >= bytes) return MPS_OK;
    cudaFree(g_ws.buf[i]);
    g_ws.buf[i] = nullptr; g_ws.cap[i] = 0;
    MPS_CUDA(cudaMalloc(&g_ws.buf[i], bytes ? bytes : 16));
    g_ws.cap[i] = bytes;
    return MPS_OK;
}

extern "C" void mps_host_workspace_release(void) { g_ws.release(); }

// The row slabs of one host-buffer call and the order in which they are uploaded and multiplied.
struct HostSlabs {
    int n = 1;
    int32_t bounds[kMaxHostSlabs + 1];
    int order[kMaxHostSlabs];
};

static int host_slabs(int32_t n_rows, int32_t nnz, const int32_t *row_ptr, HostSlabs *hs) {
    const long long items = (long long)n_rows + nnz;
    int n_slabs = (int)(items / kHostSlabMinItems);
    if (n_slabs < 1) n_slabs = 1;
    if (n_slabs > kMaxHostSlabs) n_slabs = kMaxHostSlabs;
    hs->n = n_slabs;
    if (int rc = mps_slab_bounds_items(row_ptr, n_rows, n_slabs, 4, hs->bounds)) return rc;
    // slabs with many rows first: their share of C is the largest download and should overlap the most uploads
    for (int s = 0; s < n_slabs; ++s) hs->order[s] = s;
    for (int i = 1; i < n_slabs; ++i)
        for (int j = i; j > 0 && hs->bounds[hs->order[j] + 1] - hs->bounds[hs->order[j]] > hs->bounds[hs->order[j - 1] + 1] - hs->bounds[hs->order[j - 1]]; --j) {
            const int t = hs->order[j]; hs->order[j] = hs->order[j - 1]; hs->order[j - 1] = t;
        }
    return MPS_OK;
}

// First step of a host-buffer call: the thread's workspace on the current device, then row_ptr and B on their way.
// Uploads leave in the order in which they are queued, whatever their stream, so row_ptr (small; the partitions need
// it) goes first and B, the largest single upload, right behind it - before the host looks at the caller's CSR
// arrays: nothing on the device reads row_ptr until the host has checked it.  B already on the device: it is complete
// when the work queued so far on the caller's stream has run (another GPU's share of it may still be arriving over
// NVLink meanwhile).
static int host_begin(int32_t n_rows, int32_t n_cols, int32_t dim, int dtype, const int32_t *row_ptr, const float *row_scale,
                      const float *col_scale, const void *B, bool b_on_device, cudaStream_t b_stream) {
    int dev = 0;
    MPS_CUDA(cudaGetDevice(&dev));
    if (g_ws.device != dev) { g_ws.release(); g_ws.device = dev; }
    if (!g_ws.s_in) {
        MPS_CUDA(cudaStreamCreateWithFlags(&g_ws.s_in, cudaStreamNonBlocking));
        MPS_CUDA(cudaStreamCreateWithFlags(&g_ws.s_b, cudaStreamNonBlocking));
        MPS_CUDA(cudaStreamCreateWithFlags(&g_ws.s_work, cudaStreamNonBlocking));
        MPS_CUDA(cudaStreamCreateWithFlags(&g_ws.s_out, cudaStreamNonBlocking));
        MPS_CUDA(cudaEventCreateWithFlags(&g_ws.ev_b, cudaEventDisableTiming));
        for (int i = 0; i < kMaxHostSlabs; ++i) {
            MPS_CUDA(cudaEventCreateWithFlags(&g_ws.ev_slab[i], cudaEventDisableTiming));
            MPS_CUDA(cudaEventCreateWithFlags(&g_ws.ev_done[i], cudaEventDisableTiming));
        }
        MPS_CUDA(cudaMalloc(&g_ws.d_bad, sizeof(unsigned long long)));
    }
    if (int rc = ws_reserve(0, 4 * ((size_t)n_rows + 1))) return rc;
    MPS_CUDA(cudaMemcpyAsync(g_ws.buf[0], row_ptr, 4 * ((size_t)n_rows + 1), cudaMemcpyHostToDevice, g_ws.s_in));
    // scaled product: the two factor vectors take the place of a value per non-zero; they are small and go ahead of B too
    if (row_scale) {
        if (int rc = ws_reserve(6, 4 * (size_t)n_rows)) return rc;
        MPS_CUDA(cudaMemcpyAsync(g_ws.buf[6], row_scale, 4 * (size_t)n_rows, cudaMemcpyHostToDevice, g_ws.s_in));
    }
    if (col_scale) {
        if (int rc = ws_reserve(7, 4 * (size_t)n_cols)) return rc;
        MPS_CUDA(cudaMemcpyAsync(g_ws.buf[7], col_scale, 4 * (size_t)n_cols, cudaMemcpyHostToDevice, g_ws.s_in));
    }
    if (b_on_device) {
        MPS_CUDA(cudaEventRecord(g_ws.ev_b, b_stream));
        return MPS_OK;
    }
    const size_t bytes = (dtype == MPS_F16 ? 2 : 4) * (size_t)n_cols * dim;
    if (int rc = ws_reserve(3, bytes)) return rc;
    MPS_CUDA(cudaMemcpyAsync(g_ws.buf[3], B, bytes, cudaMemcpyHostToDevice, g_ws.s_b));
    MPS_CUDA(cudaEventRecord(g_ws.ev_b, g_ws.s_b));
    return MPS_OK;
}

static int host_call(int32_t n_rows, int32_t n_cols, int32_t dim, int dtype, int32_t cost, int32_t threads_per_warp,
                     const int32_t *row_ptr, const int32_t *col_idx, const void *val, bool row_scaled, bool col_scaled, const void *B,
                     bool b_on_device, void *C, const HostSlabs &hs, long long *bad_column) {
    const size_t elem = dtype == MPS_F16 ? 2 : 4;
    const int n_slabs = hs.n;
    const int32_t *bounds = hs.bounds;
    const int *order = hs.order;

    // device layout: slab s of col_idx/val starts at an offset that is a multiple of 8 elements, so its
    // base stays 16-byte aligned and the tile kernel can stage it with bulk copies
    size_t off[kMaxHostSlabs + 1];
    off[0] = 0;
    for (int s = 0; s < n_slabs; ++s) {
        const size_t len = (size_t)(row_ptr[bounds[s + 1]] - row_ptr[bounds[s]]);
        off[s + 1] = (off[s] + len + 7) & ~(size_t)7;
    }
    const size_t rp_slab_cap = ((size_t)n_rows + 1 + 8 * (size_t)n_slabs + 8);
    const size_t bytes[6] = {4 * ((size_t)n_rows + 1), 4 * (off[n_slabs] + 8), val ? elem * (off[n_slabs] + 8) : 0,
                             b_on_device ? 0 : elem * (size_t)n_cols * dim, elem * (size_t)n_rows * dim, 4 * rp_slab_cap};
    for (int i = 0; i < 6; ++i)
        if (i != 0 && i != 3)  // host_begin() reserved the buffers of row_ptr and B, and both are on their way
            if (int rc = ws_reserve(i, bytes[i])) return rc;
    int32_t *d_rp = (int32_t *)g_ws.buf[0], *d_col = (int32_t *)g_ws.buf[1], *d_rps = (int32_t *)g_ws.buf[5];
    char *d_val = (char *)g_ws.buf[2], *d_C = (char *)g_ws.buf[4];

    cudaStream_t s_in = g_ws.s_in, s_up = g_ws.s_b, s_work = g_ws.s_work, s_out = g_ws.s_out;
    // host_begin() has queued row_ptr and B; rebasing and the partitions run beside B's upload
    const void *d_B = b_on_device ? B : g_ws.buf[3];
    // A's slabs follow B on the upload stream, in the order in which they will be multiplied; they are queued before the
    // host turns to the partitions below, each of which waits for a count from the device
    for (int i = 0; i < n_slabs; ++i) {
        const int s = order[i];
        const size_t k0 = (size_t)row_ptr[bounds[s]], len = (size_t)(row_ptr[bounds[s + 1]] - row_ptr[bounds[s]]);
        if (len) {
            MPS_CUDA(cudaMemcpyAsync(d_col + off[s], col_idx + k0, 4 * len, cudaMemcpyHostToDevice, s_up));
            if (val) MPS_CUDA(cudaMemcpyAsync(d_val + elem * off[s], (const char *)val + elem * k0, elem * len, cudaMemcpyHostToDevice, s_up));
        }
        MPS_CUDA(cudaEventRecord(g_ws.ev_slab[s], s_up));  // behind B on the same stream: B is whole when this fires
    }
    size_t rps_off[kMaxHostSlabs];
    size_t at = 0;
    for (int i = 0; i < n_slabs; ++i) {
        const int s = order[i];
        const int r0 = bounds[s], rows = bounds[s + 1] - bounds[s];
        const int slab_nnz = row_ptr[bounds[s + 1]] - row_ptr[r0];
        mps_plan *&p = g_ws.plan[s];
        if (!p || p->n_rows != rows || p->nnz != slab_nnz || p->dim != dim || p->dtype != dtype || p->cost != cost) {
            mps_plan_destroy(p);
            p = nullptr;
            if (int rc = mps_plan_create(rows, slab_nnz, dim, dtype, cost, threads_per_warp, &p)) return rc;
        }
        rps_off[s] = at;
        rebase_kernel<<<(rows + 1 + 255) / 256, 256, 0, s_in>>>(d_rp, r0, rows, d_rps + at);
        MPS_CUDA(cudaGetLastError());
        if (int rc = mps_plan_partition(p, d_rps + at, s_in)) return rc;
        at = (at + (size_t)rows + 1 + 7) & ~(size_t)7;
    }
    for (int s = n_slabs; s < kMaxHostSlabs; ++s) { mps_plan_destroy(g_ws.plan[s]); g_ws.plan[s] = nullptr; }

    MPS_CUDA(cudaStreamWaitEvent(s_work, g_ws.ev_b, 0));
    MPS_CUDA(cudaMemsetAsync(g_ws.d_bad, 0xff, sizeof(unsigned long long), s_work));
    for (int i = 0; i < n_slabs; ++i) {
        const int s = order[i];
        const int r0 = bounds[s], rows = bounds[s + 1] - bounds[s];
        const size_t k0 = (size_t)row_ptr[r0], len = (size_t)(row_ptr[bounds[s + 1]] - row_ptr[r0]);
        MPS_CUDA(cudaStreamWaitEvent(s_work, g_ws.ev_slab[s], 0));
        // the caller's column indices are checked where they have just landed, ahead of the multiply on the same stream:
        // no kernel gathers by an index outside B (the host's memory is left to the uploads)
        if (len) {
            clamp_columns_kernel<<<592, 256, 0, s_work>>>(d_col + off[s], (long long)len, (unsigned)n_cols, (long long)k0, g_ws.d_bad);
            MPS_CUDA(cudaGetLastError());
        }
        char *c_slab = d_C + elem * (size_t)r0 * dim;
        if (row_scaled || col_scaled) {  // the factors landed on the plan stream ahead of the partitions the host has waited for
            if (int rc = mps_spmm_scaled(g_ws.plan[s], d_rps + rps_off[s], d_col + off[s], row_scaled ? (const float *)g_ws.buf[6] + r0 : nullptr,
                                         col_scaled ? (const float *)g_ws.buf[7] : nullptr, d_B, c_slab, s_work))
                return rc;
        } else if (int rc = mps_spmm(g_ws.plan[s], d_rps + rps_off[s], d_col + off[s], val ? (const void *)(d_val + elem * off[s]) : nullptr,
                                     d_B, c_slab, s_work))
            return rc;
        MPS_CUDA(cudaEventRecord(g_ws.ev_done[s], s_work));
        MPS_CUDA(cudaStreamWaitEvent(s_out, g_ws.ev_done[s], 0));
        if (rows) MPS_CUDA(cudaMemcpyAsync((char *)C + elem * (size_t)r0 * dim, c_slab, elem * (size_t)rows * dim, cudaMemcpyDeviceToHost, s_out));
    }
    unsigned long long first_bad = ~0ull;
    MPS_CUDA(cudaMemcpyAsync(&first_bad, g_ws.d_bad, sizeof first_bad, cudaMemcpyDeviceToHost, s_work));
    MPS_CUDA(cudaStreamSynchronize(s_in));
    MPS_CUDA(cudaStreamSynchronize(s_up));
    MPS_CUDA(cudaStreamSynchronize(s_out));
    for (int s = 0; s < n_slabs; ++s)
        if (int rc = mps_plan_sync_check(g_ws.plan[s], s_work)) return rc;
    if (first_bad != ~0ull) *bad_column = (long long)first_bad;
    return MPS_OK;
}

static int host_entry(const char *who, int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int dtype, int32_t cost, int32_t threads_per_warp,
                      const int32_t *row_ptr, const int32_t *col_idx, const void *val, const float *row_scale, const float *col_scale,
                      const void *B, bool b_on_device, void *b_stream, void *C) {
    if (!row_ptr || !B || !C || (!col_idx && nnz > 0)) return fail(MPS_ERR_ARG, "%s: NULL argument", who);
    if (dim < 1 || cost < 1 || n_cols < 0) return fail(MPS_ERR_ARG, "%s: dim and cost must be >= 1, n_cols >= 0", who);
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "%s: unknown dtype %d", who, dtype);
    if (int rc = check_shape(n_rows, nnz)) return rc;
    if (row_ptr[n_rows] != nnz) return fail(MPS_ERR_ARG, "%s: row_ptr[n_rows] is %d, nnz is %d", who, row_ptr[n_rows], nnz);
    // row_ptr and B are on their way before the caller's CSR arrays are looked at (B is half of the upload)
    auto drain = [] {  // copies may be queued on the caller's buffers: let them finish before the caller may free those
        const std::string kept = g_error;
        for (cudaStream_t st : {g_ws.s_in, g_ws.s_b, g_ws.s_work, g_ws.s_out})
            if (st) cudaStreamSynchronize(st);
        g_error = kept;
    };
    int rc = host_begin(n_rows, n_cols, dim, dtype, row_ptr, row_scale, col_scale, B, b_on_device, (cudaStream_t)b_stream);
    const std::string begin_error = rc != MPS_OK ? g_error : std::string();
    // the caller's arrays are checked before any kernel can index by them: row_ptr here on the host (small, and the slab
    // bounds are taken from it), col_idx on the device where each slab lands; a bad index is reported in preference to any
    // other failure of the call
    HostSlabs hs;
    int bad_arg = check_csr_host(who, n_rows, n_cols, row_ptr, nullptr, 0);
    if (bad_arg == MPS_OK && n_cols == 0 && nnz > 0) bad_arg = fail(MPS_ERR_ARG, "%s: col_idx[0] = %d outside [0, 0)", who, col_idx[0]);
    if (bad_arg == MPS_OK) bad_arg = host_slabs(n_rows, nnz, row_ptr, &hs);
    if (bad_arg != MPS_OK) {
        drain();
        return bad_arg;
    }
    long long bad = -1;
    if (rc == MPS_OK)
        rc = host_call(n_rows, n_cols, dim, dtype, cost, threads_per_warp, row_ptr, col_idx, val, row_scale != nullptr, col_scale != nullptr, B, b_on_device,
                       C, hs, &bad);
    else g_error = begin_error;
    // without a usable device nothing was checked there: the same check on host threads, so that a bad index is
    // reported in preference to the missing device
    if (rc == MPS_ERR_CUDA && bad < 0) {
        const std::string kept = g_error;
        bad = first_bad_column(col_idx, nnz, n_cols, 0);
        g_error = kept;
    }
    if (rc != MPS_OK || bad >= 0) {
        // a step failed with copies possibly still queued on the caller's buffers (the message of the failure stays
        // the one reported)
        drain();
        const std::string kept = g_error;
        for (mps_plan *&p : g_ws.plan) { mps_plan_destroy(p); p = nullptr; }  // a half-built set of slab plans is not reused
        g_error = kept;
        if (bad >= 0) rc = fail(MPS_ERR_ARG, "%s: col_idx[%lld] = %d outside [0, %d)", who, bad, col_idx[bad], n_cols);
    }
    return rc;
}

extern "C" int mps_spmm_host(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int dtype, int32_t cost, int32_t threads_per_warp,
                             const int32_t *row_ptr, const int32_t *col_idx, const void *val, const void *B, void *C) {
    return host_entry("mps_spmm_host", n_rows, n_cols, nnz, dim, dtype, cost, threads_per_warp, row_ptr, col_idx, val, nullptr, nullptr, B, false, nullptr, C);
}

extern "C" int mps_spmm_host_resident_b(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int dtype, int32_t cost,
                                        int32_t threads_per_warp, const int32_t *row_ptr, const int32_t *col_idx, const void *val,
                                        const void *d_B, void *b_ready_stream, void *C) {
    return host_entry("mps_spmm_host_resident_b", n_rows, n_cols, nnz, dim, dtype, cost, threads_per_warp, row_ptr, col_idx, val, nullptr, nullptr, d_B,
                      true, b_ready_stream, C);
}

extern "C" int mps_spmm_host_scaled(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int32_t cost, int32_t threads_per_warp,
                                    const int32_t *row_ptr, const int32_t *col_idx, const float *row_scale, const float *col_scale,
                                    const void *B, void *C) {
    if (!row_scale && !col_scale) return fail(MPS_ERR_ARG, "mps_spmm_host_scaled: both scale arrays are NULL (use mps_spmm_host)");
    return host_entry("mps_spmm_host_scaled", n_rows, n_cols, nnz, dim, MPS_F32, cost, threads_per_warp, row_ptr, col_idx, nullptr, row_scale, col_scale,
                      B, false, nullptr, C);
}

// ------------------------------------------------------------------------------------- slabs (host)

extern "C" int mps_slab_bounds(const int32_t *row_ptr, int32_t n_rows, int32_t n_slabs, int32_t *bounds) {
    if (!row_ptr || !bounds || n_rows < 0 || n_slabs < 1) return fail(MPS_ERR_ARG, "mps_slab_bounds: bad argument");
    const long long nnz = row_ptr[n_rows];
    bounds[0] = 0;
    for (int g = 1; g < n_slabs; ++g) {
        const long long want = nnz * g / n_slabs;
        int lo = 0, hi = n_rows;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (row_ptr[mid] < want) lo = mid + 1;
            else hi = mid;
        }
        bounds[g] = lo;
    }
    bounds[n_slabs] = n_rows;
    return MPS_OK;
}

extern "C" int mps_slab_bounds_items(const int32_t *row_ptr, int32_t n_rows, int32_t n_slabs, int32_t row_weight, int32_t *bounds) {
    if (!row_ptr || !bounds || n_rows < 0 || n_slabs < 1 || row_weight < 0) return fail(MPS_ERR_ARG, "mps_slab_bounds_items: bad argument");
    const long long w = row_weight;
    const long long items = (long long)row_ptr[n_rows] + w * n_rows;
    bounds[0] = 0;
    for (int g = 1; g < n_slabs; ++g) {
        const long long want = items * g / n_slabs;
        int lo = 0, hi = n_rows;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if ((long long)row_ptr[mid] + w * mid < want) lo = mid + 1;
            else hi = mid;
        }
        bounds[g] = lo;
    }
    bounds[n_slabs] = n_rows;
    return MPS_OK;
}

extern "C" int mps_slab_rebase(const int32_t *row_ptr, int32_t row0, int32_t row1, int32_t *out_row_ptr) {
    if (!row_ptr || !out_row_ptr || row0 < 0 || row1 < row0) return fail(MPS_ERR_ARG, "mps_slab_rebase: bad argument");
    const int32_t base = row_ptr[row0];
    for (int32_t i = row0; i <= row1; ++i) out_row_ptr[i - row0] = row_ptr[i] - base;
    return MPS_OK;
}
