/*
 * mps.h - C ABI of the B200 merge-path CSR SpMM library (libmps_b200.so).
 *
 * C = A * B with A sparse (CSR, int32 row_ptr / col_idx, optional values), B and C dense
 * row-major with `dim` columns.  The reference (cag-uconn/MergePath-SpMM) has no function-level
 * API: its boundary is the two-line `.csr` text file and the process entry point
 * `MergePathSpMM <file> <dim> <cost> <threads_per_warp> <repeat>`.  Each entry point below names
 * the piece of the reference program it replaces (file:line inside the reference tree).
 *
 * Conventions
 *   - every function returns an mps_status (0 = ok, negative = error); nothing throws, nothing
 *     calls exit(); mps_last_error() gives the message of the calling thread's last failure;
 *   - device pointers are caller-owned; a plan owns only its scratch (tile coordinates, carry
 *     rows, status word) on the device that was current when it was created;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - launches are asynchronous; mps_plan_sync_check() waits and reports device-side errors;
 *   - there is no CPU fallback: without a usable CUDA device the compute calls fail with
 *     MPS_ERR_CUDA.
 */
#ifndef MPS_B200_H
#define MPS_B200_H

#include <stddef.h>
#include <stdint.h>

/* Every entry point is exported from a library otherwise built with hidden visibility. */
#define MPS_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    MPS_OK = 0,
    MPS_ERR_ARG = -1,         /* NULL pointer, negative size, cost < 1, dim < 1 ...            */
    MPS_ERR_IO = -2,          /* file missing / unreadable / short write                        */
    MPS_ERR_FORMAT = -3,      /* .csr text does not follow the grammar                          */
    MPS_ERR_CUDA = -4,        /* a CUDA runtime call failed (message has the CUDA error string) */
    MPS_ERR_UNSUPPORTED = -5, /* shape outside what the kernels cover (e.g. N+1+nnz >= 2^31)    */
    MPS_ERR_NOMEM = -6,
    MPS_ERR_DEVICE = -7,      /* a kernel reported a bounded wait that ran out                  */
    MPS_ERR_ALIGN = -8,       /* a device pointer is not aligned to its element size            */
    MPS_ERR_STATE = -9        /* e.g. mps_spmm before mps_plan_partition                        */
} mps_status;

typedef enum { MPS_F32 = 0, MPS_F16 = 1 } mps_dtype;

MPS_API const char *mps_last_error(void);
MPS_API const char *mps_version(void);

/* ------------------------------------------------------------------ .csr files (host) ---- */

/* A graph as the reference's loader leaves it in memory (src/MergePathSpMM.cu:26-35,143-173):
 * N = cells(line 1) - 1, nnz = last cell of line 1.  Arrays are malloc'ed by the library. */
typedef struct {
    int32_t n_rows;
    int32_t nnz;
    int32_t *row_ptr; /* n_rows + 1 */
    int32_t *col_idx; /* nnz        */
} mps_csr;

/* Replaces the two-pass getline/stringstream/stoi loader (src/MergePathSpMM.cu:119-173).
 * Same grammar: line 1 = row_ptr, line 2 = col_idx, decimal integers separated by ',', trailing
 * ',' optional, final newline optional, blanks before and after a number allowed, '\r' rejected.
 * Unlike the reference a missing file, a malformed cell, a cell count that disagrees with nnz, a
 * decreasing row_ptr or a column index outside [0, n_rows) is an error.  n_threads <= 0 picks
 * the hardware concurrency. */
MPS_API int mps_csr_load(const char *path, int n_threads, mps_csr *out);
MPS_API void mps_csr_free(mps_csr *csr);

/* The same loader for a file whose columns reach beyond its rows.  scripts/npz_to_csr.py:13-19 builds its
 * coo_matrix without a shape, so a destination index above every source index gives such a file; the
 * reference program would gather past the end of its N-row B for it (src/MergePathSpMM.cu:176-182,441).
 * Any non-negative column index is accepted and *n_cols = max(n_rows, largest index + 1) is the number of
 * rows B must have. */
MPS_API int mps_csr_load_rect(const char *path, int n_threads, mps_csr *out, int32_t *n_cols);

/* Replaces the writers scripts/npz_to_csr.py:21-28 and scripts/fetch_dataset.py:14-21:
 * every cell followed by ',', one '\n' between the lines, none at the end. */
MPS_API int mps_csr_save(const char *path, int32_t n_rows, const int32_t *row_ptr, const int32_t *col_idx);

/* Binary sidecar (no reference counterpart; the text format cannot carry values and a
 * 10^9-nnz graph is ~10 GB of text): 32-byte header, then raw row_ptr, col_idx and, when
 * val_bytes != 0, values of that element size (4 = fp32, 2 = fp16).  Load mallocs the arrays and applies
 * the text loader's checks (row_ptr non-decreasing, columns inside [0, n_rows)). */
MPS_API int mps_csr_save_bin(const char *path, int32_t n_rows, const int32_t *row_ptr, const int32_t *col_idx,
                     const void *val, int val_bytes);
MPS_API int mps_csr_load_bin(const char *path, mps_csr *out, void **val, int *val_bytes);

/* Replaces the COO -> CSR step of the reference's converters (scripts/npz_to_csr.py:13-19,
 * scripts/fetch_dataset.py:11-13: scipy coo_matrix(...).tocsr()): duplicate (src, dst) pairs collapse
 * into one entry and every row's columns come out sorted.  The matrix is square with n_nodes rows
 * (0 = largest index + 1).  Host arrays in, malloc'ed CSR out (mps_csr_free). */
MPS_API int mps_coo_to_csr(int32_t n_nodes, int64_t n_edges, const int64_t *src, const int64_t *dst, int n_threads,
                   mps_csr *out);

/* The same conversion on the device (no reference counterpart): d_src / d_dst are int64 device arrays,
 * d_row_ptr receives n_nodes + 1 entries, d_col_idx (capacity n_edges) the columns, *nnz_out the number
 * kept after duplicates collapse.  Allocates its temporaries, synchronises the stream once. */
MPS_API int mps_coo_to_csr_device(int32_t n_nodes, int64_t n_edges, const int64_t *d_src, const int64_t *d_dst,
                          int32_t *d_row_ptr, int32_t *d_col_idx, int32_t *nnz_out, void *stream);

/* CSR of the transpose, on the device (no reference counterpart: the reference has no backward pass; this is
 * what dB = A^T dC of its GCN use case multiplies with - for a symmetric A the transpose is A itself and
 * nothing has to be built).  A is n_rows x n_cols; d_row_ptr_t receives n_cols + 1 entries, d_col_idx_t and
 * d_val_t (NULL together with d_val; dtype gives the value width) nnz entries; every transposed row's
 * columns come out ascending.  Allocates its temporaries (12 bytes per non-zero), synchronises the stream. */
MPS_API int mps_csr_transpose_device(int32_t n_rows, int32_t n_cols, int32_t nnz, int dtype, const int32_t *d_row_ptr,
                             const int32_t *d_col_idx, const void *d_val, int32_t *d_row_ptr_t, int32_t *d_col_idx_t,
                             void *d_val_t, void *stream);

/* Replaces scripts/npz_to_csr.py as a whole up to the text writer: reads the members `src_li` and
 * `dst_li` (one-dimensional little-endian integer arrays) of a `.npz` archive, stored or deflated,
 * and converts them with mps_coo_to_csr; follow with mps_csr_save for the `.csr` text. */
MPS_API int mps_npz_to_csr(const char *path, int n_threads, mps_csr *out);

/* ------------------------------------------------------------------ partition ------------ */

/* Chunk count and items per chunk for a cost, exactly the reference's integer arithmetic:
 * P = max(1024, (N+1+nnz-1)/cost)  (src/MergePathSpMM.cu:138-139),
 * ipt = ceil((N+1+nnz)/P)          (src/MergePathSpMM.cu:327-328). */
MPS_API int mps_chunk_count(int32_t n_rows, int32_t nnz, int32_t cost, int32_t *n_chunks, int32_t *items_per_chunk);

/* Replaces MergePathSearch called over all chunk boundaries (src/MergePathSpMM.cu:280-297,
 * 330-334), on the device: d_xy receives n_chunks + 1 interleaved (x, y) pairs for the diagonals
 * min(ipt * t, N+1+nnz), t = 0..n_chunks, in the reference's convention (x counts row_ptr
 * entries including row_ptr[0], y counts non-zeros).  Bit-exact with the reference. */
MPS_API int mps_partition_device(const int32_t *d_row_ptr, int32_t n_rows, int32_t nnz, int32_t n_chunks,
                         int32_t *d_xy, void *stream);

/* Replaces generate_mp_sched (src/MergePathSpMM.cu:300-385), on the device: the six int arrays
 * of n_chunks entries each, written to d_six in the reference's return order (feature_start,
 * feature_start_num, feature_end, feature_end_num, start_row, end_row), bit-exact including the
 * zero-sentinel behaviour, so that they can be handed to the reference's own kernels. */
MPS_API int mps_schedule_device(const int32_t *d_row_ptr, int32_t n_rows, int32_t nnz, int32_t n_chunks,
                        int32_t *d_six, void *stream);

/* The same two results on the host, on n_threads host threads (<= 0: all): replaces MergePathSearch over
 * all chunk boundaries and generate_mp_sched where they run in the reference - on the host
 * (src/MergePathSpMM.cu:280-297, 300-385) - for callers without a device at hand.  xy receives
 * n_chunks + 1 interleaved (x, y) pairs, six the six arrays of n_chunks entries in the reference's return
 * order; both bit-exact with the reference and with the device entry points above.  Host row_ptr. */
MPS_API int mps_partition_host(const int32_t *row_ptr, int32_t n_rows, int32_t n_chunks, int32_t *xy, int n_threads);
MPS_API int mps_schedule_host(const int32_t *row_ptr, int32_t n_rows, int32_t n_chunks, int32_t *six, int n_threads);

/* ------------------------------------------------------------------ SpMM plan ------------ */

typedef struct mps_plan mps_plan;

/* Replaces the set-up part of main() (src/MergePathSpMM.cu:138-139,192-228): fixes N, nnz, dim,
 * element type and the reference's two tuning arguments.  `cost` = merge items per chunk as in
 * the reference.  `threads_per_warp` is accepted for command-line compatibility; where the
 * reference exits when it exceeds 32/dim (:224-228) the value is clamped instead (the number of
 * chunks a warp walks at once is fixed by the 128-bit row loads: 128/dim chunks for fp32; fp16 rows of up to 28
 * columns that are a multiple of 4 are read with 64-bit loads, four columns per lane, so that a warp walks at most
 * eight units - B and C then need 8-byte alignment, otherwise 16 bytes when dim is a multiple of 4 (fp32) or 8 (fp16)).
 * Allocates the plan's device scratch on the current device. */
MPS_API int mps_plan_create(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost,
                    int32_t threads_per_warp, mps_plan **out);
MPS_API void mps_plan_destroy(mps_plan *plan);

/* Optional tuning before mps_plan_partition: chunks per unit (0 = automatic; a unit is the run of
 * consecutive chunks one lane group walks with its accumulator kept in registers, a tile holds
 * block_threads/lanes_per_chunk units), gathers in flight per thread (4, 8 or 10; 0 = automatic: 10, the most that fits the registers of 12 resident blocks), staging through
 * bulk async copies (1, default) or plain loads (0), threads per tile block (64, 128, 256; 0 =
 * automatic: 64), cross-tile fix-up inside the tile kernel (1) or as a kernel of its own (0; -1 =
 * automatic: inside for up to 2048 tiles, where a second launch costs more than it saves). */
MPS_API int mps_plan_tune(mps_plan *plan, int32_t chunks_per_unit, int32_t unroll, int32_t bulk_staging,
                  int32_t block_threads, int32_t fused_fixup);

/* Replaces the call of generate_mp_sched and the eleven uploads that follow it
 * (src/MergePathSpMM.cu:192-220): searches the tile boundaries on the device, records for every tile
 * which tile ends the row its carry belongs to, and lists the rows whose carries span thousands of tiles.  Must be called once per row_ptr before mps_spmm; synchronises
 * the stream once (it reads back one counter). */
MPS_API int mps_plan_partition(mps_plan *plan, const int32_t *d_row_ptr, void *stream);

/* Replaces one iteration of the launch loops (src/MergePathSpMM.cu:230-243, 249-263) and the
 * kernels spmm_merge_path / spmm_merge_path_64 (:388-574; fp16: MergePathSpMM_fp16.cu:389-575).
 * d_val == NULL means every stored value is 1 (the .csr file has no values).  For MPS_F16 plans
 * val, B and C hold IEEE fp16 and all sums are kept in fp32 until the single rounding of C.
 * Every row of C is written exactly once per call - nothing has to be zeroed and repeated calls
 * do not accumulate (the reference's atomics do, :204,231).  Rows split across chunks are
 * combined in a fixed order, so results are bitwise reproducible.  A plan's scratch serves one
 * multiply at a time: launches that use the same plan must be ordered (same stream, or events). */
MPS_API int mps_spmm(mps_plan *plan, const int32_t *d_row_ptr, const int32_t *d_col_idx, const void *d_val,
             const void *d_B, void *d_C, void *stream);

/* The caller pattern the reference's kernels gesture at with their on-the-fly `deg_i * deg_j` value
 * (src/MergePathSpMM.cu:436-441,450,459): C[i,:] = row_scale[i] * sum_k col_scale[col[k]] * B[col[k],:]
 * for the non-zeros k of row i - e.g. GCN's D^-1/2 (A+I) D^-1/2 X with both scales = degree^-1/2 - without
 * a stored value per non-zero.  The column factor is gathered per non-zero, the row factor multiplies the
 * finished row once.  Either scale may be NULL (= all ones), not both: with d_col_scale == NULL and B already
 * multiplied by the column factor where it was produced, the multiply reads no per-non-zero value at all,
 * which is the fastest form.  fp32 plans only; scales are fp32 device arrays (n_rows and n_cols entries). */
MPS_API int mps_spmm_scaled(mps_plan *plan, const int32_t *d_row_ptr, const int32_t *d_col_idx,
                    const float *d_row_scale, const float *d_col_scale, const void *d_B, void *d_C, void *stream);

/* Waits for the stream and returns MPS_ERR_DEVICE if any kernel of this plan gave up a wait (a tile block whose
 * staged window did not arrive in time fetches it again with plain loads and finishes its rows, but the call
 * counts as failed: treat C as undefined until this returns MPS_OK). */
MPS_API int mps_plan_sync_check(mps_plan *plan, void *stream);

/* Facts about a plan: what[0]=n_chunks what[1]=items_per_chunk what[2]=chunks_per_tile
 * what[3]=n_tiles what[4]=lanes_per_chunk what[5]=elements_per_lane what[6]=unroll
 * what[7]=shared_bytes_per_block what[8]=long_rows what[9]=effective threads_per_warp
 * what[10]=kernels per mps_spmm call what[11]=long_chain threshold what[12]=chunks_per_unit
 * what[13]=units_per_tile what[14]=threads per tile block what[15]=very_long chain threshold. */
MPS_API int mps_plan_info(const mps_plan *plan, int64_t what[16]);

/* The layout behind those facts in merge items (no reference counterpart): what[0]=merge items per unit
 * (one lane group's walk), what[1]=units per tile, what[2]=merge items per tile, what[3]=n_tiles,
 * what[4]=units per reference chunk (1 unless `cost` asks for chunks longer than a tile should stage: then a
 * unit is the what[4]-th part of a chunk and what[0] = ceil(items_per_chunk / what[4]); any `cost` the
 * reference's command line accepts is therefore accepted here), what[5]=shared bytes per block,
 * what[6]=column slabs, what[7]=1 when the tile kernel performs the cross-tile fix-up itself,
 * what[8]=lane groups that share a unit (1, or 32 / lanes_per_chunk when a whole warp walks a unit, see
 * mps_plan_set_walk), what[9..11]=0 (reserved).
 * mps_layout_query gives the same numbers for a shape without a plan or a CUDA device (the automatic
 * layout for 148 SMs). */
MPS_API int mps_plan_layout(const mps_plan *plan, int64_t what[12]);
MPS_API int mps_layout_query(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost, int64_t what[12]);

/* How a unit is walked (no reference counterpart in form; in substance this is the reference's choice of
 * threads_per_warp, src/MergePathSpMM.cu:224-243: how many chunks a warp takes at once).  0: every group of
 * lanes_per_chunk lanes walks a unit of its own (a warp at dim 16 walks eight units side by side).  1: the whole warp
 * walks one unit - its lane groups take consecutive non-zeros, keep partial sums of the row in progress and combine
 * them with xor-shuffles in a fixed tree at every row end - so no lane idles where neighbouring units would end
 * their rows at different places.  -1: automatic.  Full-width lanes (dim a multiple of 4 fp32 / 8 fp16, fewer than 32
 * lanes per row; not the narrow fp16 rows of four columns per lane), 64-thread blocks and unroll 8 only; elsewhere the setting is ignored.  Changes the summation order
 * (still fixed and reproducible); call before mps_plan_partition. */
MPS_API int mps_plan_set_walk(mps_plan *plan, int32_t warp_per_unit);

/* Per-kernel timing (no reference counterpart; the reference is timed from outside with nvprof,
 * README.md:41-46): while enabled, every mps_spmm records a CUDA event pair around its tile
 * kernel on the launching stream.  mps_plan_profile_read waits for the stream and returns the
 * summed tile-kernel time in milliseconds and the number of launches since the last read. */
MPS_API int mps_plan_profile(mps_plan *plan, int enable);
MPS_API int mps_plan_profile_read(mps_plan *plan, void *stream, double *tile_ms, int32_t *launches);

/* Algorithmic bytes of one SpMM: 4(N+1) + nnz(4 + s_val) + nnz*dim*s + N*dim*s, s = 4 or 2;
 * has_val = 0 drops the value term. */
MPS_API int64_t mps_algorithmic_bytes(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int has_val);

/* Measures what this GPU can do with the multiply's access pattern (no reference counterpart): whole rows
 * of `row_bytes` (32..512, a power of two) fetched at random with 128-bit loads from a device table of
 * `table_rows` rows, about `gathers` of them in one launch after one warm-up launch, 1024 threads per SM with
 * eight loads in flight each.  *ms = the timed launch (CUDA events on `stream`), *gathered_bytes = the bytes it
 * fetched.  A table well inside the L2 gives the L2 -> SM gather rate, a table far larger than the L2 the
 * random-row rate of HBM; the multiply's gathered bytes per second belong beside these two, not beside a copy
 * bandwidth.  d_sink: 4 bytes per thread of the launch (148 SMs x 1024 x 4 bytes = 0.6 MB on a B200).
 * Allocates nothing but two events; blocking. */
MPS_API int mps_gather_probe(const void *d_table, int64_t table_rows, int32_t row_bytes, int64_t gathers, void *d_sink,
                     int64_t sink_bytes, void *stream, float *ms, int64_t *gathered_bytes);

/* The same fetch loop over the caller's own row numbers (no reference counterpart): d_index holds n_index row numbers
 * in [0, table_rows) - typically the multiply's col_idx with d_table = B - and every group of threads fetches a
 * contiguous run of them in order, as a lane group of the multiply walks its unit.  What this launch reaches is the
 * rate at which this GPU can deliver THIS stream of rows (its reuse, its L2 hit rate, its DRAM misses) to a kernel that
 * only fetches; the multiply's gathered bytes per second divided by it says how much the multiply's own work (staging,
 * fused multiply-adds, row ends) costs on top.  The indices are not checked. */
MPS_API int mps_gather_probe_stream(const void *d_table, int64_t table_rows, int32_t row_bytes, const int32_t *d_index,
                            int64_t n_index, void *d_sink, int64_t sink_bytes, void *stream, float *ms,
                            int64_t *gathered_bytes);

/* ------------------------------------------------------------------ host-buffer call ----- */

/* The whole reference program body on HOST buffers (src/MergePathSpMM.cu:187-267): upload A and
 * B, partition, multiply once, download C.  B has n_cols rows (n_cols = n_rows for the square
 * matrices of the file format; a row slab of a larger matrix has fewer rows than columns).
 * Device buffers live in a per-thread workspace that only grows, so repeated calls do not
 * reallocate.  Blocking.
 * The caller's arrays are validated on host threads before any kernel indexes by them (the reference
 * checks nothing, its helper :41-52 is never called): row_ptr[0] == 0, row_ptr non-decreasing,
 * row_ptr[n_rows] == nnz, every col_idx inside [0, n_cols) - else MPS_ERR_ARG naming the position.  row_ptr
 * is checked on the host; col_idx where each slab of it lands on the device, ahead of the multiply on the
 * same stream (an index outside B is replaced by 0 in the workspace copy before any kernel gathers by it,
 * and C is then meaningless), so the check costs the uploads nothing.  The uploads of row_ptr and B are queued
 * before the host check (nothing on the device reads row_ptr until the host has passed it); a call that fails
 * the check returns once they have drained.  A bad index is reported in preference
 * to any other failure of the call, also on a machine without a device (there the host scans col_idx). */
MPS_API int mps_spmm_host(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int dtype, int32_t cost,
                  int32_t threads_per_warp, const int32_t *row_ptr, const int32_t *col_idx,
                  const void *val, const void *B, void *C);

/* As mps_spmm_host, with B already in device memory (no reference counterpart: the reference is one
 * process on one GPU).  This is the call of a rank in a multi-process job: every rank uploads only its
 * share of B's rows into a full-size device buffer and an all-gather over NVLink (NCCL, the caller's)
 * completes it, instead of every rank pulling all of B over PCIe.  d_B must be whole once the work
 * queued so far on `b_ready_stream` has run; the call orders its multiplies behind that point and
 * uploads A meanwhile, so the gather overlaps the upload.  A (row_ptr, col_idx, val) and C stay host
 * buffers; validation as for mps_spmm_host. */
MPS_API int mps_spmm_host_resident_b(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int dtype, int32_t cost,
                             int32_t threads_per_warp, const int32_t *row_ptr, const int32_t *col_idx,
                             const void *val, const void *d_B, void *b_ready_stream, void *C);

/* mps_spmm_host for the product mps_spmm_scaled forms: C[i,:] = row_scale[i] * sum_k col_scale[col[k]] * B[col[k],:].
 * This is the shape of the reference program itself, which uploads one number per node (its `degrees`,
 * src/MergePathSpMM.cu:183-190,207-209) and forms every value in the kernel (:436-441) instead of storing one per
 * non-zero: the call moves n_rows + n_cols floats where mps_spmm_host moves nnz values (GCN on a graph of average
 * degree 32, dim 64: a quarter fewer bytes to the device).  fp32; row_scale has n_rows entries, col_scale n_cols,
 * either may be NULL (= all ones), not both.  Validation, slabs and workspace as for mps_spmm_host. */
MPS_API int mps_spmm_host_scaled(int32_t n_rows, int32_t n_cols, int32_t nnz, int32_t dim, int32_t cost,
                         int32_t threads_per_warp, const int32_t *row_ptr, const int32_t *col_idx,
                         const float *row_scale, const float *col_scale, const void *B, void *C);
MPS_API void mps_host_workspace_release(void);

/* ------------------------------------------------------------------ no-allocation call --- */

/* No counterpart in the reference.  For callers that are not allowed to allocate device memory
 * when they call (a plugin living inside a host framework's fixed arena, a process whose device
 * memory is fully committed at start-up, a loop that cannot afford cudaMalloc's device-wide
 * synchronisation): partition + multiply + check in one blocking call whose scratch is a fixed
 * array inside the library image instead of a plan's cudaMalloc'ed buffers.  Inputs and output are
 * the caller's device buffers as for mps_spmm; `cost`/`threads_per_warp` as for mps_plan_create.
 *
 * Limits: with T = tiles of the automatic layout (mps_plan_info what[3] of an equivalent plan),
 * T * column_slabs <= MPS_NOALLOC_MAX_TILES and T * dim <= MPS_NOALLOC_MAX_CARRY_FLOATS, else MPS_ERR_UNSUPPORTED
 * with the numbers in mps_last_error().  A tile holds about 1,088 merge items (rows + non-zeros),
 * so at dim 64 that is about 17 million merge items, at dim 128 about 9 million, at dim <= 32 about 35
 * million.  Every GPU that loads the library holds MPS_NOALLOC_SCRATCH_BYTES for this
 * array until the process exits.
 *
 * The array is shared by every call on a device: calls that overlap on the GPU race on it, so
 * issue them one after another.  The first call on each device looks up the array's address; make
 * that call before starting any stream capture.  Calls no cudaMalloc/cudaFree and no allocating
 * library routine. */
#define MPS_NOALLOC_MAX_TILES 32768
#define MPS_NOALLOC_MAX_CARRY_FLOATS (1u << 20)
#define MPS_NOALLOC_SCRATCH_BYTES (9u << 20)
MPS_API int mps_spmm_noalloc(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost,
                     int32_t threads_per_warp, const int32_t *d_row_ptr, const int32_t *d_col_idx,
                     const void *d_val, const void *d_B, void *d_C, void *stream);

/* ------------------------------------------------------------------ multi-GPU slabs ------ */

/* Row slabs of equal non-zero count for n_slabs devices (no reference counterpart - the
 * reference is single-GPU): bounds[g] = first row whose start offset is >= g*nnz/n_slabs,
 * bounds[0] = 0, bounds[n_slabs] = n_rows.  Host row_ptr. */
MPS_API int mps_slab_bounds(const int32_t *row_ptr, int32_t n_rows, int32_t n_slabs, int32_t *bounds);

/* As mps_slab_bounds, but equalising weighted merge items, non-zeros + row_weight * rows:
 * bounds[g] = first row r with row_ptr[r] + row_weight*r >= g*(nnz + row_weight*n_rows)/n_slabs.
 * A slab of many short rows writes far more of C (and ends far more rows) than a slab of few long
 * ones with the same non-zero count; row_weight = 1 is the merge path's own cost measure,
 * larger values charge a row end more than a gathered non-zero.  row_weight >= 0. */
MPS_API int mps_slab_bounds_items(const int32_t *row_ptr, int32_t n_rows, int32_t n_slabs, int32_t row_weight,
                          int32_t *bounds);

/* Slab g of a host CSR with row_ptr rebased to 0: writes row1 - row0 + 1 entries. */
MPS_API int mps_slab_rebase(const int32_t *row_ptr, int32_t row0, int32_t row1, int32_t *out_row_ptr);

/* ------------------------------------------------------------------ multi-GPU driver ----- */

/* Single-process driver over n_gpus devices of one node (no reference counterpart).  create: cuts
 * the HOST CSR into row slabs of equal (nnz + 4*rows), uploads slab g to devices[g] (NULL = 0..n-1),
 * plans and partitions it there, and allocates on every device a full copy of B and a full-height C.  The host
 * arrays are validated first (as in mps_spmm_host: MPS_ERR_ARG for a decreasing row_ptr or a column index
 * outside [0, n_cols), before any device is touched).
 * set_b: replicates a host B (n_cols x dim): with NCCL at hand and every slab on a device of its own each device
 * uploads 1/n_gpus of B's rows and one in-place all-gather over NVLink completes every copy (B crosses PCIe once
 * in total, not once per device); otherwise every device uploads all of it.  spmm: `repeat` multiplies on all devices at once, each
 * into its own rows of its C; *ms_spmm = time per multiply, the maximum over devices (CUDA events).
 * gather_c != 0 then makes every device's C complete with one grouped NCCL broadcast per slab over
 * NVLink (*ms_gather); NCCL is loaded on first use, and only this option needs it.  get_c: from_gpu
 * < 0 collects every slab from the device that computed it, otherwise copies the whole C that
 * device `from_gpu` holds.  One host thread drives all devices; the calls wait for completion. */
typedef struct mps_multi mps_multi;
MPS_API int mps_multi_create(int32_t n_gpus, const int32_t *devices, int32_t n_rows, int32_t n_cols, int32_t dim,
                     int dtype, int32_t cost, int32_t threads_per_warp, const int32_t *row_ptr,
                     const int32_t *col_idx, const void *val, mps_multi **out);
MPS_API void mps_multi_destroy(mps_multi *m);
MPS_API int mps_multi_slab(const mps_multi *m, int32_t g, int32_t *device, int32_t *row0, int32_t *row1, int32_t *nnz,
                   void **d_C);
MPS_API int mps_multi_set_b(mps_multi *m, const void *host_B);
MPS_API int mps_multi_spmm(mps_multi *m, int32_t repeat, int32_t gather_c, float *ms_spmm, float *ms_gather);
MPS_API int mps_multi_get_c(mps_multi *m, void *host_C, int32_t from_gpu);

#ifdef __cplusplus
}
#endif
#endif /* MPS_B200_H */
