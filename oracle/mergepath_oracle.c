/*
 * CPU oracle for the merge-path CSR SpMM hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so that tests, the smoke check and the bench's
 * CPU-baseline leg have an independent answer to compare the CUDA path with.
 *
 * Parity status: PINNED.  The partition / schedule restatement below is
 * checked (tests/test_oracle_golden.py) against vectors produced by the
 * reference's own host functions MergePathSearch and generate_mp_sched
 * (src/MergePathSpMM.cu:280-385), compiled unmodified from the reference tree
 * by oracle/Makefile into oracle/_ref/, and committed under tests/golden/.
 * The reference ships no tests or golden vectors of its own.
 *
 * Sections
 *   1. merge-path search, chunk count, coordinates     (ref :138-139, :280-297)
 *   2. the six-array schedule incl. its sentinel quirk (ref :300-385)
 *   3. sequential emulation of the reference kernels   (ref :408-479, :503-573)
 *   4. fp64 CSR loop (numeric ground truth) and an OpenMP fp32 CSR loop
 *      (the timed host baseline; the reference has no CPU SpMM)
 *   5. CPU model of the tiled kernel's summation order (bit-exact target for
 *      the CUDA kernels of this repository; no reference counterpart)
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/oracle.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }
static inline int64_t lmin(int64_t a, int64_t b) { return a < b ? a : b; }

/* ------------------------------------------------------------------ 1 -- */

/* Number of chunks ("threads" in the reference's wording) for a given cost:
 * (N+1+nnz-1)/cost in C integer division, never below 1024.
 * Follows src/MergePathSpMM.cu:138-139. */
ORC_API int orc_chunk_count(int n_rows, int nnz, int cost) {
    int64_t p = ((int64_t)n_rows + 1 + (int64_t)nnz - 1) / (int64_t)cost;
    if (p < 1024) p = 1024;
    return (int)p;
}

/* Items per chunk: ceil((N+1+nnz)/P).  Follows src/MergePathSpMM.cu:327-328. */
ORC_API int orc_items_per_chunk(int n_rows, int nnz, int n_chunks) {
    int64_t total = (int64_t)n_rows + 1 + (int64_t)nnz;
    return (int)((total + n_chunks - 1) / n_chunks);
}

/* One diagonal of the merge of list A = row_ptr[0..N] (all N+1 entries, so
 * row_ptr[0] is a merge item) with list B = 0,1,..,nnz-1.  Ties take the
 * row_ptr entry first.  x = row_ptr entries consumed, y = non-zeros consumed.
 * Follows src/MergePathSpMM.cu:280-297; the reference materialises list B as
 * an identity array, here B[k] = k is used directly.  `n_list_a` is what the
 * reference passes as num_rows, i.e. N+1 (:333-334). */
ORC_API void orc_merge_path_search(int64_t diagonal, const int *row_ptr,
                                   int n_list_a, int nnz, int *out_x, int *out_y) {
    int64_t lo = diagonal - nnz;
    if (lo < 0) lo = 0;
    int64_t hi = lmin(diagonal, n_list_a);
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if ((int64_t)row_ptr[mid] <= diagonal - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    *out_x = (int)lmin(lo, n_list_a);
    *out_y = (int)(diagonal - lo);
}

/* Coordinates of all P+1 chunk boundaries: diagonal t = min(ipt*t, total).
 * xy is int[2*(P+1)], interleaved (x,y). */
ORC_API void orc_partition(const int *row_ptr, int n_rows, int nnz, int n_chunks, int *xy) {
    int64_t total = (int64_t)n_rows + 1 + nnz;
    int64_t ipt = (total + n_chunks - 1) / n_chunks;
    for (int64_t t = 0; t <= n_chunks; ++t) {
        int64_t d = lmin(ipt * t, total);
        orc_merge_path_search(d, row_ptr, n_rows + 1, nnz, &xy[2 * t], &xy[2 * t + 1]);
    }
}

/* ------------------------------------------------------------------ 2 -- */

/* The reference's per-chunk schedule, six int[P] arrays in the order the
 * reference returns them (:380-383):
 *   head_at, head_len, tail_at, tail_len, first_row, last_row
 * (the reference's feature_start, feature_start_num, feature_end,
 * feature_end_num, start_row, end_row).  Zero doubles as "no partial row",
 * which loses a tail partial that begins at non-zero 0 (:365-369) - kept. */
ORC_API void orc_schedule(const int *row_ptr, int n_rows, int nnz, int n_chunks,
                          int *head_at, int *head_len, int *tail_at, int *tail_len,
                          int *first_row, int *last_row) {
    int64_t total = (int64_t)n_rows + 1 + nnz;
    int64_t ipt = (total + n_chunks - 1) / n_chunks;
    for (int64_t t = 0; t < n_chunks; ++t) {
        int64_t d0 = lmin(ipt * t, total), d1 = lmin(d0 + ipt, total);
        int x0, y0, x1, y1;
        orc_merge_path_search(d0, row_ptr, n_rows + 1, nnz, &x0, &y0);
        orc_merge_path_search(d1, row_ptr, n_rows + 1, nnz, &x1, &y1);
        int first = imax(x0 - 1, 0);
        int last = x1 - 1;
        int h_at = (row_ptr[first] == y0 || t == 0) ? 0 : y0;
        int t_at = (row_ptr[last] == y1) ? 0 : y1;
        int h_len = 0, t_len = 0;
        if (h_at != 0) {
            if (first == last && t_at != 0) { h_len = t_at - h_at; t_at = 0; }
            else h_len = row_ptr[first + 1] - h_at;
        }
        if (t_at != 0) { t_len = t_at - row_ptr[last]; t_at = row_ptr[last]; }
        head_at[t] = h_at; head_len[t] = h_len;
        tail_at[t] = t_at; tail_len[t] = t_len;
        first_row[t] = first; last_row[t] = last;
    }
}

/* ------------------------------------------------------------------ 3 -- */

/* Sequential emulation of the reference kernels: chunk after chunk, one
 * column at a time, atomics replaced by "+=" on a zero-initialised C.  The
 * non-zero's value is float(deg[i])*float(deg[j]); the tail partial uses a
 * source factor of 1 (:468, :562).  Product and sum are separate roundings
 * (__fmaf_rn(a,b,0) then +=).  With deg == 1 everywhere this is a unit-valued
 * SpMM except for what the zero sentinel drops.  Follows :408-479. */
ORC_API void orc_ref_kernel_emulate_f32(const int *row_ptr, const int *col, const int *deg,
                                        const float *B, float *C, int n_rows, int dim,
                                        int n_chunks, const int *head_at, const int *head_len,
                                        const int *tail_at, const int *tail_len,
                                        const int *first_row, const int *last_row) {
    (void)n_rows;
    for (int t = 0; t < n_chunks; ++t) {
        for (int j = 0; j < dim; ++j) {
            int row = first_row[t], stop = last_row[t];
            if (head_at[t] != 0) {
                float src = (float)deg[row], part = 0.0f;
                for (int q = 0; q < head_len[t]; ++q) {
                    int c = col[head_at[t] + q];
                    float w = src * (float)deg[c];
                    float prod = w * B[(size_t)c * dim + j];
                    part += prod;
                }
                C[(size_t)row * dim + j] += part;
                ++row;
            }
            for (; row < stop; ++row) {
                float src = (float)deg[row], acc = 0.0f;
                for (int k = row_ptr[row]; k < row_ptr[row + 1]; ++k) {
                    int c = col[k];
                    float w = src * (float)deg[c];
                    float prod = w * B[(size_t)c * dim + j];
                    acc += prod;
                }
                C[(size_t)row * dim + j] = acc;
            }
            if (tail_at[t] != 0) {
                float part = 0.0f;
                for (int q = 0; q < tail_len[t]; ++q) {
                    int c = col[tail_at[t] + q];
                    float w = 1.0f * (float)deg[c];
                    float prod = w * B[(size_t)c * dim + j];
                    part += prod;
                }
                C[(size_t)stop * dim + j] += part;
            }
        }
    }
}

/* ------------------------------------------------------------------ 4 -- */

static inline float half_bits_to_float(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t float_to_half_bits(float f) {
    _Float16 v = (_Float16)f; /* round to nearest even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

/* Ground truth: C = A*B accumulated in fp64.  val == NULL means all ones.
 * is_half selects fp16 storage for val and B (bit patterns in uint16). */
ORC_API void orc_spmm_f64(const int *row_ptr, const int *col, const void *val, const void *B,
                          double *C, int n_rows, int dim, int is_half) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int i = 0; i < n_rows; ++i) {
        double *out = C + (size_t)i * dim;
        for (int j = 0; j < dim; ++j) out[j] = 0.0;
        for (int k = row_ptr[i]; k < row_ptr[i + 1]; ++k) {
            size_t base = (size_t)col[k] * dim;
            if (is_half) {
                double a = val ? (double)half_bits_to_float(((const uint16_t *)val)[k]) : 1.0;
                const uint16_t *b = (const uint16_t *)B + base;
                for (int j = 0; j < dim; ++j) out[j] += a * (double)half_bits_to_float(b[j]);
            } else {
                double a = val ? (double)((const float *)val)[k] : 1.0;
                const float *b = (const float *)B + base;
                for (int j = 0; j < dim; ++j) out[j] += a * (double)b[j];
            }
        }
    }
}

/* Scale of each output element, sum_k |a_ik * b_kj| in fp64: the denominator
 * of the scale-aware error that summation-order noise is measured against. */
ORC_API void orc_spmm_abs_f64(const int *row_ptr, const int *col, const void *val, const void *B,
                              double *S, int n_rows, int dim, int is_half) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int i = 0; i < n_rows; ++i) {
        double *out = S + (size_t)i * dim;
        for (int j = 0; j < dim; ++j) out[j] = 0.0;
        for (int k = row_ptr[i]; k < row_ptr[i + 1]; ++k) {
            size_t base = (size_t)col[k] * dim;
            if (is_half) {
                double a = val ? (double)half_bits_to_float(((const uint16_t *)val)[k]) : 1.0;
                const uint16_t *b = (const uint16_t *)B + base;
                for (int j = 0; j < dim; ++j) out[j] += fabs(a * (double)half_bits_to_float(b[j]));
            } else {
                double a = val ? (double)((const float *)val)[k] : 1.0;
                const float *b = (const float *)B + base;
                for (int j = 0; j < dim; ++j) out[j] += fabs(a * (double)b[j]);
            }
        }
    }
}

/* Host baseline: fp32 CSR SpMM, rows split over threads at equal non-zero
 * counts, inner loop over the feature dimension (vectorisable).  Returns the
 * number of threads used.  The reference has no CPU SpMM; this is the
 * "multithreaded host CSR loop" its GPU numbers are reported beside. */
ORC_API int orc_spmm_f32_omp(const int *row_ptr, const int *col, const float *val, const float *B,
                             float *C, int n_rows, int dim, int n_threads) {
    int used = 1;
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
    used = n_threads;
#else
    n_threads = 1;
#endif
    int64_t nnz = row_ptr[n_rows];
#pragma omp parallel num_threads(n_threads)
    {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        /* first row whose start offset reaches this thread's share of nnz */
        int64_t want_lo = nnz * tid / n_threads, want_hi = nnz * (tid + 1) / n_threads;
        int lo = 0, hi = n_rows;
        while (lo < hi) { int m = (lo + hi) >> 1; if (row_ptr[m] < want_lo) lo = m + 1; else hi = m; }
        int r0 = (tid == 0) ? 0 : lo;
        lo = 0; hi = n_rows;
        while (lo < hi) { int m = (lo + hi) >> 1; if (row_ptr[m] < want_hi) lo = m + 1; else hi = m; }
        int r1 = (tid == n_threads - 1) ? n_rows : lo;
        for (int i = r0; i < r1; ++i) {
            float *restrict out = C + (size_t)i * dim;
            for (int j = 0; j < dim; ++j) out[j] = 0.0f;
            for (int k = row_ptr[i]; k < row_ptr[i + 1]; ++k) {
                const float a = val ? val[k] : 1.0f;
                const float *restrict b = B + (size_t)col[k] * dim;
#pragma omp simd
                for (int j = 0; j < dim; ++j) out[j] += a * b[j];
            }
        }
    }
    return used;
}

/* ------------------------------------------------------------------ 5 -- */

/* CPU model of the tiled CUDA kernels of this repository: the same unit
 * boundaries, the same fused multiply-adds in the same order, the same
 * fixed-order fix-up inside a tile and across tiles, so the GPU result must
 * equal it bit for bit.
 *
 *   chunk  c : merge items [ipt*c, ipt*(c+1)), one reference chunk
 *   unit     : unit_items consecutive merge items (cpu whole chunks, or the k-th
 *              part of a chunk when `cost` asks for chunks longer than a tile),
 *              walked in order by one lane group with one running accumulator,
 *              acc = fmaf(a, b, acc)
 *   tile   t : nu consecutive units; tiles cover [0, N+1+nnz) and no more
 *   a row that ends inside a unit is stored directly unless it began in an
 *   earlier unit, in which case the unit's share is its "head"; what is left
 *   at the unit's end is its "carry".
 *   in-tile fix-up  : row = 0 + carry[s] + .. + carry[u-1] + head[u]
 *   cross-tile      : row = 0 + tcarry[s] + .. + tcarry[t-1] + thead[t];
 *                     chains longer than long_chain use 16 interleaved
 *                     strands, strand g = sum of tcarry[s+g], tcarry[s+g+16]..
 *                     then 0 + strand[0] + .. + strand[15] + thead[t].
 * is_half: val/B/C hold fp16 bit patterns, all sums stay in fp32 and C is
 * rounded once.  val == NULL means all ones.  Returns 0, or -1 on bad args. */
typedef struct {
    const int *rp, *col;
    const void *val, *B;
    void *C;
    int dim, is_half;
    const float *row_scale, *col_scale; /* scaled variant: value(i,j) = row_scale[i]*col_scale[j]; NULL otherwise */
} model_io;

static inline float model_val(const model_io *io, int k) {
    if (io->col_scale) return io->col_scale[io->col[k]];
    if (!io->val) return 1.0f;
    return io->is_half ? half_bits_to_float(((const uint16_t *)io->val)[k]) : ((const float *)io->val)[k];
}
static inline float model_b(const model_io *io, int c, int j) {
    size_t at = (size_t)c * io->dim + j;
    return io->is_half ? half_bits_to_float(((const uint16_t *)io->B)[at]) : ((const float *)io->B)[at];
}
static inline void model_store(const model_io *io, int row, const float *v_in) {
    size_t at = (size_t)row * io->dim;
    float scaled[1024];
    const float *v = v_in;
    if (io->row_scale) { /* the row factor multiplies the finished row once */
        for (int j = 0; j < io->dim; ++j) scaled[j] = v_in[j] * io->row_scale[row];
        v = scaled;
    }
    if (io->is_half) for (int j = 0; j < io->dim; ++j) ((uint16_t *)io->C)[at + j] = float_to_half_bits(v[j]);
    else memcpy((float *)io->C + at, v, sizeof(float) * io->dim);
}

/* acc <- part[0..groups) added pairwise, level by level (distance 1, 2, 4, ..) */
#define MODEL_TREE(dst)                                                                                  \
    do {                                                                                                 \
        memcpy(tree, part, sizeof(float) * (size_t)groups * dim);                                        \
        for (int off_ = 1; off_ < groups; off_ <<= 1)                                                    \
            for (int s_ = 0; s_ < groups; s_ += 2 * off_)                                                \
                for (int j_ = 0; j_ < dim; ++j_) tree[(size_t)s_ * dim + j_] += tree[(size_t)(s_ + off_) * dim + j_]; \
        memcpy(dst, tree, sizeof(float) * dim);                                                          \
    } while (0)

/* unit_items: merge items per unit; nu: units per tile.  The tiles are independent until the cross-tile fix-up,
 * so they are walked by all host threads (every thread owns its scratch; each row of C, each tcarry / thead row is
 * written by exactly one tile), which lets the model check a full-size product in seconds. */
static int tile_model_items(const int *row_ptr, const int *col, const void *val, const float *row_scale, const float *col_scale,
                            const void *B, void *C, int n_rows, int nnz, int dim, int is_half, int64_t unit_items, int nu,
                            int long_chain, int groups) {
    if (unit_items < 1 || nu < 1 || dim < 1 || dim > 1024) return -1;
    if (!(groups == 1 || groups == 2 || groups == 4 || groups == 8 || groups == 16)) return -1;
    model_io io = {row_ptr, col, val, B, C, dim, is_half, row_scale, col_scale};
    const int64_t total = (int64_t)n_rows + 1 + nnz;
    const int64_t tile_items = unit_items * nu;
    int64_t T64 = (total + tile_items - 1) / tile_items;
    if (T64 < 1) T64 = 1;
    if (T64 > 0x7fffffff) return -1;
    const int T = (int)T64;
    int *tx = malloc(sizeof(int) * ((size_t)T + 1)), *ty = malloc(sizeof(int) * ((size_t)T + 1));
    float *tcarry = calloc((size_t)T * dim, sizeof(float));
    float *thead = calloc((size_t)T * dim, sizeof(float));
    if (!tx || !ty || !tcarry || !thead) { free(tx); free(ty); free(tcarry); free(thead); return -1; }

#pragma omp parallel for schedule(static)
    for (int t = 0; t <= T; ++t)
        orc_merge_path_search(lmin(tile_items * (int64_t)t, total), row_ptr, n_rows + 1, nnz, &tx[t], &ty[t]);

#pragma omp parallel
    {
        int *fx = malloc(sizeof(int) * (nu + 1)), *fy = malloc(sizeof(int) * (nu + 1));
        float *carry = malloc(sizeof(float) * (size_t)nu * dim);
        float *head = malloc(sizeof(float) * (size_t)nu * dim);
        char *has_head = malloc(nu);
        float *acc = malloc(sizeof(float) * dim), *sum = malloc(sizeof(float) * dim);
        float *part = malloc(sizeof(float) * (size_t)groups * dim), *tree = malloc(sizeof(float) * (size_t)groups * dim);
#pragma omp for schedule(dynamic, 64)
        for (int t = 0; t < T; ++t) {
            for (int u = 0; u <= nu; ++u)
                orc_merge_path_search(lmin(tile_items * (int64_t)t + unit_items * (int64_t)u, total), row_ptr, n_rows + 1, nnz, &fx[u], &fy[u]);
            for (int u = 0; u < nu; ++u) {
                const int x0 = fx[u], y0 = fy[u], x1 = fx[u + 1], y1 = fy[u + 1];
                const int cont = x0 >= 1 && y0 > row_ptr[x0 - 1];
                int x = x0, first = 1;
                has_head[u] = 0;
                /* `groups` lane groups share the unit: group s folds the non-zeros y0 + s, y0 + s + groups, .. of the
                 * row in progress into part[s]; at a row end the partial sums are added in a fixed tree (neighbours
                 * first: s with s ^ 1, then ^ 2, ..), which is what the kernel's xor-shuffles compute.  groups == 1 is
                 * the plain walk: one running sum. */
                for (int j = 0; j < groups * dim; ++j) part[j] = 0.0f;
                for (int k = y0; k <= y1; ++k) {
                    /* consume every marker that precedes non-zero k (all that are left when k == y1) */
                    while (x < x1 && (k == y1 || row_ptr[x] <= k)) {
                        if (x >= 1) {
                            MODEL_TREE(acc);
                            if (first && cont) { memcpy(head + (size_t)u * dim, acc, sizeof(float) * dim); has_head[u] = 1; }
                            else model_store(&io, x - 1, acc);
                            first = 0;
                            for (int j = 0; j < groups * dim; ++j) part[j] = 0.0f;
                        }
                        ++x;
                    }
                    if (k == y1) break;
                    const float a = model_val(&io, k);
                    const int cc = col[k];
                    float *restrict pacc = part + (size_t)((k - y0) % groups) * dim;
                    if (!is_half) { /* same fused multiply-adds, read straight from the fp32 row */
                        const float *restrict b = (const float *)B + (size_t)cc * dim;
#pragma omp simd
                        for (int j = 0; j < dim; ++j) pacc[j] = fmaf(a, b[j], pacc[j]);
                    } else {
                        for (int j = 0; j < dim; ++j) pacc[j] = fmaf(a, model_b(&io, cc, j), pacc[j]);
                    }
                }
                MODEL_TREE(acc);
                memcpy(carry + (size_t)u * dim, acc, sizeof(float) * dim);
            }
            /* in-tile fix-up */
            for (int u = 0; u < nu; ++u) {
                if (!has_head[u]) continue;
                int s = u;
                while (s > 0 && fx[s] == fx[u]) --s;
                const int from_prev = fx[0] == fx[u] && ty[t] > row_ptr[tx[t] - 1];
                for (int j = 0; j < dim; ++j) sum[j] = 0.0f;
                for (int q = s; q < u; ++q) for (int j = 0; j < dim; ++j) sum[j] += carry[(size_t)q * dim + j];
                for (int j = 0; j < dim; ++j) sum[j] += head[(size_t)u * dim + j];
                if (from_prev) memcpy(thead + (size_t)t * dim, sum, sizeof(float) * dim);
                else model_store(&io, fx[u] - 1, sum);
            }
            {
                int s = nu;
                while (s > 0 && fx[s] == fx[nu]) --s;
                for (int j = 0; j < dim; ++j) sum[j] = 0.0f;
                for (int q = s; q < nu; ++q) for (int j = 0; j < dim; ++j) sum[j] += carry[(size_t)q * dim + j];
                memcpy(tcarry + (size_t)t * dim, sum, sizeof(float) * dim);
            }
        }
        free(fx); free(fy); free(carry); free(head); free(has_head); free(acc); free(sum); free(part); free(tree);
    }
    /* cross-tile fix-up */
#pragma omp parallel
    {
        float *sum = malloc(sizeof(float) * dim);
        float *strand = malloc(sizeof(float) * 16 * dim);
#pragma omp for schedule(dynamic, 256)
        for (int t = 1; t < T; ++t) {
            if (!(tx[t] >= 1 && tx[t + 1] > tx[t] && ty[t] > row_ptr[tx[t] - 1])) continue;
            int f = t;
            while (f > 0 && tx[f - 1] == tx[t]) --f; /* first tile that starts in this row */
            const int s = f - 1, len = t - s;
            for (int j = 0; j < dim; ++j) sum[j] = 0.0f;
            if (len > long_chain) {
                for (int g = 0; g < 16; ++g) {
                    float *sg = strand + (size_t)g * dim;
                    for (int j = 0; j < dim; ++j) sg[j] = 0.0f;
                    for (int q = s + g; q < t; q += 16) for (int j = 0; j < dim; ++j) sg[j] += tcarry[(size_t)q * dim + j];
                }
                for (int g = 0; g < 16; ++g) for (int j = 0; j < dim; ++j) sum[j] += strand[(size_t)g * dim + j];
            } else {
                for (int q = s; q < t; ++q) for (int j = 0; j < dim; ++j) sum[j] += tcarry[(size_t)q * dim + j];
            }
            for (int j = 0; j < dim; ++j) sum[j] += thead[(size_t)t * dim + j];
            model_store(&io, tx[t] - 1, sum);
        }
        free(sum); free(strand);
    }
    free(tx); free(ty); free(tcarry); free(thead);
    return 0;
}

/* Layout given the way a whole-chunk plan reports it: nch chunks per tile, cpu chunks per unit, ipt from `cost`;
 * unit_items > 0 overrides cpu * ipt (sub-chunk units: a unit is a part of one chunk). */
static int tile_model_impl(const int *row_ptr, const int *col, const void *val, const float *row_scale, const float *col_scale,
                           const void *B, void *C, int n_rows, int nnz, int dim, int is_half, int cost, int nch, int cpu,
                           int long_chain, int64_t unit_items, int groups) {
    if (cost < 1 || nch < 1 || cpu < 1 || nch % cpu != 0) return -1;
    const int P = orc_chunk_count(n_rows, nnz, cost);
    const int64_t ipt = orc_items_per_chunk(n_rows, nnz, P);
    if (unit_items <= 0) unit_items = ipt * cpu;
    return tile_model_items(row_ptr, col, val, row_scale, col_scale, B, C, n_rows, nnz, dim, is_half, unit_items, nch / cpu, long_chain, groups);
}

ORC_API int orc_tile_model(const int *row_ptr, const int *col, const void *val, const void *B,
                           void *C, int n_rows, int nnz, int dim, int is_half, int cost,
                           int nch, int cpu, int long_chain, int64_t unit_items, int groups) {
    return tile_model_impl(row_ptr, col, val, NULL, NULL, B, C, n_rows, nnz, dim, is_half, cost, nch, cpu, long_chain, unit_items, groups);
}

/* The scaled variant (fp32): value(i,j) = row_scale[i] * col_scale[j]; the column factor enters each fused
 * multiply-add, the row factor multiplies the finished row once.  No reference counterpart beyond the gesture
 * at src/MergePathSpMM.cu:436-441. */
ORC_API int orc_tile_model_scaled(const int *row_ptr, const int *col, const float *row_scale, const float *col_scale,
                                  const float *B, float *C, int n_rows, int nnz, int dim, int cost, int nch, int cpu,
                                  int long_chain, int64_t unit_items) {
    return tile_model_impl(row_ptr, col, NULL, row_scale, col_scale, B, C, n_rows, nnz, dim, 0, cost, nch, cpu, long_chain, unit_items, 1);
}

/* Nnz-balanced row slabs for G devices: bounds[g] = first row whose start
 * offset is >= g*nnz/G (bounds[0] = 0, bounds[G] = N). */
ORC_API void orc_slab_bounds(const int *row_ptr, int n_rows, int n_slabs, int *bounds) {
    int64_t nnz = row_ptr[n_rows];
    bounds[0] = 0;
    for (int g = 1; g < n_slabs; ++g) {
        int64_t want = nnz * g / n_slabs;
        int lo = 0, hi = n_rows;
        while (lo < hi) { int m = (lo + hi) >> 1; if (row_ptr[m] < want) lo = m + 1; else hi = m; }
        bounds[g] = lo;
    }
    bounds[n_slabs] = n_rows;
}
