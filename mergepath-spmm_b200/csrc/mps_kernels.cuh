// Device code of the B200 merge-path CSR SpMM (sm_100a).
//
// Work decomposition (all diagonals are the reference's: chunk c covers merge items
// [ipt*c, ipt*(c+1)) of the merge of row_ptr[0..N] with 0..nnz-1, src/MergePathSpMM.cu:327-334):
//
//   tile   = `tile_items` consecutive merge items (a whole number of units), one thread block.  Its two boundary coordinates come from
//            the plan (searched once per row_ptr by partition_kernel); the block stages the tile's
//            row_ptr / col_idx / val windows into shared memory with bulk async copies that
//            complete on an mbarrier (no val window without stored values; a tile with more row ends
//            than the row_ptr window holds reads row_ptr from global memory).
//   unit   = `unit_items` consecutive merge items of the tile - a run of whole chunks, or the k-th part of one chunk
//            when the cost asks for chunks longer than a unit should be - walked in order by one group of GL
//            lanes (or by a whole warp, SPREAD); the unit boundaries are re-searched in the staged row_ptr window.
//            A lane owns VEC adjacent columns and gathers its part of every B row with one 128-bit
//            load, U (10) loads in flight before the first fused multiply-add; the accumulator stays in
//            registers across the chunk boundaries inside the unit.  Rows that end inside the unit
//            and began there are stored directly; a row that began earlier leaves its share as the
//            unit's "head", what is left at the unit's end is its "carry" (shared memory, fp32).
//   fix-up = inside the tile, in unit order, by the group that ended the row; across tiles by the
//            tile block whose contribution to the row arrives last (a counter per ending tile; nobody
//            waits), which adds the tiles' carry rows in tile order.  No atomics touch C, every row
//            of C is stored exactly once, sums are bitwise reproducible.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mps {

constexpr int kWarpsPerSm = 24;      // resident warps per SM the register allocation is held to (768 threads)
// ... for a kernel with U gathers in flight per thread: deeper batches hold more registers and trade resident warps for them
constexpr int warps_per_sm(int u) { return u <= 8 ? kWarpsPerSm : (u <= 10 ? 22 : 20); }
constexpr int kMaxBlock = 256;       // largest tile block (threads); 64 and 128 are the other sizes
constexpr int kStrands = 16;         // interleaved partial sums of the long-row fix-up
constexpr int kAlign = 8;            // staging windows start on multiples of 8 elements (>= 16 bytes)
constexpr int kWaitPolls = 1 << 22;  // bounded mbarrier wait

enum DeviceStatus : int { kDevOk = 0, kDevStageTimeout = 1 };

struct TileParams {
    const int *rp;
    const int *col;
    const void *val;  // nullptr: all ones
    const float *row_scale;  // scaled product (fp32 plans): value of non-zero (i, j) = row_scale[i] * col_scale[j], the row factor
    const float *col_scale;  // applied once, to the finished row; a nullptr factor is 1; both nullptr for the plain product
    const void *B;
    void *C;
    const int2 *tile_xy;  // n_tiles + 1 boundary coordinates, reference convention
    float *tcarry;        // n_tiles x dim
    float *thead;         // n_tiles x dim
    int *status;
    const int *consumer;  // per tile: the tile that ends the row this tile's carry belongs to, or -1
    const int *need;      // per tile: contributions its cross-tile fix-up waits for (0 = none)
    int *cnt;             // per (column slab, tile): contributions that have arrived; zero between launches
    int long_chain, very_long;
    int fused;  // 1: the tile kernel signals and performs the cross-tile fix-up itself; 0: fixup_kernel follows
    long long total;  // N + 1 + nnz
    int n_rows, nnz, dim;
    int unit_items, tile_items, n_tiles;  // merge items per unit, per tile (= units per tile x unit_items)
    int smem_bytes;                       // dynamic shared memory of this launch (no value window when val is nullptr)
    int bulk;  // 1: bulk async staging (needs 16-byte aligned rp/col/val)
};

// ---------------------------------------------------------------------------------------------
// merge-path search, reference convention (src/MergePathSpMM.cu:280-297 with list B = identity)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int2 merge_path_search_global(long long diag, const int *__restrict__ rp, int n_list_a, int nnz) {
    long long lo = diag - nnz;
    if (lo < 0) lo = 0;
    long long hi = diag < n_list_a ? diag : n_list_a;
    while (lo < hi) {
        long long mid = (lo + hi) >> 1;
        if ((long long)__ldg(rp + mid) <= diag - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    if (lo > n_list_a) lo = n_list_a;
    return make_int2((int)lo, (int)(diag - lo));
}

// count coordinates for diagonals min(step * t, total), t = 0..count-1
static __global__ void partition_kernel(const int *__restrict__ rp, int n_rows, int nnz, long long step, long long total,
                                 int count, int2 *__restrict__ out) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= count) return;
    long long d = step * (long long)t;
    if (d > total) d = total;
    out[t] = merge_path_search_global(d, rp, n_rows + 1, nnz);
}

// The reference's six per-chunk arrays (src/MergePathSpMM.cu:336-376), one thread per chunk.
static __global__ void schedule_kernel(const int *__restrict__ rp, int n_rows, int nnz, long long ipt, long long total,
                                int n_chunks, int *__restrict__ six) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_chunks) return;
    long long d0 = ipt * (long long)t;
    if (d0 > total) d0 = total;
    long long d1 = d0 + ipt;
    if (d1 > total) d1 = total;
    const int2 a = merge_path_search_global(d0, rp, n_rows + 1, nnz);
    const int2 b = merge_path_search_global(d1, rp, n_rows + 1, nnz);
    const int first = a.x > 0 ? a.x - 1 : 0;
    const int last = b.x - 1;
    const int rp_first = __ldg(rp + first), rp_last = __ldg(rp + last);
    int head_at = (rp_first == a.y || t == 0) ? 0 : a.y;
    int tail_at = (rp_last == b.y) ? 0 : b.y;
    int head_len = 0, tail_len = 0;
    if (head_at != 0) {
        if (first == last && tail_at != 0) { head_len = tail_at - head_at; tail_at = 0; }
        else head_len = __ldg(rp + first + 1) - head_at;
    }
    if (tail_at != 0) { tail_len = tail_at - rp_last; tail_at = rp_last; }  // 0 stays the "none" mark
    const size_t p = (size_t)n_chunks;
    six[t] = head_at;
    six[p + t] = head_len;
    six[2 * p + t] = tail_at;
    six[3 * p + t] = tail_len;
    six[4 * p + t] = first;
    six[5 * p + t] = last;
}

// ---------------------------------------------------------------------------------------------
// mbarrier / bulk-copy wrappers (1-D bulk copy global -> shared of this block, completion counted
// in bytes on an mbarrier; source, destination and size are multiples of 16 bytes)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// L2 policy for data that is read once (the CSR windows): evict first, so that the streamed arrays do
// not displace rows of B, which are the only data with reuse.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Returns false when the phase did not complete within the poll limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kWaitPolls; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 32) __nanosleep(64);
    }
    return false;
}

// ---------------------------------------------------------------------------------------------
// per-lane column vectors
// ---------------------------------------------------------------------------------------------
// Lane<T, VEC>: one lane's VEC adjacent columns.  `scalar` is how the non-zero's value is held while a
// batch is in flight: float for fp32 storage, the fp16 bit pattern for fp16 storage (the sm_100
// mixed-precision fma takes fp16 factors and an fp32 addend, which equals converting both factors to
// fp32 first - an fp16 x fp16 product is exact in fp32 - without spending instructions on conversion).
template <typename T, int VEC>
struct Lane;

__device__ __forceinline__ void fma_f32_f16x2(float &acc0, float &acc1, unsigned short a, uint32_t b_pair) {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "fma.rn.f32.f16 %0, %3, lo, %0;\n\t"
        "fma.rn.f32.f16 %1, %3, hi, %1;\n\t}"
        : "+f"(acc0), "+f"(acc1)
        : "r"(b_pair), "h"(a));
}

template <>
struct Lane<float, 4> {
    typedef float4 raw;
    typedef float scalar;
    static __device__ __forceinline__ scalar value(float v) { return v; }
    static __device__ __forceinline__ scalar from_float(float v) { return v; }
    static __device__ __forceinline__ scalar one() { return 1.0f; }
    static __device__ __forceinline__ raw load(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ void fma(float (&acc)[4], float a, const raw &b) {
        acc[0] = fmaf(a, b.x, acc[0]); acc[1] = fmaf(a, b.y, acc[1]);
        acc[2] = fmaf(a, b.z, acc[2]); acc[3] = fmaf(a, b.w, acc[3]);
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <>
struct Lane<float, 1> {
    typedef float raw;
    typedef float scalar;
    static __device__ __forceinline__ scalar value(float v) { return v; }
    static __device__ __forceinline__ scalar from_float(float v) { return v; }
    static __device__ __forceinline__ scalar one() { return 1.0f; }
    static __device__ __forceinline__ raw load(const float *p) { return __ldg(p); }
    static __device__ __forceinline__ void fma(float (&acc)[1], float a, const raw &b) { acc[0] = fmaf(a, b, acc[0]); }
    static __device__ __forceinline__ void store(float *p, const float (&v)[1]) { __stcs(p, v[0]); }
};
template <>
struct Lane<__half, 8> {
    typedef uint4 raw;
    typedef unsigned short scalar;
    static __device__ __forceinline__ scalar value(__half v) { return __half_as_ushort(v); }
    static __device__ __forceinline__ scalar from_float(float) { return (unsigned short)0x3C00; }  // scaled products are fp32-only
    static __device__ __forceinline__ scalar one() { return (unsigned short)0x3C00; }
    static __device__ __forceinline__ raw load(const __half *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
    static __device__ __forceinline__ void fma(float (&acc)[8], scalar a, const raw &b) {
        fma_f32_f16x2(acc[0], acc[1], a, b.x);
        fma_f32_f16x2(acc[2], acc[3], a, b.y);
        fma_f32_f16x2(acc[4], acc[5], a, b.z);
        fma_f32_f16x2(acc[6], acc[7], a, b.w);
    }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[8]) {
        uint4 o;
        __half2 *h = reinterpret_cast<__half2 *>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        __stcs(reinterpret_cast<uint4 *>(p), o);
    }
};
// Four fp16 columns per lane (one 64-bit load): narrow fp16 rows, where eight columns per lane would leave a warp with
// sixteen lane groups walking sixteen units.
template <>
struct Lane<__half, 4> {
    typedef uint2 raw;
    typedef unsigned short scalar;
    static __device__ __forceinline__ scalar value(__half v) { return __half_as_ushort(v); }
    static __device__ __forceinline__ scalar from_float(float) { return (unsigned short)0x3C00; }  // scaled products are fp32-only
    static __device__ __forceinline__ scalar one() { return (unsigned short)0x3C00; }
    static __device__ __forceinline__ raw load(const __half *p) { return __ldg(reinterpret_cast<const uint2 *>(p)); }
    static __device__ __forceinline__ void fma(float (&acc)[4], scalar a, const raw &b) {
        fma_f32_f16x2(acc[0], acc[1], a, b.x);
        fma_f32_f16x2(acc[2], acc[3], a, b.y);
    }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[4]) {
        uint2 o;
        __half2 *h = reinterpret_cast<__half2 *>(&o);
        h[0] = __floats2half2_rn(v[0], v[1]);
        h[1] = __floats2half2_rn(v[2], v[3]);
        __stcs(reinterpret_cast<uint2 *>(p), o);
    }
};
template <>
struct Lane<__half, 1> {
    typedef __half raw;
    typedef float scalar;
    static __device__ __forceinline__ scalar value(__half v) { return __half2float(v); }
    static __device__ __forceinline__ scalar from_float(float v) { return v; }
    static __device__ __forceinline__ scalar one() { return 1.0f; }
    static __device__ __forceinline__ raw load(const __half *p) { return __ldg(p); }
    static __device__ __forceinline__ void fma(float (&acc)[1], float a, const raw &b) { acc[0] = fmaf(a, __half2float(b), acc[0]); }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[1]) { *p = __float2half_rn(v[0]); }
};

template <int VEC>
__device__ __forceinline__ void smem_put(float *dst, const float (&v)[VEC]) {
    if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[i] = v[i];
    }
}
template <int VEC>
__device__ __forceinline__ void vec_add(float (&acc)[VEC], const float *src) {
    if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 f = *reinterpret_cast<const float4 *>(src + i);
            acc[i] += f.x; acc[i + 1] += f.y; acc[i + 2] += f.z; acc[i + 3] += f.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] += src[i];
    }
}
template <int VEC>
__device__ __forceinline__ void scale_by(float (&v)[VEC], float f) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] *= f;
}
template <int VEC>
__device__ __forceinline__ void gmem_put_f32(float *dst, const float (&v)[VEC]) {
    if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[i] = v[i];
    }
}

// Shared-memory layout of one tile block, shared by host (size) and device (offsets).
struct TileSmem {
    int off_fx, off_fy, off_rp, off_col, off_val, off_carry, off_head, bytes;
    __host__ __device__ static int up16(int v) { return (v + 15) & ~15; }
    // row_ptr entries the window holds: a quarter of the tile's merge items (rows of three non-zeros on average still
    // fit).  A tile with more markers than that reads row_ptr from global memory instead (shorter rows are rare, and
    // a row end touches row_ptr once); the shared memory this saves goes to the L1, which holds the gathers in flight.
    __host__ __device__ static int rp_entries(int tile_items) {
        const int q = tile_items / 4 < 64 ? 64 : tile_items / 4;
        return (q < tile_items ? q : tile_items) + 2 * kAlign + 8;
    }
    __host__ __device__ TileSmem(int n_units, int tile_items, int slab_cols, int elem_bytes) {
        const int win = tile_items + 2 * kAlign + 8;  // window plus alignment slack on both sides
        int o = 16;                                   // mbarrier
        off_fx = o; o = up16(o + 4 * (n_units + 1));
        off_fy = o; o = up16(o + 4 * (n_units + 1));
        off_rp = o; o = up16(o + 4 * rp_entries(tile_items));
        off_col = o; o = up16(o + 4 * win);
        off_val = o; o = up16(o + elem_bytes * win);
        off_carry = o; o = up16(o + 4 * n_units * slab_cols);
        off_head = o; o = up16(o + 4 * n_units * slab_cols);
        bytes = o;
    }
};

// Staging of elements [base, hi) of a global array of arr_len elements so that element i lands at
// s_dst[i - base]; base is a multiple of kAlign.  The 16-byte-granular part [base, bulk_end) goes
// through one bulk copy; the ragged end (at most the array's last kAlign-1 elements) is fetched
// with plain loads.
__device__ __forceinline__ long long bulk_end_of(long long base, long long hi, long long arr_len) {
    if (hi <= base) return base;
    long long e = (hi + kAlign - 1) & ~(long long)(kAlign - 1);
    const long long cap = arr_len & ~(long long)(kAlign - 1);
    if (e > cap) e = cap;
    return e > base ? e : base;
}
template <typename E>
__device__ __forceinline__ void stage_ragged(E *s_dst, const E *g_src, long long base, long long bulk_end, long long hi, int tid) {
    const long long i = bulk_end + tid;
    if (i < hi) s_dst[i - base] = g_src[i];
}

// ---------------------------------------------------------------------------------------------
// cross-tile fix-up helpers
// ---------------------------------------------------------------------------------------------
// Tile t needs a cross-tile fix-up when it ends (consumes a marker of) a row that began in an
// earlier tile.  Returns that row, and in `s` the first tile whose carry belongs to it.
__device__ __forceinline__ int fixup_candidate(const int2 *__restrict__ xy, const int *__restrict__ rp, int t, int &s) {
    const int2 a = __ldg(xy + t), b = __ldg(xy + t + 1);
    if (!(a.x >= 1 && b.x > a.x && a.y > __ldg(rp + a.x - 1))) return -1;
    // f = first tile that starts with x == a.x (tiles f..t start inside the row); f >= 1
    int lo = 0, hi = t;
    if (__ldg(xy + t - 1).x != a.x) lo = t;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(xy + mid).x < a.x) lo = mid + 1;
        else hi = mid;
    }
    s = lo - 1;
    return a.x - 1;
}

__device__ __forceinline__ void store_c(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_c(__half *p, float v) { *p = __float2half_rn(v); }

// Cross-tile fix-up of tile e, run by the tile block whose contribution arrived last: columns
// [col0, col1) of row x_e - 1 = 0 + tcarry[s] + .. + tcarry[e-1] + thead[e] in that order, or, for
// chains longer than long_chain, 16 interleaved strands (strand g = tcarry[s+g] + tcarry[s+g+16] + ..)
// added in strand order, then thead[e].  The operands were written by other blocks: read through L2.
template <typename T, int BLOCK>
__device__ __forceinline__ void block_fixup(const TileParams &p, int e, int chain, int col0, int col1, int tid) {
    const int row = __ldg(p.tile_xy + e).x - 1;
    const int s = e - chain;
    const size_t dim = (size_t)p.dim;
    for (int j = col0 + tid; j < col1; j += BLOCK) {
        float sum = 0.0f;
        if (chain <= p.long_chain) {
            for (int q = s; q < e; ++q) sum += __ldcg(p.tcarry + (size_t)q * dim + j);
        } else {
            float sg[kStrands];
#pragma unroll
            for (int g = 0; g < kStrands; ++g) sg[g] = 0.0f;
            int q = s;
            for (; q + kStrands <= e; q += kStrands) {
#pragma unroll
                for (int g = 0; g < kStrands; ++g) sg[g] += __ldcg(p.tcarry + (size_t)(q + g) * dim + j);
            }
#pragma unroll
            for (int g = 0; g < kStrands; ++g)
                if (q + g < e) sg[g] += __ldcg(p.tcarry + (size_t)(q + g) * dim + j);
#pragma unroll
            for (int g = 0; g < kStrands; ++g) sum += sg[g];
        }
        sum += __ldcg(p.thead + (size_t)e * dim + j);
        if (p.row_scale) sum *= __ldg(p.row_scale + row);
        store_c(static_cast<T *>(p.C) + (size_t)row * dim + j, sum);
    }
}

// ---------------------------------------------------------------------------------------------
// the tile kernel
// ---------------------------------------------------------------------------------------------
// One block = one tile = GPC units; unit u = `cpu` consecutive chunks walked by one group of GL
// lanes with the accumulator kept in registers across the chunk boundaries inside the unit.
// SCALED: the value of non-zero (i, j) is row_scale[i] * col_scale[j] instead of a stored value (a kernel of
// its own so that the plain product carries none of its selects).
// SPREAD: a unit is walked by a whole warp instead of one lane group.  The warp's 32/GL lane groups take consecutive
// non-zeros of the unit (group s the non-zeros at offset s, s + 32/GL, .. from the unit's start), each keeping a partial
// sum of the row in progress; at every row end the partial sums are combined with xor-shuffles in a fixed tree and the
// first group stores the row.  All lanes of a warp then follow the same rows, so none is masked off where the units of
// neighbouring groups would end their rows at different places - which is what costs at small dim, where a warp holds
// eight groups.
template <typename T, int VEC, int GL, int U, int BLOCK, bool SCALED, bool SPREAD = false>
__global__ void __launch_bounds__(BLOCK, warps_per_sm(U) * 32 / BLOCK) spmm_tile_kernel(const TileParams p) {
    constexpr int kBlock = BLOCK;
    constexpr int UL = SPREAD ? 32 : GL;   // lanes that walk one unit
    constexpr int G = UL / GL;             // lane groups per unit (1 unless SPREAD)
    constexpr int GPC = kBlock / UL;       // units per block
    constexpr int SLAB = GL * VEC;         // columns covered by one block
    extern __shared__ __align__(128) unsigned char smem[];
    const TileSmem L(GPC, p.tile_items, SLAB, p.val != nullptr ? (int)sizeof(T) : 0);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem);
    int *s_fx = reinterpret_cast<int *>(smem + L.off_fx);
    int *s_fy = reinterpret_cast<int *>(smem + L.off_fy);
    int *s_rp = reinterpret_cast<int *>(smem + L.off_rp);
    int *s_col = reinterpret_cast<int *>(smem + L.off_col);
    T *s_val = reinterpret_cast<T *>(smem + L.off_val);
    float *s_carry = reinterpret_cast<float *>(smem + L.off_carry);
    float *s_head = reinterpret_cast<float *>(smem + L.off_head);

    const int tid = threadIdx.x;
    const int g = tid / UL, l = tid % GL;   // unit of this thread, lane inside its group
    [[maybe_unused]] const int sg = (tid % UL) / GL;  // group inside the unit (SPREAD), else 0
    const int t = blockIdx.x;
    const int coff = blockIdx.y * SLAB + l * VEC;  // first column of this lane
    const bool active = coff < p.dim;
    const bool has_val = p.val != nullptr;
    [[maybe_unused]] const float *__restrict__ cs = p.col_scale, *__restrict__ rs = p.row_scale;
    const T *__restrict__ Bl = static_cast<const T *>(p.B) + coff;  // this lane's columns of B
    T *__restrict__ Cl = static_cast<T *>(p.C) + coff;
    const unsigned dim = (unsigned)p.dim;
    // one gathered row of B (this lane's columns)
    auto gather = [&](unsigned ci) -> typename Lane<T, VEC>::raw { return Lane<T, VEC>::load(Bl + (size_t)ci * dim); };

    const int2 c0 = __ldg(p.tile_xy + t), c1 = __ldg(p.tile_xy + t + 1);
    const int X0 = c0.x, Y0 = c0.y, X1 = c1.x, Y1 = c1.y;
    // row_ptr entries [max(X0-1,0), X1) and non-zeros [Y0, Y1) are what this tile touches
    const int rp_first = X0 > 0 ? X0 - 1 : 0;
    const int rp_base = rp_first & ~(kAlign - 1);
    const int y_base = Y0 & ~(kAlign - 1);

    // ---- stage the tile's windows ----
    const bool rp_staged = X1 - rp_base + kAlign <= TileSmem::rp_entries(p.tile_items);  // block-uniform (the copy rounds its end up)
    bool staged = false;
    if (p.bulk) {
        const uint32_t bar = smem_u32(s_bar);
        if (tid == 0) mbar_init(bar, 1);
        __syncthreads();
        const long long rp_be = rp_staged ? bulk_end_of(rp_base, X1, (long long)p.n_rows + 1) : (long long)rp_base;
        const long long y_be = bulk_end_of(y_base, Y1, p.nnz);
        if (tid == 0) {
            const uint32_t n_rp = (uint32_t)(rp_be - rp_base) * 4u;
            const uint32_t n_col = (uint32_t)(y_be - y_base) * 4u;
            const uint32_t n_val = has_val ? (uint32_t)(y_be - y_base) * (uint32_t)sizeof(T) : 0u;
            const uint64_t once = l2_evict_first_policy();
            mbar_arrive_expect(bar, n_rp + n_col + n_val);  // the single arrival the phase waits for
            if (n_rp) bulk_g2s(smem_u32(s_rp), p.rp + rp_base, n_rp, bar, once);
            if (n_col) bulk_g2s(smem_u32(s_col), p.col + y_base, n_col, bar, once);
            if (n_val) bulk_g2s(smem_u32(s_val), static_cast<const T *>(p.val) + y_base, n_val, bar, once);
        }
        if (rp_staged) stage_ragged<int>(s_rp, p.rp, rp_base, rp_be, X1, tid);
        stage_ragged<int>(s_col, p.col, y_base, y_be, Y1, tid);
        if (has_val) stage_ragged<T>(s_val, static_cast<const T *>(p.val), y_base, y_be, Y1, tid);
        // the first warp watches the mbarrier; the others park at the block barrier below
        bool ok = true;
        if (tid < 32) {
            ok = mbar_wait_bounded(bar, 0);
            if (!ok && tid == 0) atomicExch(p.status, (int)kDevStageTimeout);
        }
        // A wait that ran out marks the call as failed (the host reads the status word) but the block does not
        // leave: it fetches the same windows with plain loads below and carries on, so that its counters and its
        // rows of C are complete and its shared memory stays its own for as long as a late copy could still land
        // (a late copy writes the very bytes the plain loads wrote).
        staged = !__syncthreads_or(!ok);
    }
    if (!staged) {
        if (rp_staged)
            for (int i = rp_base + tid; i < X1; i += kBlock) s_rp[i - rp_base] = p.rp[i];
        for (int i = y_base + tid; i < Y1; i += kBlock) s_col[i - y_base] = p.col[i];
        if (has_val)
            for (int i = y_base + tid; i < Y1; i += kBlock) s_val[i - y_base] = static_cast<const T *>(p.val)[i];
        __syncthreads();
    }
    const int *w_rp = rp_staged ? s_rp - rp_base : p.rp;  // indexable by global row_ptr index (shared window, or the array itself)
    const int *__restrict__ w_col = s_col - y_base;  // indexable by global non-zero index
    const T *__restrict__ w_val = s_val - y_base;

    // ---- unit boundaries, searched in the staged row_ptr window ----
    if (tid <= GPC) {
        int2 r;
        if (tid == 0) r = c0;
        else if (tid == GPC) r = c1;
        else {
            long long d = (long long)t * p.tile_items + (long long)tid * p.unit_items;
            if (d > p.total) d = p.total;
            long long lo = d - Y1 > X0 ? d - Y1 : X0;
            long long hi = d - Y0 < X1 ? d - Y0 : X1;
            while (lo < hi) {
                const long long mid = (lo + hi) >> 1;
                if ((long long)w_rp[mid] <= d - mid - 1) lo = mid + 1;
                else hi = mid;
            }
            r = make_int2((int)lo, (int)(d - lo));
        }
        s_fx[tid] = r.x;
        s_fy[tid] = r.y;
    }
    __syncthreads();

    // ---- walk this group's unit ----
    if constexpr (!SPREAD) {
        const int x0 = s_fx[g], y0 = s_fy[g], x1 = s_fx[g + 1], y1 = s_fy[g + 1];
        bool head_pending = x0 >= 1 && y0 > w_rp[x0 - 1];  // first row began before this unit
        int x = x0;
        int next_mark = x < x1 ? w_rp[x] : 0x7fffffff;  // non-zero index that marker x precedes
        float acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
        // scaled product: the factor of the row being summed, fetched when the row starts so that its latency
        // hides behind the row's gathers
        [[maybe_unused]] float row_s = 1.0f;
        if constexpr (SCALED) { if (rs && x >= 1 && x < x1) row_s = __ldg(rs + x - 1); }

        auto end_row = [&]() {
            if (x >= 1) {  // marker x ends row x-1 (marker 0 ends nothing)
                if (head_pending) {
                    smem_put<VEC>(s_head + g * SLAB + l * VEC, acc);
                    head_pending = false;
                } else if (active) {
                    if constexpr (SCALED) scale_by<VEC>(acc, row_s);
                    Lane<T, VEC>::store(Cl + (size_t)(x - 1) * dim, acc);
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
            }
            ++x;
            next_mark = x < x1 ? w_rp[x] : 0x7fffffff;
            if constexpr (SCALED) { if (rs && x < x1) row_s = __ldg(rs + x - 1); }
        };

        int k = y0;
        // full batches: U gathers in flight, no bound checks
        for (; k + U <= y1; k += U) {
            typename Lane<T, VEC>::raw b[U];
            typename Lane<T, VEC>::scalar a[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned ci = (unsigned)w_col[k + u];
                if constexpr (SCALED) a[u] = cs ? Lane<T, VEC>::from_float(__ldg(cs + ci)) : Lane<T, VEC>::one();
                else a[u] = has_val ? Lane<T, VEC>::value(w_val[k + u]) : Lane<T, VEC>::one();
                if (active) b[u] = gather(ci);
            }
            while (next_mark <= k) end_row();
            if (next_mark >= k + U) {  // no row ends inside the batch
                if (active) {
#pragma unroll
                    for (int u = 0; u < U; ++u) Lane<T, VEC>::fma(acc, a[u], b[u]);
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    while (next_mark <= k + u) end_row();
                    if (active) Lane<T, VEC>::fma(acc, a[u], b[u]);
                }
            }
        }
        // remainder: fewer than U non-zeros
        if (k < y1) {
            typename Lane<T, VEC>::raw b[U];
            typename Lane<T, VEC>::scalar a[U];
#pragma unroll
            for (int u = 0; u < U - 1; ++u) {
                if (k + u < y1) {
                    const unsigned ci = (unsigned)w_col[k + u];
                    if constexpr (SCALED) a[u] = cs ? Lane<T, VEC>::from_float(__ldg(cs + ci)) : Lane<T, VEC>::one();
                else a[u] = has_val ? Lane<T, VEC>::value(w_val[k + u]) : Lane<T, VEC>::one();
                    if (active) b[u] = gather(ci);
                }
            }
#pragma unroll
            for (int u = 0; u < U - 1; ++u) {
                if (k + u < y1) {
                    while (next_mark <= k + u) end_row();
                    if (active) Lane<T, VEC>::fma(acc, a[u], b[u]);
                }
            }
        }
        while (x < x1) end_row();
        smem_put<VEC>(s_carry + g * SLAB + l * VEC, acc);
    } else {
        // ---- the warp walks its unit: group sg takes the non-zeros y0 + sg, y0 + sg + G, .. ----
        const int x0 = s_fx[g], y0 = s_fy[g], x1 = s_fx[g + 1], y1 = s_fy[g + 1];
        bool head_pending = x0 >= 1 && y0 > w_rp[x0 - 1];
        int x = x0;
        int next_mark = x < x1 ? w_rp[x] : 0x7fffffff;
        float acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
        // partial sums of the groups -> every lane holds the row: level by level, partner group sg ^ 1, ^ 2, ^ 4
        auto combine = [&]() {
#pragma unroll
            for (int off = GL; off < 32; off <<= 1) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
            }
        };
        auto end_row = [&]() {  // warp-uniform: every lane of the warp sees the same x and next_mark
            if (x >= 1) {
                combine();
                if (head_pending) {
                    if (sg == 0) smem_put<VEC>(s_head + g * SLAB + l * VEC, acc);
                    head_pending = false;
                } else if (active && sg == 0) {
                    Lane<T, VEC>::store(Cl + (size_t)(x - 1) * dim, acc);
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
            }
            ++x;
            next_mark = x < x1 ? w_rp[x] : 0x7fffffff;
        };
        // one slice = the G consecutive non-zeros [base, base + G), one per group; `mine` says whether this group's
        // non-zero exists (remainder) - its operands a, b are already in registers
        auto fold_slice = [&](int base, bool mine, typename Lane<T, VEC>::scalar a, const typename Lane<T, VEC>::raw &b) {
            while (next_mark <= base) end_row();
            const int j = base + sg;
            if (next_mark >= base + G) {  // no row ends inside the slice
                if (active && mine) Lane<T, VEC>::fma(acc, a, b);
            } else {
                int lo = base;
                while (next_mark < base + G) {  // rows that end inside the slice, one after the other
                    if (active && mine && j >= lo && j < next_mark) Lane<T, VEC>::fma(acc, a, b);
                    lo = next_mark;
                    end_row();
                }
                if (active && mine && j >= lo) Lane<T, VEC>::fma(acc, a, b);
            }
        };
        constexpr int NB = G * U;  // non-zeros per batch of the warp
        int k = y0;
        for (; k + NB <= y1; k += NB) {
            typename Lane<T, VEC>::raw b[U];
            typename Lane<T, VEC>::scalar a[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = k + u * G + sg;
                const unsigned ci = (unsigned)w_col[j];
                a[u] = has_val ? Lane<T, VEC>::value(w_val[j]) : Lane<T, VEC>::one();
                if (active) b[u] = gather(ci);
            }
            if (next_mark >= k + NB) {  // no row ends inside the batch
                if (active) {
#pragma unroll
                    for (int u = 0; u < U; ++u) Lane<T, VEC>::fma(acc, a[u], b[u]);
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) fold_slice(k + u * G, true, a[u], b[u]);
            }
        }
        if (k < y1) {  // remainder: fewer than NB non-zeros
            typename Lane<T, VEC>::raw b[U];
            typename Lane<T, VEC>::scalar a[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = k + u * G + sg;
                if (j < y1) {
                    const unsigned ci = (unsigned)w_col[j];
                    a[u] = has_val ? Lane<T, VEC>::value(w_val[j]) : Lane<T, VEC>::one();
                    if (active) b[u] = gather(ci);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (k + u * G < y1) fold_slice(k + u * G, k + u * G + sg < y1, a[u], b[u]);
        }
        while (x < x1) end_row();
        combine();
        if (sg == 0) smem_put<VEC>(s_carry + g * SLAB + l * VEC, acc);
    }
    __syncthreads();

    // ---- in-tile fix-up: the group finishes the row its unit ended first, if it began earlier ----
    {
        const int x0 = s_fx[g], x1 = s_fx[g + 1], y0 = s_fy[g];
        if (sg == 0 && x0 >= 1 && x1 > x0 && y0 > w_rp[x0 - 1]) {
            int s = g;
            while (s > 0 && s_fx[s] == x0) --s;
            const bool from_prev = s_fx[0] == x0 && Y0 > w_rp[X0 - 1];  // row began before this tile
            float sum[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) sum[i] = 0.0f;
            for (int q = s; q < g; ++q) vec_add<VEC>(sum, s_carry + q * SLAB + l * VEC);
            vec_add<VEC>(sum, s_head + g * SLAB + l * VEC);
            if (active) {
                if (from_prev) gmem_put_f32<VEC>(p.thead + (size_t)t * dim + coff, sum);
                else {
                    if constexpr (SCALED) { if (rs) scale_by<VEC>(sum, __ldg(rs + x0 - 1)); }
                    Lane<T, VEC>::store(Cl + (size_t)(x0 - 1) * dim, sum);
                }
            }
        }
    }
    // ---- tile carry: everything after the last marker of the tile ----
    if (g == GPC - 1 && sg == 0) {
        const int xe = s_fx[GPC];
        int s = GPC;
        while (s > 0 && s_fx[s] == xe) --s;
        float sum[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) sum[i] = 0.0f;
        for (int q = s; q < GPC; ++q) vec_add<VEC>(sum, s_carry + q * SLAB + l * VEC);
        if (active) gmem_put_f32<VEC>(p.tcarry + (size_t)t * dim + coff, sum);
    }

    // ---- cross-tile fix-up without a second kernel (small problems, where a launch costs more than this):
    // every contribution (a tile's carry, the ending tile's head) bumps the counter of the tile that ends
    // the row; the block that brings the count to `need` finds everything in place and sums it, in the
    // fixed order.  No block ever waits for another.  The fence below has to wait for this thread's
    // stores to C as well, which is why large problems run fixup_kernel after the tile kernel instead.
    if (!p.fused) return;
    __threadfence();  // this thread's tcarry / thead stores are visible device-wide before the count moves
    __syncthreads();
    int *s_todo = s_fx;  // the unit boundaries are no longer needed
    if (tid == 0) {
        __threadfence();
        int *cnt = p.cnt + (size_t)blockIdx.y * p.n_tiles;
        int todo0 = -1, todo1 = -1;
        const int e = __ldg(p.consumer + t);
        if (e >= 0 && atomicAdd(cnt + e, 1) + 1 == __ldg(p.need + e)) todo0 = e;
        const int mine = __ldg(p.need + t);
        if (mine > 0 && atomicAdd(cnt + t, 1) + 1 == mine) todo1 = t;
        if (todo0 >= 0) cnt[todo0] = 0;  // ready for the next launch
        if (todo1 >= 0) cnt[todo1] = 0;
        __threadfence();
        s_todo[0] = todo0;
        s_todo[1] = todo1;
    }
    __syncthreads();
    const int col0 = blockIdx.y * SLAB, col1 = col0 + SLAB < p.dim ? col0 + SLAB : p.dim;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int e = s_todo[i];
        if (e < 0) continue;
        const int chain = __ldg(p.need + e) - 1;
        if (chain <= p.very_long) block_fixup<T, kBlock>(p, e, chain, col0, col1, tid);  // longer chains: fixup_kernel, after this one
    }
}

// ---------------------------------------------------------------------------------------------
// cross-tile fix-up
// ---------------------------------------------------------------------------------------------
// Plan time, one thread per tile: how many contributions the tile's cross-tile fix-up waits for
// (its own head plus one carry per tile of the chain), which tile consumes this tile's carry, and the
// list of tiles whose chain is too long to be summed by one tile block (very_long).
static __global__ void fixup_plan_kernel(const int2 *__restrict__ xy, const int *__restrict__ rp, int n_tiles, int very_long,
                                  int *__restrict__ consumer, int *__restrict__ need, int *__restrict__ list, int *__restrict__ count,
                                  int capacity) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tiles) return;
    int s = 0, n = 0;
    if (t >= 1 && fixup_candidate(xy, rp, t, s) >= 0) {
        n = t - s + 1;
        if (t - s > very_long) {
            const int at = atomicAdd(count, 1);
            if (at < capacity) list[at] = t;
        }
    }
    need[t] = n;
    // the row in progress when tile t ends is row xe-1; it is ended by the tile e that consumes marker xe:
    // j = first boundary with x > xe, e = j - 1 (>= t + 1)
    const int xe = __ldg(xy + t + 1).x;
    int lo = t + 2, hi = n_tiles + 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(xy + mid).x > xe) hi = mid;
        else lo = mid + 1;
    }
    int e = -1;
    if (lo <= n_tiles) {
        e = lo - 1;
        const int2 a = __ldg(xy + e);
        if (!(a.x >= 1 && a.y > __ldg(rp + a.x - 1))) e = -1;  // the row starts exactly where tile e starts: nothing carried in
    }
    consumer[t] = e;
}

// Chains longer than very_long (a row spanning thousands of tiles): one block of kStrands warps per
// listed tile (the first blocks of fixup_kernel).  Strand g adds carries s+g, s+g+16, ... in order, then strand 0
// adds the strands in order and the tile's head last - the same order block_fixup uses.
template <typename T>
__device__ __forceinline__ void fixup_long_block(const int2 *__restrict__ xy, const int *__restrict__ rp, const float *__restrict__ tcarry,
                                                 const float *__restrict__ thead, T *__restrict__ C, int t, int dim,
                                                 const float *__restrict__ row_scale) {
    __shared__ float part[kStrands][32];
    const int g = threadIdx.x / 32, lane = threadIdx.x % 32;
    int s;
    const int row = fixup_candidate(xy, rp, t, s);
    if (row < 0) return;  // cannot happen for a listed tile
    for (int j0 = 0; j0 < dim; j0 += 32) {
        const int j = j0 + lane;
        float sg = 0.0f;
        if (j < dim)
            for (int q = s + g; q < t; q += kStrands) sg += tcarry[(size_t)q * dim + j];
        part[g][lane] = sg;
        __syncthreads();
        if (g == 0 && j < dim) {
            float sum = 0.0f;
#pragma unroll
            for (int k = 0; k < kStrands; ++k) sum += part[k][lane];
            sum += thead[(size_t)t * dim + j];
            if (row_scale) sum *= __ldg(row_scale + row);
            store_c(C + (size_t)row * dim + j, sum);
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void store_c4(float *p, const float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store_c4(__half *p, const float4 v) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<const unsigned *>(&lo);
    w.y = *reinterpret_cast<const unsigned *>(&hi);
    *reinterpret_cast<uint2 *>(p) = w;
}

// Cross-tile fix-up after the tile kernel, one launch of kStrands * 32 threads per block:
//   blocks [0, n_long): one block per listed tile whose chain exceeds very_long (fixup_long_block);
//   the other blocks (large problems only; none when the tile kernel does the fix-up itself): L lanes per
//   tile that ends a carried-in row, same sums in the same order as block_fixup in the tile kernel.  V4 (dim a
//   multiple of 4): a lane takes four columns at a time, so L = dim/4 lanes finish a row in one pass and a warp
//   serves 32/L tiles.
template <typename T, int L, bool V4>
__global__ void __launch_bounds__(kStrands * 32) fixup_kernel(const TileParams p, const int *__restrict__ long_list, int n_long) {
    if ((int)blockIdx.x < n_long) {
        fixup_long_block<T>(p.tile_xy, p.rp, p.tcarry, p.thead, static_cast<T *>(p.C), long_list[blockIdx.x], p.dim, p.row_scale);
        return;
    }
    const int gid = ((int)blockIdx.x - n_long) * (kStrands * 32) + (int)threadIdx.x;
    const int t = 1 + gid / L, lane = gid % L;
    if (t >= p.n_tiles) return;
    const int n = __ldg(p.need + t);
    if (n <= 0 || n - 1 > p.very_long) return;
    const int chain = n - 1;
    if (!V4 || chain > p.long_chain) {
        block_fixup<T, L>(p, t, chain, 0, p.dim, lane);
        return;
    }
    const int row = __ldg(p.tile_xy + t).x - 1;
    const size_t dim = (size_t)p.dim;
    for (int j = lane * 4; j < p.dim; j += L * 4) {
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int q = t - chain; q < t; ++q) {
            const float4 c = __ldcg(reinterpret_cast<const float4 *>(p.tcarry + (size_t)q * dim + j));
            sum.x += c.x; sum.y += c.y; sum.z += c.z; sum.w += c.w;
        }
        const float4 h = __ldcg(reinterpret_cast<const float4 *>(p.thead + (size_t)t * dim + j));
        sum.x += h.x; sum.y += h.y; sum.z += h.z; sum.w += h.w;
        if (p.row_scale) {
            const float r = __ldg(p.row_scale + row);
            sum.x *= r; sum.y *= r; sum.z *= r; sum.w *= r;
        }
        store_c4(static_cast<T *>(p.C) + (size_t)row * dim + j, sum);
    }
}

}  // namespace mps
