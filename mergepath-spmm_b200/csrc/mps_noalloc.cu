// mps_spmm_noalloc: the SpMM for callers that must not allocate device memory.
//
// Who cannot allocate: code that runs inside somebody else's memory allotment or under a rule that
// forbids the allocator at call time - a plugin handed a fixed arena by its host framework, a
// service whose device memory is fully pre-committed at start-up, a latency-critical loop where
// cudaMalloc's implicit device synchronisation is not acceptable.  Such a caller still owns A, B
// and C; what it cannot provide is the plan's scratch (tile coordinates, one carry row and one head
// row per tile, the long-row list, two counters).  Here that scratch lives in one file-scope device
// array of fixed size, part of the library image: every GPU that loads the library holds
// MPS_NOALLOC_SCRATCH_BYTES of it until the process exits.
//
// Consequences spelled out:
//   - problems whose scratch does not fit are rejected with MPS_ERR_UNSUPPORTED (limits below);
//   - all calls on a device share the array, so two calls that overlap on the GPU (different
//     streams or host threads) race on it - serialise them;
//   - the array keeps the previous call's contents; what must start at zero (status word, long-row
//     counter, the per-tile arrival counters) is cleared by every call, everything else is written
//     before it is read;
//   - the first call on each device looks up the array's device address (cudaGetSymbolAddress) -
//     make that first call outside any stream capture.
// Nothing in this path calls cudaMalloc, cudaFree or a library routine that allocates.
#include "mps.h"

#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "mps_internal.h"
#include "mps_plan.h"

using mps::fail;

namespace {

constexpr int kMaxTiles = MPS_NOALLOC_MAX_TILES;
constexpr size_t kMaxCarryFloats = MPS_NOALLOC_MAX_CARRY_FLOATS;
constexpr int kMaxLong = kMaxTiles / 32 + 2;  // very-long-row list entries (more than the plan ever asks for)

// byte offsets inside the scratch array, each a multiple of 256
constexpr size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
constexpr size_t kOffStatus = 0;
constexpr size_t kOffCount = 256;
constexpr size_t kOffTileXy = 512;
constexpr size_t kOffLongList = kOffTileXy + up256(sizeof(int2) * ((size_t)kMaxTiles + 1));
constexpr size_t kOffConsumer = kOffLongList + up256(sizeof(int) * (size_t)kMaxLong);
constexpr size_t kOffNeed = kOffConsumer + up256(sizeof(int) * (size_t)kMaxTiles);
constexpr size_t kOffCnt = kOffNeed + up256(sizeof(int) * (size_t)kMaxTiles);
constexpr size_t kOffCarry = kOffCnt + up256(sizeof(int) * (size_t)kMaxTiles);
constexpr size_t kOffHead = kOffCarry + up256(sizeof(float) * kMaxCarryFloats);
constexpr size_t kScratchBytes = kOffHead + up256(sizeof(float) * kMaxCarryFloats);
static_assert(kScratchBytes <= MPS_NOALLOC_SCRATCH_BYTES, "the header states the size of the scratch array");

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never a
// pointer that a kernel could use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
unsigned char *g_scratch_base[kMaxDevices];  // device address of g_noalloc_scratch, per device

// Device address of the scratch on the current device; looked up once per device.
int scratch_base(unsigned char **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MPS_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(MPS_ERR_UNSUPPORTED, "device ordinal %d outside the %d this entry point tracks", dev, kMaxDevices);
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_scratch_base[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return fail(MPS_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        g_scratch_base[dev] = static_cast<unsigned char *>(ptr);
    }
    *out = g_scratch_base[dev];
    return MPS_OK;
}

}  // namespace

extern "C" int mps_spmm_noalloc(int32_t n_rows, int32_t nnz, int32_t dim, int dtype, int32_t cost, int32_t threads_per_warp,
                                const int32_t *d_row_ptr, const int32_t *d_col_idx, const void *d_val, const void *d_B, void *d_C,
                                void *stream) {
    if (!d_row_ptr || !d_B || !d_C || (!d_col_idx && nnz > 0)) return fail(MPS_ERR_ARG, "mps_spmm_noalloc: NULL argument");
    if (dim < 1 || cost < 1) return fail(MPS_ERR_ARG, "mps_spmm_noalloc: dim and cost must be >= 1 (dim=%d cost=%d)", dim, cost);
    if (dtype != MPS_F32 && dtype != MPS_F16) return fail(MPS_ERR_ARG, "mps_spmm_noalloc: unknown dtype %d", dtype);
    if (n_rows < 0 || nnz < 0) return fail(MPS_ERR_ARG, "mps_spmm_noalloc: negative size");
    if ((long long)n_rows + 1 + nnz >= 1LL << 31) return fail(MPS_ERR_UNSUPPORTED, "mps_spmm_noalloc: N+1+nnz does not fit 31 bits");

    mps_plan plan;  // lives on this stack frame; owns nothing
    mps::plan_init_shape(&plan, n_rows, nnz, dim, dtype, cost, threads_per_warp);
    if (int rc = mps::plan_finish_layout(&plan)) return rc;
    const size_t carry_floats = (size_t)plan.n_tiles * (size_t)dim;
    if ((long long)plan.n_tiles * plan.n_col_slabs > kMaxTiles || carry_floats > kMaxCarryFloats)
        return fail(MPS_ERR_UNSUPPORTED,
                    "mps_spmm_noalloc: this problem needs %d tiles and %zu carry floats; the built-in scratch holds at most %d tiles and "
                    "%zu floats (tiles x dim) - use mps_plan_create/mps_spmm, which allocate what they need",
                    plan.n_tiles, carry_floats, kMaxTiles, kMaxCarryFloats);

    unsigned char *base = nullptr;
    if (int rc = scratch_base(&base)) return rc;
    plan.d_status = reinterpret_cast<int *>(base + kOffStatus);
    plan.d_long_count = reinterpret_cast<int *>(base + kOffCount);
    plan.d_tile_xy = reinterpret_cast<int2 *>(base + kOffTileXy);
    plan.d_long_list = reinterpret_cast<int *>(base + kOffLongList);
    plan.d_consumer = reinterpret_cast<int *>(base + kOffConsumer);
    plan.d_need = reinterpret_cast<int *>(base + kOffNeed);
    plan.d_cnt = reinterpret_cast<int *>(base + kOffCnt);
    plan.d_tcarry = reinterpret_cast<float *>(base + kOffCarry);
    plan.d_thead = reinterpret_cast<float *>(base + kOffHead);
    plan.long_capacity = plan.n_tiles / plan.long_chain + 2;  // <= kMaxLong because n_tiles <= kMaxTiles

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(plan.d_status, 0, sizeof(int), st);  // left over from the previous call otherwise
    if (e != cudaSuccess) return fail(MPS_ERR_CUDA, "cudaMemsetAsync(status): %s", cudaGetErrorString(e));
    if (int rc = mps_plan_partition(&plan, d_row_ptr, stream)) return rc;  // clears the long-row counter and the arrival counters itself
    if (int rc = mps_spmm(&plan, d_row_ptr, d_col_idx, d_val, d_B, d_C, stream)) return rc;
    return mps_plan_sync_check(&plan, stream);
}
