// mps_gather_probe: the rate at which this GPU serves the access pattern of the SpMM - whole rows of a dense
// table fetched at random with 128-bit loads - measured by a kernel that does nothing else.  With a table
// that fits the L2 it gives the L2 -> SM gather rate, with a table far larger than the L2 the rate of random
// rows out of HBM; the bench reports the multiply's gathered bytes per second against both, because a plain
// copy bandwidth says little about a gather that the L2 serves.  No reference counterpart.
#include <cuda_runtime.h>
#include <stdint.h>

#include "mps.h"
#include "mps_internal.h"

using mps::fail;

namespace {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    return x ^ (x >> 16);
}

// A group of LANES threads fetches one row (LANES x 16 bytes) per step, kInFlight rows before it touches the data.
// Row numbers come from a per-group linear congruential sequence (two instructions per row, so that the kernel
// measures the memory system and not its own index arithmetic), the same in every lane of a group; what is
// loaded is xor-folded into one word per thread and stored once, so the loads cannot be dropped.
constexpr int kInFlight = 8;

template <int LANES>
__global__ void __launch_bounds__(256, 4) gather_probe_kernel(const uint4 *__restrict__ table, uint32_t table_rows, int steps, uint32_t seed,
                                                          uint32_t *__restrict__ sink) {
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t group = tid / LANES, lane = tid % LANES;
    uint32_t x = mix32(group * 0x9E3779B1u + seed);
    uint32_t fold = 0;
    const uint4 *__restrict__ mine = table + lane;
    for (int s = 0; s < steps; s += kInFlight) {
        uint4 v[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            x = x * 1664525u + 1013904223u;
            const uint32_t row = __umulhi(x, table_rows);
            v[u] = __ldg(mine + (size_t)row * LANES);
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) fold ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    sink[tid] = fold;
}

// The same fetch loop over a caller's row numbers (the multiply's own col_idx): group g takes the run
// index[g * steps .. (g + 1) * steps) in order, as a lane group of the multiply walks its unit.
template <int LANES>
__global__ void __launch_bounds__(256, 4) gather_stream_kernel(const uint4 *__restrict__ table, const int *__restrict__ index, long long n_index,
                                                           int steps, uint32_t *__restrict__ sink) {
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t group = tid / LANES, lane = tid % LANES;
    uint32_t fold = 0;
    const uint4 *__restrict__ mine = table + lane;
    const long long first = (long long)group * steps;
    for (int s = 0; s < steps; s += kInFlight) {
        uint4 v[kInFlight];
        if (first + s + kInFlight <= n_index) {
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) v[u] = __ldg(mine + (size_t)(uint32_t)__ldg(index + first + s + u) * LANES);
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) fold ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
        } else {
            for (int u = 0; u < kInFlight && first + s + u < n_index; ++u) {
                const uint4 w = __ldg(mine + (size_t)(uint32_t)__ldg(index + first + s + u) * LANES);
                fold ^= w.x ^ w.y ^ w.z ^ w.w;
            }
        }
    }
    sink[tid] = fold;
}

template <int LANES>
void launch(const void *table, uint32_t rows, const int *index, long long n_index, int steps, uint32_t seed, uint32_t *sink, int blocks,
            cudaStream_t st) {
    if (index) gather_stream_kernel<LANES><<<blocks, 256, 0, st>>>(static_cast<const uint4 *>(table), index, n_index, steps, sink);
    else gather_probe_kernel<LANES><<<blocks, 256, 0, st>>>(static_cast<const uint4 *>(table), rows, steps, seed, sink);
}

}  // namespace

static int probe(const void *d_table, int64_t table_rows, int32_t row_bytes, const int32_t *d_index, int64_t gathers, void *d_sink,
                 int64_t sink_bytes, void *stream, float *ms, int64_t *gathered_bytes) {
    if (!d_table || !d_sink || !ms || !gathered_bytes) return fail(MPS_ERR_ARG, "mps_gather_probe: NULL argument");
    if (table_rows < 1 || table_rows > 0xffffffffll || gathers < 1) return fail(MPS_ERR_ARG, "mps_gather_probe: table_rows and gathers must be positive");
    if (row_bytes != 32 && row_bytes != 64 && row_bytes != 128 && row_bytes != 256 && row_bytes != 512)
        return fail(MPS_ERR_ARG, "mps_gather_probe: row_bytes must be 32, 64, 128, 256 or 512");
    if ((uintptr_t)d_table % 16) return fail(MPS_ERR_ALIGN, "mps_gather_probe: the table must be 16-byte aligned");
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return fail(MPS_ERR_CUDA, "mps_gather_probe: no CUDA device");
    const int lanes = row_bytes / 16;
    const int blocks = sms * 4;  // 1024 threads per SM, eight 128-bit loads in flight each: 128 KB on the way per SM
    const long long threads = (long long)blocks * 256, groups = threads / lanes;
    if (sink_bytes < threads * 4) return fail(MPS_ERR_ARG, "mps_gather_probe: the sink needs %lld bytes", threads * 4);
    long long steps = (gathers + groups - 1) / groups;
    steps = (steps + kInFlight - 1) / kInFlight * kInFlight;
    if (steps > (1 << 24)) return fail(MPS_ERR_ARG, "mps_gather_probe: too many gathers for one launch");
    const int *index = reinterpret_cast<const int *>(d_index);
    cudaStream_t st = (cudaStream_t)stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) {
        if (e0) cudaEventDestroy(e0);
        return fail(MPS_ERR_CUDA, "mps_gather_probe: cudaEventCreate failed");
    }
    auto run = [&](uint32_t seed) {
        switch (lanes) {
            case 2: launch<2>(d_table, (uint32_t)table_rows, index, gathers, (int)steps, seed, (uint32_t *)d_sink, blocks, st); break;
            case 4: launch<4>(d_table, (uint32_t)table_rows, index, gathers, (int)steps, seed, (uint32_t *)d_sink, blocks, st); break;
            case 8: launch<8>(d_table, (uint32_t)table_rows, index, gathers, (int)steps, seed, (uint32_t *)d_sink, blocks, st); break;
            case 16: launch<16>(d_table, (uint32_t)table_rows, index, gathers, (int)steps, seed, (uint32_t *)d_sink, blocks, st); break;
            default: launch<32>(d_table, (uint32_t)table_rows, index, gathers, (int)steps, seed, (uint32_t *)d_sink, blocks, st); break;
        }
    };
    run(1);  // warm-up: a table that fits the L2 is resident after this pass
    cudaEventRecord(e0, st);
    run(2);
    cudaEventRecord(e1, st);
    cudaError_t e = cudaEventSynchronize(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    float t = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return fail(MPS_ERR_CUDA, "mps_gather_probe: %s", cudaGetErrorString(e));
    *ms = t;
    *gathered_bytes = (d_index ? gathers : groups * steps) * (long long)row_bytes;
    return MPS_OK;
}

extern "C" int mps_gather_probe(const void *d_table, int64_t table_rows, int32_t row_bytes, int64_t gathers, void *d_sink, int64_t sink_bytes,
                                void *stream, float *ms, int64_t *gathered_bytes) {
    return probe(d_table, table_rows, row_bytes, nullptr, gathers, d_sink, sink_bytes, stream, ms, gathered_bytes);
}

extern "C" int mps_gather_probe_stream(const void *d_table, int64_t table_rows, int32_t row_bytes, const int32_t *d_index, int64_t n_index,
                                       void *d_sink, int64_t sink_bytes, void *stream, float *ms, int64_t *gathered_bytes) {
    if (!d_index) return fail(MPS_ERR_ARG, "mps_gather_probe_stream: d_index is NULL");
    return probe(d_table, table_rows, row_bytes, d_index, n_index, d_sink, sink_bytes, stream, ms, gathered_bytes);
}
