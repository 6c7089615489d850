// Launch chain of one multiply: picks the instantiation of spmm_tile_kernel that the plan's layout names and
// launches it with the fix-up kernel that follows.  Included by the three translation units that instantiate
// the kernels (fp32, fp32 scaled, fp16), so that they compile side by side; mps_api.cu calls their entry points.
#pragma once
#include <cuda_runtime.h>

#include "mps.h"
#include "mps_internal.h"
#include "mps_kernels.cuh"
#include "mps_plan.h"

namespace mps {

#define MPS_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess) return fail(MPS_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

template <typename T, int VEC, int GL, int U, int BLOCK, bool SCALED>
static int launch_tile_k(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    auto kern = spmm_tile_kernel<T, VEC, GL, U, BLOCK, SCALED>;
    if (tp.smem_bytes > 48 * 1024) MPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp.smem_bytes));
    dim3 grid((unsigned)p->n_tiles, (unsigned)p->n_col_slabs);
    kern<<<grid, BLOCK, tp.smem_bytes, st>>>(tp);
    MPS_CUDA(cudaGetLastError());
    return MPS_OK;
}

template <typename T, int VEC, int GL, int U, int BLOCK, bool SCALED>
static int launch_tile(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    if constexpr (BLOCK < GL) {
        return fail(MPS_ERR_STATE, "block of %d threads cannot hold a group of %d lanes", BLOCK, GL);
    } else {
        return launch_tile_k<T, VEC, GL, U, BLOCK, SCALED>(p, tp, st);
    }
}

template <typename T, int VEC, int GL, int U, bool SCALED>
static int launch_tile_b(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    switch (p->block) {
        case 64: return launch_tile<T, VEC, GL, U, 64, SCALED>(p, tp, st);
        case 128: return launch_tile<T, VEC, GL, U, 128, SCALED>(p, tp, st);
        case 256: return launch_tile<T, VEC, GL, U, 256, SCALED>(p, tp, st);
    }
    return fail(MPS_ERR_STATE, "no kernel for blocks of %d threads", p->block);
}

template <typename T, int VEC, int GL, bool SCALED>
static int launch_tile_u(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    if (p->unroll == 10) return launch_tile_b<T, VEC, GL, 10, SCALED>(p, tp, st);
    if (p->unroll == 8) return launch_tile_b<T, VEC, GL, 8, SCALED>(p, tp, st);
    return launch_tile_b<T, VEC, GL, 4, SCALED>(p, tp, st);
}

template <typename T, int VEC, bool SCALED>
static int launch_tile_gl(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    switch (p->gl) {
        case 2: return launch_tile_u<T, VEC, 2, SCALED>(p, tp, st);
        case 4: return launch_tile_u<T, VEC, 4, SCALED>(p, tp, st);
        case 8: return launch_tile_u<T, VEC, 8, SCALED>(p, tp, st);
        case 16: return launch_tile_u<T, VEC, 16, SCALED>(p, tp, st);
        case 32: return launch_tile_u<T, VEC, 32, SCALED>(p, tp, st);
    }
    return fail(MPS_ERR_STATE, "no kernel for %d lanes per chunk", p->gl);
}

// Narrow rows with half the columns per lane (fp16, four columns per lane): groups of 2, 4 or 8 lanes only - wider rows
// take the full vector.
template <typename T, int VEC, bool SCALED>
static int launch_tile_gl_narrow(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    switch (p->gl) {
        case 2: return launch_tile_u<T, VEC, 2, SCALED>(p, tp, st);
        case 4: return launch_tile_u<T, VEC, 4, SCALED>(p, tp, st);
        case 8: return launch_tile_u<T, VEC, 8, SCALED>(p, tp, st);
    }
    return fail(MPS_ERR_STATE, "no narrow-row kernel for %d lanes per chunk", p->gl);
}

// The variant with a warp per unit: one block size (64), one unroll (8).
template <typename T, int VEC, int GL>
static int launch_tile_warp_k(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    auto kern = spmm_tile_kernel<T, VEC, GL, 8, 64, false, true>;
    if (tp.smem_bytes > 48 * 1024) MPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tp.smem_bytes));
    dim3 grid((unsigned)p->n_tiles, (unsigned)p->n_col_slabs);
    kern<<<grid, 64, tp.smem_bytes, st>>>(tp);
    MPS_CUDA(cudaGetLastError());
    return MPS_OK;
}
template <typename T, int VEC>
static int launch_tile_warp(const mps_plan *p, const TileParams &tp, cudaStream_t st) {
    switch (p->gl) {
        case 2: return launch_tile_warp_k<T, VEC, 2>(p, tp, st);
        case 4: return launch_tile_warp_k<T, VEC, 4>(p, tp, st);
        case 8: return launch_tile_warp_k<T, VEC, 8>(p, tp, st);
        case 16: return launch_tile_warp_k<T, VEC, 16>(p, tp, st);
    }
    return fail(MPS_ERR_STATE, "no warp-per-unit kernel for %d lanes per chunk", p->gl);
}

template <typename T, int FULLVEC, bool SCALED>
static int spmm_typed(mps_plan *p, const TileParams &tp, cudaStream_t st) {
    int rc;
    const bool prof = p->profiling && p->prof_used < kProfSlots;
    if (prof) MPS_CUDA(cudaEventRecord(p->prof_ev[2 * p->prof_used], st));
    if (p->vec == 1) rc = launch_tile_b<T, 1, 32, 4, SCALED>(p, tp, st);
    else if (p->vec != FULLVEC) {
        if constexpr (FULLVEC == 8 && !SCALED) rc = launch_tile_gl_narrow<T, 4, SCALED>(p, tp, st);
        else rc = fail(MPS_ERR_STATE, "no kernel with %d columns per lane", p->vec);
    } else if (p->walk && !SCALED) {
        if constexpr (!SCALED) rc = launch_tile_warp<T, FULLVEC>(p, tp, st);
        else rc = MPS_ERR_STATE;
    } else rc = launch_tile_gl<T, FULLVEC, SCALED>(p, tp, st);
    if (rc != MPS_OK) return rc;
    if (prof) { MPS_CUDA(cudaEventRecord(p->prof_ev[2 * p->prof_used + 1], st)); ++p->prof_used; }
    // one launch after the tile kernel: a block per row whose chain is too long for anyone else, then (large
    // problems, where the tile kernel does not fix up across tiles itself) dim/4 lanes per remaining tile
    const long long tiles = (!p->fused && p->n_tiles > 1) ? p->n_tiles - 1 : 0;
    if (tiles > 0 || p->n_long > 0) {
        const int threads = kStrands * 32;
        const int quads = p->dim / 4;  // lanes a row needs at four columns each
        auto blocks = [&](int lanes) { return (unsigned)(p->n_long + (tiles * lanes + threads - 1) / threads); };
        if (p->vec == 1) fixup_kernel<T, 32, false><<<blocks(32), threads, 0, st>>>(tp, p->d_long_list, p->n_long);
        else if (quads <= 4) fixup_kernel<T, 4, true><<<blocks(4), threads, 0, st>>>(tp, p->d_long_list, p->n_long);
        else if (quads <= 8) fixup_kernel<T, 8, true><<<blocks(8), threads, 0, st>>>(tp, p->d_long_list, p->n_long);
        else if (quads <= 16) fixup_kernel<T, 16, true><<<blocks(16), threads, 0, st>>>(tp, p->d_long_list, p->n_long);
        else fixup_kernel<T, 32, true><<<blocks(32), threads, 0, st>>>(tp, p->d_long_list, p->n_long);
        MPS_CUDA(cudaGetLastError());
    }
    return MPS_OK;
}

#undef MPS_CUDA

}  // namespace mps
