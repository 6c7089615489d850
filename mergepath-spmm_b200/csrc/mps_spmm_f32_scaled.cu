// Instantiates the fp32 kernels of the scaled product (mps_spmm_scaled); a translation unit of its own so that the three sets compile in parallel.
#include "mps_dispatch.cuh"

namespace mps {
int spmm_f32_scaled(mps_plan *p, const TileParams &tp, cudaStream_t st) { return spmm_typed<float, 4, true>(p, tp, st); }
}  // namespace mps
