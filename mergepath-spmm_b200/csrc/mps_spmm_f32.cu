// Instantiates the fp32 kernels of the plain product; a translation unit of its own so that the three sets compile in parallel.
#include "mps_dispatch.cuh"

namespace mps {
int spmm_f32(mps_plan *p, const TileParams &tp, cudaStream_t st) { return spmm_typed<float, 4, false>(p, tp, st); }
}  // namespace mps
