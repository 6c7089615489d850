// Instantiates the fp16-storage / fp32-accumulate kernels; a translation unit of its own so that the three sets compile in parallel.
#include "mps_dispatch.cuh"

namespace mps {
int spmm_f16(mps_plan *p, const TileParams &tp, cudaStream_t st) { return spmm_typed<__half, 8, false>(p, tp, st); }
}  // namespace mps
