// Interpreted tile kernels of the strided pointwise engine (see chain.cu for
// the overview and chain.cuh for the kernels): any program, operand classes
// read at run time.
#include "chain.cuh"

namespace fb {

void launch_interp_tile(cudaStream_t stream, const TileParams& TP, unsigned grid, bool vector, float* out) {
  if (vector)
    chain_tile_kernel<VectorTile<-1>, Interp><<<grid, kChThreads, 0, stream>>>(TP, out);
  else
    chain_tile_kernel<ScalarTile, Interp><<<grid, kChThreads, 0, stream>>>(TP, out);
}

}  // namespace fb
