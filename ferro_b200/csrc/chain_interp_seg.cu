// Interpreted segment kernels of the strided pointwise engine (see chain.cu
// for the overview and chain.cuh for the kernels): any program; VEC = 4 with
// float4 accesses or 1, one or four vectors per thread.
#include "chain.cuh"

namespace fb {

void launch_interp_seg(cudaStream_t stream, const ChainParams& P, uint64_t nseg, unsigned grid, bool vec, int unroll,
                       float* out) {
  if (vec) {
    if (unroll == 4) chain_seg_kernel<4, 4, Interp><<<grid, kChThreads, 0, stream>>>(P, nseg, out);
    else chain_seg_kernel<4, 1, Interp><<<grid, kChThreads, 0, stream>>>(P, nseg, out);
  } else {
    if (unroll == 4) chain_seg_kernel<1, 4, Interp><<<grid, kChThreads, 0, stream>>>(P, nseg, out);
    else chain_seg_kernel<1, 1, Interp><<<grid, kChThreads, 0, stream>>>(P, nseg, out);
  }
}

}  // namespace fb
