// Launcher for ferro's own CUDA kernels recompiled for sm_100a (see build_ref_gpu.py, which
// puts the reference kernel text in front of this file with -include).  Launch geometry is the
// reference's:
//   LayerNorm        one 256-thread block per row (crates/ferro-cuda/src/lib.rs:1283, 1310)
//   softmax stats    one REDUCE_BLOCK-thread block per row (lib.rs:624-629)
//   softmax apply    LaunchConfig::for_num_elems(n) (lib.rs:665), which in cudarc 0.19 is
//                    ceil(n / 1024) blocks of 1024 threads
// Measurement infrastructure: the library never loads this.
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {

__attribute__((visibility("default"))) int ref_gpu_layer_norm(cudaStream_t s, const float* x, const float* w, const float* b,
                                                               float* y, float* h, float* stds, unsigned rows, unsigned cols,
                                                               float eps) {
  if (rows == 0) return 0;
  const unsigned has_w = w != nullptr, has_b = b != nullptr;
  if (h && stds) ref_layer_norm<<<rows, 256, 0, s>>>(x, has_w ? w : x, has_b ? b : x, y, h, stds, cols, eps, has_w, has_b);
  else ref_layer_norm_output<<<rows, 256, 0, s>>>(x, has_w ? w : x, has_b ? b : x, y, cols, eps, has_w, has_b);
  return (int)cudaGetLastError();
}

__attribute__((visibility("default"))) int ref_gpu_softmax(cudaStream_t s, const float* x, float* stats, float* out,
                                                            unsigned rows, unsigned cols, int log) {
  const unsigned n = rows * cols;
  if (n == 0) return 0;
  ref_softmax_row_stats<<<rows, REF_REDUCE_BLOCK, 0, s>>>(x, stats, cols);
  const unsigned blocks = (n + 1023u) / 1024u;
  if (log) ref_log_softmax_apply<<<blocks, 1024, 0, s>>>(x, stats, out, n, cols);
  else ref_softmax_apply<<<blocks, 1024, 0, s>>>(x, stats, out, n, cols);
  return (int)cudaGetLastError();
}

}  // extern "C"
