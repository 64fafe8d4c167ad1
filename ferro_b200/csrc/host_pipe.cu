// LayerNorm forward + backward for callers whose tensors live in HOST memory.
//
// ferro users who keep their data on the host reach the device through
// alloc_from_host / copy_to_host (crates/ferro-cuda/src/lib.rs:571-588,
// 674-686): upload everything, compute, download everything, one after the
// other on one stream.  Rows of a LayerNorm are independent, so the same
// request is cut into row chunks here and run as a three-stage pipeline on
// three streams - upload chunk k + 1 while chunk k is computed and chunk k - 1
// is downloaded - which keeps both directions of the host link busy at once;
// the host link, not the kernels, bounds this path (about 1 GB each way per
// [32768, 4096] step).  The parameter gradients are the only values that
// couple the chunks: each chunk writes its own partial dgamma / dbeta row and
// one fb_sum_dim adds them in chunk order.
//
// The handle owns three streams and a few events, nothing else: device staging
// is the caller's (fb_host_ln_device_bytes), as everywhere in this library.
// Host buffers should be pinned (cudaHostRegister / cudaMallocHost); pageable
// memory works but serialises the copies.
#include <new>
#include <vector>

#include "common.cuh"

struct fb_host_ln {
  int device;
  int chunks;
  cudaStream_t h2d, compute, d2h;
  std::vector<cudaEvent_t> ev_in, ev_out;
  cudaEvent_t ev_done, ev_read;
};

using namespace fb;

namespace {
struct Layout {
  uint64_t x, g, y, dx, mu, rs, w, b, part, dwb, ws, ws_bytes, total;
};
uint64_t up256(uint64_t v) { return (v + 255) / 256 * 256; }
Layout layout(uint64_t rows, uint64_t cols, int chunks) {
  Layout L{};
  const uint64_t rc = rows * cols * 4, cr = rows / (uint64_t)chunks;
  uint64_t o = 0;
  L.x = o; o += up256(rc);
  L.g = o; o += up256(rc);
  L.y = o; o += up256(rc);
  L.dx = o; o += up256(rc);
  L.mu = o; o += up256(rows * 4);
  L.rs = o; o += up256(rows * 4);
  L.w = o; o += up256(cols * 4);
  L.b = o; o += up256(cols * 4);
  L.part = o; o += up256((uint64_t)chunks * 2 * cols * 4);
  L.dwb = o; o += up256(2 * cols * 4);
  const uint64_t a = fb_layer_norm_bwd_workspace_bytes(cr, cols), c = fb_reduce_dim_workspace_bytes(1, (uint64_t)chunks, 2 * cols);
  L.ws_bytes = up256((a > c ? a : c) + 16);
  L.ws = o; o += L.ws_bytes;
  L.total = o;
  return L;
}
}  // namespace

extern "C" {

int fb_host_ln_create(int chunks, fb_host_ln** out) {
  if (!out) return fail(FB_ERR_INVALID_ARG, "fb_host_ln_create: null handle slot");
  *out = nullptr;
  if (chunks < 1 || chunks > 64) return fail(FB_ERR_INVALID_ARG, "fb_host_ln_create: chunks must be 1 .. 64");
  fb_host_ln* h = new (std::nothrow) fb_host_ln();
  if (!h) return fail(FB_ERR_CUDA, "fb_host_ln_create: out of host memory");
  h->chunks = chunks;
  cudaError_t e = cudaGetDevice(&h->device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->h2d, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->compute, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->d2h, cudaStreamNonBlocking);
  h->ev_in.resize(chunks);
  h->ev_out.resize(chunks);
  for (int c = 0; c < chunks && e == cudaSuccess; ++c) {
    e = cudaEventCreateWithFlags(&h->ev_in[c], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_out[c], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_read, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventRecord(h->ev_done, h->compute);
  if (e == cudaSuccess) e = cudaEventRecord(h->ev_read, h->d2h);
  if (e != cudaSuccess) {
    delete h;  // the process keeps whatever was created; creation failures are not a steady-state path
    return cuda_fail(e, "fb_host_ln_create");
  }
  *out = h;
  return FB_OK;
}

uint64_t fb_host_ln_device_bytes(uint64_t rows, uint64_t cols, int chunks) {
  if (rows == 0 || cols == 0 || chunks < 1 || rows % (uint64_t)chunks) return 0;
  return layout(rows, cols, chunks).total;
}

int fb_host_ln_run(fb_host_ln* h, uint64_t rows, uint64_t cols, float eps, const float* x, const float* g,
                   const float* weight, const float* bias, float* y, float* dx, float* mean, float* rstd,
                   float* dweight_dbias, void* device_staging, uint64_t staging_bytes) {
  const char* name = "fb_host_ln_run";
  if (!h) return fail(FB_ERR_INVALID_ARG, "%s: null handle", name);
  uint64_t total;
  if (cols == 0 || mul_overflows(rows, cols, &total) || total > (UINT64_MAX >> 4))
    return fail(FB_ERR_INVALID_SHAPE, "%s: bad shape", name);
  if (rows == 0) return FB_OK;
  if (rows % (uint64_t)h->chunks) return fail(FB_ERR_INVALID_SHAPE, "%s: rows must divide into the %d chunks", name, h->chunks);
  if (!x || !g || !weight || !bias || !y || !dx || !mean || !rstd || !dweight_dbias)
    return fail(FB_ERR_INVALID_ARG, "%s: null host buffer", name);
  const Layout L = layout(rows, cols, h->chunks);
  if (!device_staging || staging_bytes < L.total || (reinterpret_cast<uintptr_t>(device_staging) & 255))
    return fail(FB_ERR_WORKSPACE, "%s: needs %llu bytes of 256-byte aligned device staging", name, (unsigned long long)L.total);
  char* d = static_cast<char*>(device_staging);
  auto F = [&](uint64_t off) { return reinterpret_cast<float*>(d + off); };
  const uint64_t cr = rows / (uint64_t)h->chunks, cb = cr * cols * 4;
  // uploads: parameters, then the row chunks of x and g
  FB_CUDA(cudaStreamWaitEvent(h->h2d, h->ev_done, 0));  // the previous call no longer reads the device inputs
  FB_CUDA(cudaMemcpyAsync(F(L.w), weight, cols * 4, cudaMemcpyHostToDevice, h->h2d));
  FB_CUDA(cudaMemcpyAsync(F(L.b), bias, cols * 4, cudaMemcpyHostToDevice, h->h2d));
  for (int c = 0; c < h->chunks; ++c) {
    const uint64_t ro = (uint64_t)c * cr * cols;
    FB_CUDA(cudaMemcpyAsync(F(L.x) + ro, x + ro, cb, cudaMemcpyHostToDevice, h->h2d));
    FB_CUDA(cudaMemcpyAsync(F(L.g) + ro, g + ro, cb, cudaMemcpyHostToDevice, h->h2d));
    FB_CUDA(cudaEventRecord(h->ev_in[c], h->h2d));
  }
  FB_CUDA(cudaStreamWaitEvent(h->compute, h->ev_read, 0));  // the previous call's downloads have left the device outputs
  for (int c = 0; c < h->chunks; ++c) {
    const uint64_t ro = (uint64_t)c * cr * cols, rr = (uint64_t)c * cr;
    FB_CUDA(cudaStreamWaitEvent(h->compute, h->ev_in[c], 0));
    if (int rc = fb_layer_norm_fwd(h->compute, F(L.x) + ro, F(L.w), F(L.b), cr, cols, eps, F(L.y) + ro, nullptr, nullptr,
                                   F(L.mu) + rr, F(L.rs) + rr))
      return rc;
    float* part = F(L.part) + (uint64_t)c * 2 * cols;
    if (int rc = fb_layer_norm_bwd(h->compute, F(L.g) + ro, nullptr, nullptr, F(L.x) + ro, F(L.mu) + rr, F(L.rs) + rr, F(L.w),
                                   cr, cols, F(L.dx) + ro, part, part + cols, d + L.ws, L.ws_bytes))
      return rc;
    FB_CUDA(cudaEventRecord(h->ev_out[c], h->compute));
    FB_CUDA(cudaStreamWaitEvent(h->d2h, h->ev_out[c], 0));
    FB_CUDA(cudaMemcpyAsync(y + ro, F(L.y) + ro, cb, cudaMemcpyDeviceToHost, h->d2h));
    FB_CUDA(cudaMemcpyAsync(dx + ro, F(L.dx) + ro, cb, cudaMemcpyDeviceToHost, h->d2h));
  }
  if (int rc = fb_sum_dim(h->compute, F(L.part), 1, (uint64_t)h->chunks, 2 * cols, F(L.dwb), d + L.ws, L.ws_bytes)) return rc;
  FB_CUDA(cudaEventRecord(h->ev_done, h->compute));
  FB_CUDA(cudaStreamWaitEvent(h->d2h, h->ev_done, 0));
  FB_CUDA(cudaMemcpyAsync(mean, F(L.mu), rows * 4, cudaMemcpyDeviceToHost, h->d2h));
  FB_CUDA(cudaMemcpyAsync(rstd, F(L.rs), rows * 4, cudaMemcpyDeviceToHost, h->d2h));
  FB_CUDA(cudaMemcpyAsync(dweight_dbias, F(L.dwb), 2 * cols * 4, cudaMemcpyDeviceToHost, h->d2h));
  FB_CUDA(cudaEventRecord(h->ev_read, h->d2h));
  return FB_OK;
}

int fb_host_ln_synchronize(fb_host_ln* h) {
  if (!h) return fail(FB_ERR_INVALID_ARG, "fb_host_ln_synchronize: null handle");
  FB_CUDA(cudaStreamSynchronize(h->d2h));
  FB_CUDA(cudaStreamSynchronize(h->compute));
  return FB_OK;
}

int fb_host_ln_destroy(fb_host_ln* h) {
  if (!h) return FB_OK;
  cudaStreamSynchronize(h->d2h);
  cudaStreamSynchronize(h->compute);
  cudaStreamSynchronize(h->h2d);
  for (cudaEvent_t e : h->ev_in) cudaEventDestroy(e);
  for (cudaEvent_t e : h->ev_out) cudaEventDestroy(e);
  cudaEventDestroy(h->ev_done);
  cudaEventDestroy(h->ev_read);
  cudaStreamDestroy(h->h2d);
  cudaStreamDestroy(h->compute);
  cudaStreamDestroy(h->d2h);
  delete h;
  return FB_OK;
}

}  // extern "C"
