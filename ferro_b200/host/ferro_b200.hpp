// Header-only C++ mirror of ferro's device backend seam over libferro_b200.
//
// `fb::CudaBackend` carries the `*_dev` methods of
// `ferro_core::dispatch::Backend` (crates/ferro-core/src/dispatch.rs:199-665)
// that `ferro_cuda::CudaBackend` implements on the memory-bound path
// (crates/ferro-cuda/src/lib.rs:1032-1707): same names, same argument meaning,
// errors as exceptions carrying the variant ferro would return.  It is the
// native host side for callers that are not Rust; the Rust binding a ferro
// maintainer would write is the same few lines per method.
//
// Buffers are `fb::DeviceBuffer` (whole contiguous f32 or i64 device storage,
// dispatch.rs:143-147), allocated with cudaMallocAsync on the backend's one
// non-default stream (lib.rs:308-312).  Everything is asynchronous on that
// stream; `synchronize()` is explicit.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "../../include/ferro_b200.h"

namespace fb {

// ferro_core::Error variants this path can produce (crates/ferro-core/src/error.rs).
struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct InvalidShape : Error { using Error::Error; };
struct Unsupported : Error { using Error::Error; };

inline void check(int rc) {
  if (rc == FB_OK) return;
  const std::string msg = fb_last_error();
  if (rc == FB_ERR_INVALID_SHAPE) throw InvalidShape(msg);
  throw Unsupported(msg);
}
inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Unsupported(std::string("CUDA error: ") + cudaGetErrorString(e) + " at " + what);
}

enum class DType { F32, I64 };

class DeviceBuffer {
 public:
  DeviceBuffer(void* p, size_t len, DType dt, cudaStream_t s) : ptr_(p), len_(len), dtype_(dt), stream_(s) {}
  ~DeviceBuffer() { if (ptr_) cudaFreeAsync(ptr_, stream_); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  size_t len() const { return len_; }
  DType dtype() const { return dtype_; }
  float* f32() const { return static_cast<float*>(ptr_); }
  int64_t* i64() const { return static_cast<int64_t*>(ptr_); }
  void* raw() const { return ptr_; }

 private:
  void* ptr_;
  size_t len_;
  DType dtype_;
  cudaStream_t stream_;
};
using Buf = std::unique_ptr<DeviceBuffer>;

struct UnaryKind { int code; float p0 = 0.0f, p1 = 0.0f; };    // dispatch.rs:18-43
struct BinaryKind { int code; float p0 = 0.0f, p1 = 0.0f; };   // dispatch.rs:68-76
using AdamWStep = fb_adamw_hparams;                            // dispatch.rs:92-100

class CudaBackend {
 public:
  explicit CudaBackend(int ordinal = 0) : ordinal_(ordinal) {
    cuda_check(cudaSetDevice(ordinal), "cudaSetDevice");
    cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  }
  ~CudaBackend() {
    if (scratch_) cudaFree(scratch_);
    if (stream_) cudaStreamDestroy(stream_);
  }
  cudaStream_t stream() const { return stream_; }
  // Waits for the stream, then reads the device status word: a pipelined kernel whose bounded
  // wait gave up has returned early with its outputs incomplete, and this is where the host
  // learns of it (recorded driver errors surface the same way, lib.rs:593-597, 1938-1946).
  void synchronize() {
    cuda_check(cudaStreamSynchronize(stream_), "synchronize");
    const int faults = fb_device_faults(1);
    if (faults > 0)
      throw Unsupported("CUDA error: " + std::to_string(faults) +
                        " bounded device wait(s) gave up; outputs of the kernels launched since the last check are undefined");
  }

  // ---- transfers (lib.rs:571-588, 674-686) ------------------------------------------------
  Buf alloc_uninit(size_t n, DType dt = DType::F32) {
    void* p = nullptr;
    const size_t bytes = n * (dt == DType::F32 ? 4 : 8);
    if (bytes) cuda_check(cudaMallocAsync(&p, bytes, stream_), "cudaMallocAsync");
    return std::make_unique<DeviceBuffer>(p, n, dt, stream_);
  }
  Buf alloc_from_host(const std::vector<float>& data) {
    Buf b = alloc_uninit(data.size());
    if (!data.empty())
      cuda_check(cudaMemcpyAsync(b->raw(), data.data(), data.size() * 4, cudaMemcpyHostToDevice, stream_), "upload");
    synchronize();  // the host vector may go away
    return b;
  }
  Buf alloc_i64_from_host(const std::vector<int64_t>& data) {
    Buf b = alloc_uninit(data.size(), DType::I64);
    if (!data.empty())
      cuda_check(cudaMemcpyAsync(b->raw(), data.data(), data.size() * 8, cudaMemcpyHostToDevice, stream_), "upload");
    synchronize();
    return b;
  }
  std::vector<float> copy_to_host(const DeviceBuffer& b) {
    if (b.dtype() != DType::F32) throw Unsupported("copy_to_host on an i64 buffer");
    std::vector<float> out(b.len());
    if (b.len()) cuda_check(cudaMemcpyAsync(out.data(), b.raw(), b.len() * 4, cudaMemcpyDeviceToHost, stream_), "download");
    synchronize();
    return out;
  }
  std::vector<int64_t> copy_i64_to_host(const DeviceBuffer& b) {
    if (b.dtype() != DType::I64) throw Unsupported("copy_i64_to_host on an f32 buffer");
    std::vector<int64_t> out(b.len());
    if (b.len()) cuda_check(cudaMemcpyAsync(out.data(), b.raw(), b.len() * 8, cudaMemcpyDeviceToHost, stream_), "download");
    synchronize();
    return out;
  }

  // ---- elementwise ----------------------------------------------------------------------------
  Buf unary_dev(UnaryKind k, const DeviceBuffer& x) {
    Buf out = alloc_uninit(x.len());
    check(fb_unary(s(), k.code, k.p0, k.p1, x.f32(), out->f32(), x.len()));
    return out;
  }
  Buf binary_dev(BinaryKind k, const DeviceBuffer& a, const DeviceBuffer& b) {
    if (a.len() != b.len()) throw InvalidShape("binary_dev: length mismatch");
    Buf out = alloc_uninit(a.len());
    check(fb_binary(s(), k.code, k.p0, k.p1, a.f32(), b.f32(), out->f32(), a.len()));
    return out;
  }
  Buf binary_bc_dev(BinaryKind k, const DeviceBuffer& a, const std::vector<uint64_t>& sa, const DeviceBuffer& b,
                    const std::vector<uint64_t>& sb, const std::vector<uint64_t>& out_shape) {
    if (numel(sa) != a.len() || numel(sb) != b.len()) throw InvalidShape("binary_bc_dev: buffer length does not match its shape");
    Buf out = alloc_uninit(numel(out_shape));
    check(fb_binary_bc(s(), k.code, k.p0, k.p1, a.f32(), sa.data(), (int)sa.size(), b.f32(), sb.data(), (int)sb.size(),
                       out->f32(), out_shape.data(), (int)out_shape.size()));
    return out;
  }
  Buf materialize_dev(const DeviceBuffer& x, const std::vector<uint64_t>& shape, const std::vector<int64_t>& strides,
                      int64_t offset) {
    Buf out = alloc_uninit(numel(shape));
    check(fb_materialize(s(), x.f32(), x.len(), strides.data(), offset, shape.data(), (int)shape.size(), out->f32()));
    return out;
  }
  Buf chain_dev(const std::vector<fb_chain_step>& steps, const std::vector<fb_chain_operand>& operands,
                const std::vector<uint64_t>& shape) {
    Buf out = alloc_uninit(numel(shape));
    check(fb_chain(s(), steps.data(), (int)steps.size(), operands.data(), (int)operands.size(), shape.data(),
                   (int)shape.size(), out->f32()));
    return out;
  }

  // ---- in-place family ---------------------------------------------------------------------------
  Buf fill_dev(float value, size_t n) {
    Buf out = alloc_uninit(n);
    check(fb_fill(s(), out->f32(), value, n));
    return out;
  }
  void fill_inplace_dev(DeviceBuffer& dst, float value) { check(fb_fill(s(), dst.f32(), value, dst.len())); }
  void affine_inplace_dev(DeviceBuffer& dst, float mul, float add) { check(fb_affine_inplace(s(), dst.f32(), mul, add, dst.len())); }
  void binary_inplace_dev(BinaryKind k, DeviceBuffer& dst, const DeviceBuffer& src) {
    if (dst.len() != src.len()) throw InvalidShape("binary_inplace_dev: length mismatch");
    check(fb_binary_inplace(s(), k.code, dst.f32(), src.f32(), dst.len()));
  }
  void axpy_inplace_dev(float alpha, DeviceBuffer& dst, const DeviceBuffer& src) {
    if (dst.len() != src.len()) throw InvalidShape("axpy_inplace_dev: length mismatch");
    check(fb_axpy_inplace(s(), alpha, dst.f32(), src.f32(), dst.len()));
  }
  void copy_into_dev(DeviceBuffer& dst, const DeviceBuffer& src) {
    if (dst.len() != src.len()) throw InvalidShape("copy_into_dev: length mismatch");
    check(fb_copy(s(), dst.f32(), src.f32(), dst.len()));
  }
  Buf copy_dev(const DeviceBuffer& src) {
    Buf out = alloc_uninit(src.len());
    check(fb_copy(s(), out->f32(), src.f32(), src.len()));
    return out;
  }
  Buf gather_rows_dev(const DeviceBuffer& w, const DeviceBuffer& idx, uint64_t dim_size, uint64_t inner) {
    if (idx.dtype() != DType::I64) throw Unsupported("gather_rows_dev: indices must be an i64 buffer");
    Buf out = alloc_uninit(idx.len() * inner);
    check(fb_gather_rows(s(), w.f32(), idx.i64(), idx.len(), dim_size, inner, out->f32(), nullptr));
    return out;
  }

  // ---- reductions -------------------------------------------------------------------------------------
  Buf reduce_dev(int kind, const DeviceBuffer& x) {
    Buf out = alloc_uninit(1);
    const uint64_t ws = fb_reduce_workspace_bytes(x.len());
    check(fb_reduce(s(), kind, x.f32(), x.len(), out->f32(), scratch(ws), ws));
    return out;
  }
  Buf sum_dim_dev(const DeviceBuffer& x, const std::vector<uint64_t>& shape, size_t dim) {
    uint64_t o, r, i;
    split(shape, dim, o, r, i);
    Buf out = alloc_uninit(o * i);
    const uint64_t ws = fb_reduce_dim_workspace_bytes(o, r, i);
    check(fb_sum_dim(s(), x.f32(), o, r, i, out->f32(), scratch(ws), ws));
    return out;
  }
  std::pair<Buf, Buf> max_dim_dev(const DeviceBuffer& x, const std::vector<uint64_t>& shape, size_t dim) {
    uint64_t o, r, i;
    split(shape, dim, o, r, i);
    Buf val = alloc_uninit(o * i), idx = alloc_uninit(o * i, DType::I64);
    const uint64_t ws = fb_reduce_dim_workspace_bytes(o, r, i);
    check(fb_max_dim(s(), x.f32(), o, r, i, val->f32(), idx->i64(), scratch(ws), ws));
    return {std::move(val), std::move(idx)};
  }

  // ---- softmax family ------------------------------------------------------------------------------------
  Buf softmax_dev(const DeviceBuffer& x, uint64_t rows, uint64_t cols) {
    Buf y = alloc_uninit(x.len());
    check(fb_softmax_fwd(s(), x.f32(), rows, cols, y->f32()));
    return y;
  }
  Buf log_softmax_dev(const DeviceBuffer& x, uint64_t rows, uint64_t cols) {
    Buf y = alloc_uninit(x.len());
    check(fb_log_softmax_fwd(s(), x.f32(), rows, cols, y->f32()));
    return y;
  }
  Buf softmax_backward_dev(const DeviceBuffer& g, const DeviceBuffer& y, uint64_t rows, uint64_t cols) {
    Buf dx = alloc_uninit(y.len());
    check(fb_softmax_bwd(s(), g.f32(), y.f32(), rows, cols, dx->f32()));
    return dx;
  }
  Buf log_softmax_backward_dev(const DeviceBuffer& g, const DeviceBuffer& y, uint64_t rows, uint64_t cols) {
    Buf dx = alloc_uninit(y.len());
    check(fb_log_softmax_bwd(s(), g.f32(), y.f32(), rows, cols, dx->f32()));
    return dx;
  }

  // ---- LayerNorm --------------------------------------------------------------------------------------------
  // (y, h, stds), dispatch.rs:369-373.
  std::tuple<Buf, Buf, Buf> layer_norm_dev(const DeviceBuffer& x, const DeviceBuffer* w, const DeviceBuffer* b,
                                           uint64_t rows, uint64_t cols, float eps) {
    if (cols == 0 || rows * cols != x.len()) throw InvalidShape("layer_norm_dev: rows x cols does not match the buffer");
    Buf y = alloc_uninit(x.len()), h = alloc_uninit(x.len()), sd = alloc_uninit(rows);
    check(fb_layer_norm_fwd(s(), x.f32(), w ? w->f32() : nullptr, b ? b->f32() : nullptr, rows, cols, eps, y->f32(),
                            h->f32(), sd->f32(), nullptr, nullptr));
    return {std::move(y), std::move(h), std::move(sd)};
  }
  Buf layer_norm_output_dev(const DeviceBuffer& x, const DeviceBuffer* w, const DeviceBuffer* b, uint64_t rows,
                            uint64_t cols, float eps) {
    if (cols == 0 || rows * cols != x.len()) throw InvalidShape("layer_norm_output_dev: rows x cols does not match the buffer");
    Buf y = alloc_uninit(x.len());
    check(fb_layer_norm_fwd(s(), x.f32(), w ? w->f32() : nullptr, b ? b->f32() : nullptr, rows, cols, eps, y->f32(),
                            nullptr, nullptr, nullptr, nullptr));
    return y;
  }
  // (dx, dweight, dbias) from ferro's saved tensors (h, stds).
  std::tuple<Buf, Buf, Buf> layer_norm_backward_dev(const DeviceBuffer& g, const DeviceBuffer& h, const DeviceBuffer& stds,
                                                    const DeviceBuffer* w, uint64_t rows, uint64_t cols) {
    Buf dx = alloc_uninit(g.len()), dw = alloc_uninit(cols), db = alloc_uninit(cols);
    const uint64_t ws = fb_layer_norm_bwd_workspace_bytes(rows, cols);
    check(fb_layer_norm_bwd(s(), g.f32(), h.f32(), stds.f32(), nullptr, nullptr, nullptr, w ? w->f32() : nullptr, rows,
                            cols, dx->f32(), dw->f32(), db->f32(), scratch(ws), ws));
    return {std::move(dx), std::move(dw), std::move(db)};
  }

  // Tensor::residual_layernorm (crates/ferro-core/src/fused_ops.rs:106-231): (y, h, stds) of layer_norm(x + residual).
  std::tuple<Buf, Buf, Buf> residual_layer_norm_dev(const DeviceBuffer& x, const DeviceBuffer& residual, const DeviceBuffer* w,
                                                    const DeviceBuffer* b, uint64_t rows, uint64_t cols, float eps) {
    if (residual.len() != x.len()) throw InvalidShape("residual_layer_norm_dev: x and residual differ in length");
    Buf y = alloc_uninit(x.len()), h = alloc_uninit(x.len()), sd = alloc_uninit(rows);
    check(fb_residual_layer_norm_fwd(s(), x.f32(), residual.f32(), w ? w->f32() : nullptr, b ? b->f32() : nullptr, rows,
                                     cols, eps, y->f32(), h->f32(), sd->f32(), nullptr, nullptr, nullptr));
    return {std::move(y), std::move(h), std::move(sd)};
  }

  // RmsNorm::forward (crates/ferro-core/src/nn.rs:272-279) as one kernel: (y, rstd); and its backward: (dx, dweight).
  std::pair<Buf, Buf> rms_norm_dev(const DeviceBuffer& x, const DeviceBuffer* w, uint64_t rows, uint64_t cols, float eps) {
    Buf y = alloc_uninit(x.len()), rs = alloc_uninit(rows);
    check(fb_rms_norm_fwd(s(), x.f32(), w ? w->f32() : nullptr, rows, cols, eps, y->f32(), rs->f32()));
    return {std::move(y), std::move(rs)};
  }
  std::pair<Buf, Buf> rms_norm_backward_dev(const DeviceBuffer& g, const DeviceBuffer& x, const DeviceBuffer& rstd,
                                            const DeviceBuffer* w, uint64_t rows, uint64_t cols) {
    Buf dx = alloc_uninit(g.len()), dw = alloc_uninit(cols);
    const uint64_t ws = fb_layer_norm_bwd_workspace_bytes(rows, cols);
    check(fb_rms_norm_bwd(s(), g.f32(), x.f32(), rstd.f32(), w ? w->f32() : nullptr, rows, cols, dx->f32(), dw->f32(),
                          scratch(ws), ws));
    return {std::move(dx), std::move(dw)};
  }

  // ---- optimizers ----------------------------------------------------------------------------------------------
  void sgd_step_dev(DeviceBuffer& p, DeviceBuffer& v, const DeviceBuffer& g, float lr, float momentum, bool nesterov) {
    check(fb_sgd_step(s(), p.f32(), v.f32(), g.f32(), p.len(), lr, momentum, nesterov ? 1 : 0));
  }
  void adamw_step_dev(DeviceBuffer& p, DeviceBuffer& m, DeviceBuffer& v, const DeviceBuffer& g, AdamWStep hp) {
    check(fb_adamw_step(s(), p.f32(), m.f32(), v.f32(), g.f32(), p.len(), hp));
  }
  void adamw_step_capturable_dev(DeviceBuffer& p, DeviceBuffer& m, DeviceBuffer& v, const DeviceBuffer& g,
                                 const DeviceBuffer& t, float lr, float beta1, float beta2, float eps, float wd) {
    check(fb_adamw_step_capturable(s(), p.f32(), m.f32(), v.f32(), g.f32(), t.f32(), p.len(), lr, beta1, beta2, eps, wd));
  }
  void scalar_increment_dev(DeviceBuffer& t, float beta1, float beta2) { check(fb_scalar_increment(s(), t.f32(), beta1, beta2)); }

 private:
  fb_stream_t s() const { return reinterpret_cast<fb_stream_t>(stream_); }
  static uint64_t numel(const std::vector<uint64_t>& shape) {
    uint64_t n = 1;
    for (uint64_t d : shape) n *= d;
    return n;
  }
  static void split(const std::vector<uint64_t>& shape, size_t dim, uint64_t& o, uint64_t& r, uint64_t& i) {
    if (dim >= shape.size()) throw InvalidShape("dim out of range");
    o = i = 1;
    for (size_t d = 0; d < dim; ++d) o *= shape[d];
    for (size_t d = dim + 1; d < shape.size(); ++d) i *= shape[d];
    r = shape[dim];
  }
  // Scratch owned by the host side of the ABI, grown on demand; all users are ordered on one stream.
  void* scratch(uint64_t bytes) {
    if (bytes <= scratch_bytes_) return scratch_;
    synchronize();
    if (scratch_) cudaFree(scratch_);
    cuda_check(cudaMalloc(&scratch_, bytes), "cudaMalloc(scratch)");
    scratch_bytes_ = bytes;
    return scratch_;
  }
  int ordinal_;
  cudaStream_t stream_ = nullptr;
  void* scratch_ = nullptr;
  uint64_t scratch_bytes_ = 0;
};

}  // namespace fb
