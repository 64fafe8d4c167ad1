// DLPack exchange of device tensors without host staging.
//
// ferro's Python binding exports a CUDA tensor zero-copy (kDLCUDA, the
// allocation's base pointer plus a byte offset for views) behind a
// conservative fence - it synchronises the allocation's stream on the host -
// and imports a kDLCUDA tensor by downloading it, gathering through the
// strides on the host and uploading the result
// (crates/ferro-py/src/dlpack.rs:1-20, 216-256, 355-511, 535-600;
// crates/ferro-py/src/lib.rs:32-46, 2071-2103).  Here both directions stay on
// the device and on streams: the export hands the producer's work over to the
// consumer's stream with an event (no host synchronisation), the import
// gathers a strided producer tensor into a contiguous buffer with the
// library's own strided-copy kernel.  The descriptor checks are the ones
// dlpack.rs makes, with its messages.
//
// The structs below are the DLPack C ABI (dlpack.h, version 0.x "dltensor"
// capsules), restated.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace {

struct DLDevice { int32_t device_type; int32_t device_id; };
struct DLDataType { uint8_t code; uint8_t bits; uint16_t lanes; };
struct DLTensor {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
};
struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(DLManagedTensor*);
};

constexpr int32_t kDLCPU = 1, kDLCUDA = 2;
constexpr uint8_t kDLInt = 0, kDLFloat = 2;

struct Owner {  // manager_ctx of the tensors this library exports
  void* owner;
  fb_dlpack_release_fn release;
  int64_t dims[2 * FB_MAX_RANK];  // shape, then strides
};

void exported_deleter(DLManagedTensor* m) {
  if (!m) return;
  Owner* o = static_cast<Owner*>(m->manager_ctx);
  if (o) {
    if (o->release) o->release(o->owner);
    free(o);
  }
  free(m);
}

}  // namespace

using namespace fb;

extern "C" {

int fb_dlpack_export(const void* data, uint64_t byte_offset, int dtype, int ndim, const int64_t* shape,
                     const int64_t* strides, int device_ordinal, void* owner, fb_dlpack_release_fn release,
                     void** managed_out) {
  const char* name = "fb_dlpack_export";
  if (!managed_out) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  *managed_out = nullptr;
  if (dtype != FB_ST_F32 && dtype != FB_ST_I64) return fail(FB_ERR_UNSUPPORTED, "%s: dtype %d is not f32 or i64", name, dtype);
  if (ndim < 0 || ndim > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 0..%d", name, ndim, FB_MAX_RANK);
  if (ndim && !shape) return fail(FB_ERR_INVALID_ARG, "%s: null shape", name);
  if (device_ordinal < 0) return fail(FB_ERR_INVALID_ARG, "%s: negative device ordinal", name);
  const uint64_t width = dtype == FB_ST_F32 ? 4 : 8;
  if (byte_offset % width) return fail(FB_ERR_INVALID_ARG, "%s: view offset is not element-aligned", name);
  uint64_t numel = 1;
  for (int d = 0; d < ndim; ++d) {
    if (shape[d] < 0) return fail(FB_ERR_INVALID_SHAPE, "%s: negative extent in dimension %d", name, d);
    if (mul_overflows(numel, (uint64_t)shape[d], &numel) || numel > (UINT64_MAX >> 4))
      return fail(FB_ERR_INVALID_SHAPE, "%s: element count overflows", name);
  }
  if (numel && !data) return fail(FB_ERR_INVALID_ARG, "%s: CUDA buffer has null device pointer", name);
  DLManagedTensor* m = static_cast<DLManagedTensor*>(calloc(1, sizeof(DLManagedTensor)));
  Owner* o = static_cast<Owner*>(calloc(1, sizeof(Owner)));
  if (!m || !o) {
    free(m);
    free(o);
    return fail(FB_ERR_UNSUPPORTED, "%s: out of host memory", name);
  }
  o->owner = owner;
  o->release = release;
  for (int d = 0; d < ndim; ++d) {
    o->dims[d] = shape[d];
    if (strides) o->dims[FB_MAX_RANK + d] = strides[d];
  }
  m->dl_tensor.data = const_cast<void*>(data);
  m->dl_tensor.device = DLDevice{kDLCUDA, device_ordinal};
  m->dl_tensor.ndim = ndim;
  m->dl_tensor.dtype = DLDataType{dtype == FB_ST_F32 ? kDLFloat : kDLInt, (uint8_t)(width * 8), 1};
  m->dl_tensor.shape = o->dims;
  m->dl_tensor.strides = strides ? o->dims + FB_MAX_RANK : nullptr;  // NULL: compact row-major
  m->dl_tensor.byte_offset = byte_offset;
  m->manager_ctx = o;
  m->deleter = exported_deleter;
  *managed_out = m;
  return FB_OK;
}

void fb_dlpack_delete(void* managed) {
  DLManagedTensor* m = static_cast<DLManagedTensor*>(managed);
  if (m && m->deleter) m->deleter(m);
}

int fb_dlpack_handoff(fb_stream_t producer, int has_consumer, int64_t consumer) {
  const char* name = "fb_dlpack_handoff";
  // __dlpack__(stream): None and 1 are the legacy default stream, 2 the per-thread default stream, any
  // other positive value a stream handle; 0 is ambiguous and -1 (no synchronisation) is not offered
  // (crates/ferro-py/src/lib.rs:32-46).
  cudaStream_t to;
  if (!has_consumer || consumer == 1) to = cudaStreamLegacy;
  else if (consumer == 2) to = cudaStreamPerThread;
  else if (consumer == 0) return fail(FB_ERR_INVALID_ARG, "%s: CUDA DLPack stream 0 is ambiguous; use None, 1, or 2", name);
  else if (consumer < 0)
    return fail(FB_ERR_INVALID_ARG,
                "%s: CUDA DLPack stream must be a positive pointer-sized integer; no-sync (-1) is unsupported", name);
  else to = reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(consumer));
  if (to == producer) return FB_OK;
  cudaEvent_t ev;
  FB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, producer);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(to, ev, 0);
  cudaEventDestroy(ev);  // the wait, once enqueued, does not need the handle
  if (e != cudaSuccess) return cuda_fail(e, name);
  return FB_OK;
}

int fb_dlpack_describe(const void* managed, fb_dlpack_desc* out) {
  const char* name = "fb_dlpack_describe";
  if (!managed || !out) return fail(FB_ERR_INVALID_ARG, "%s: null dltensor capsule", name);
  const DLTensor& t = static_cast<const DLManagedTensor*>(managed)->dl_tensor;
  memset(out, 0, sizeof(*out));
  if (t.device.device_type != kDLCPU && t.device.device_type != kDLCUDA)
    return fail(FB_ERR_UNSUPPORTED, "%s: only CPU (kDLCPU) and CUDA (kDLCUDA) DLPack tensors are supported", name);
  const bool f32 = t.dtype.code == kDLFloat && t.dtype.bits == 32 && t.dtype.lanes == 1;
  const bool i64 = t.dtype.code == kDLInt && t.dtype.bits == 64 && t.dtype.lanes == 1;
  if (!f32 && !i64) return fail(FB_ERR_UNSUPPORTED, "%s: unsupported DLPack dtype; expected float32 or int64", name);
  if (t.ndim < 0) return fail(FB_ERR_INVALID_SHAPE, "%s: DLPack tensor has negative ndim", name);
  if (t.ndim > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d above %d", name, t.ndim, FB_MAX_RANK);
  if (t.ndim > 0 && !t.shape) return fail(FB_ERR_INVALID_ARG, "%s: DLPack tensor has null shape", name);
  uint64_t nonzero = 1;
  bool empty = false;
  for (int d = 0; d < t.ndim; ++d) {
    const int64_t e = t.shape[d];
    if (e < 0) return fail(FB_ERR_INVALID_SHAPE, "%s: DLPack tensor has negative extent (%lld) in dimension %d", name, (long long)e, d);
    if (e == 0) empty = true;
    // the product of the nonzero extents is checked even when a zero axis would mask an overflow
    if (mul_overflows(nonzero, (uint64_t)(e ? e : 1), &nonzero))
      return fail(FB_ERR_INVALID_SHAPE, "%s: DLPack tensor element count overflows usize", name);
    out->shape[d] = (uint64_t)e;
  }
  const uint64_t numel = empty ? 0 : nonzero;
  const uint64_t width = f32 ? 4 : 8;
  if (numel > (uint64_t)INT64_MAX / width) return fail(FB_ERR_INVALID_SHAPE, "%s: DLPack tensor byte count exceeds allocation capacity", name);
  // Strides are in elements.  Every reachable offset must stay inside [0, numel) of the described
  // span, or a gather would read outside the producer's buffer.
  bool contiguous = true;
  if (t.strides) {
    __int128 lo = 0, hi = 0;
    int64_t expect = 1;
    for (int d = t.ndim - 1; d >= 0; --d) {
      const int64_t s = t.strides[d];
      out->strides[d] = s;
      if (numel) {
        const __int128 span = ((__int128)t.shape[d] - 1) * s;
        if (span < 0) lo += span; else hi += span;
        if (t.shape[d] != 1 && s != expect) contiguous = false;
        expect *= t.shape[d];
      }
    }
    if (numel && (lo < 0 || hi >= (__int128)numel))
      return fail(FB_ERR_INVALID_SHAPE, "%s: DLPack tensor strides reach outside the described element range", name);
  } else {
    int64_t s = 1;
    for (int d = t.ndim - 1; d >= 0; --d) {
      out->strides[d] = s;
      s *= (int64_t)(t.shape[d] ? t.shape[d] : 1);
    }
  }
  if (numel && !t.data) return fail(FB_ERR_INVALID_ARG, "%s: DLPack tensor has null data pointer", name);
  if (t.byte_offset % width) return fail(FB_ERR_INVALID_ARG, "%s: DLPack byte_offset is not element-aligned", name);
  if (t.device.device_type == kDLCUDA && t.device.device_id < 0)
    return fail(FB_ERR_INVALID_ARG, "%s: DLPack tensor has negative device_id", name);
  const uintptr_t addr = reinterpret_cast<uintptr_t>(t.data) + t.byte_offset;
  if (numel && addr % width) return fail(FB_ERR_INVALID_ARG, "%s: DLPack data pointer is not element-aligned", name);
  out->data = numel ? reinterpret_cast<void*>(addr) : nullptr;
  out->on_device = t.device.device_type == kDLCUDA;
  out->device_id = t.device.device_id;
  out->dtype = f32 ? FB_ST_F32 : FB_ST_I64;
  out->rank = t.ndim;
  out->numel = numel;
  out->contiguous = contiguous ? 1 : 0;
  return FB_OK;
}

int fb_dlpack_import_into(fb_stream_t stream, const void* managed, void* dst, uint64_t dst_bytes) {
  const char* name = "fb_dlpack_import_into";
  fb_dlpack_desc d;
  if (int rc = fb_dlpack_describe(managed, &d)) return rc;
  const uint64_t width = d.dtype == FB_ST_F32 ? 4 : 8;
  if (dst_bytes != d.numel * width)
    return fail(FB_ERR_INVALID_SHAPE, "%s: destination holds %llu bytes, the tensor %llu", name,
                (unsigned long long)dst_bytes, (unsigned long long)(d.numel * width));
  if (d.numel == 0) return FB_OK;
  if (!dst) return fail(FB_ERR_INVALID_ARG, "%s: null destination", name);
  if (d.contiguous) {
    FB_CUDA(cudaMemcpyAsync(dst, d.data, dst_bytes, d.on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream));
    return FB_OK;
  }
  if (!d.on_device || d.dtype != FB_ST_F32)
    return fail(FB_ERR_UNSUPPORTED, "%s: a strided tensor is gathered on the device for float32 CUDA input only", name);
  // The span the strides can reach is [0, numel) elements from `data` (checked above).
  return fb_materialize(stream, static_cast<const float*>(d.data), d.numel, d.strides, 0, d.shape, d.rank,
                        static_cast<float*>(dst));
}

}  // extern "C"
