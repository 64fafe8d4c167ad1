/* libferro_b200 - C ABI of the B200 (sm_100a) kernels for ferro's
 * memory-bound device path.
 *
 * Every entry point is what one `*_dev` method of ferro's
 * `ferro_core::dispatch::Backend` trait (crates/ferro-core/src/dispatch.rs:199-665),
 * as implemented by `CudaBackend` (crates/ferro-cuda/src/lib.rs:1032-1707),
 * would call instead of launching an nvrtc-compiled kernel.  The comment on
 * each declaration names the trait method and the launch site it replaces.
 *
 * Conventions (the contract of that seam, restated):
 *  - All buffers are device pointers to f32 (i64 where said), allocated by the
 *    caller, inputs AND outputs; the library allocates nothing, frees nothing
 *    and keeps no pointer after the call returns.  Outputs may be
 *    uninitialised on entry: every element a call claims is written.
 *  - Calls are asynchronous on `stream`; there is no host synchronisation, no
 *    allocation and no module loading on the launch path, so calls may be
 *    recorded into a CUDA graph (crates/ferro-cuda/src/lib.rs:891-901).
 *  - The return value is an fb_status (ferro_b200_kinds.h).  Non-zero means
 *    nothing was launched and nothing was modified; fb_last_error() gives the
 *    message for the calling thread.  Nothing traps, aborts or asserts.
 *  - A zero-length problem returns FB_OK without launching
 *    (crates/ferro-cuda/src/lib.rs:485-489).
 *  - Sizes are uint64_t element counts, strides are int64_t element strides,
 *    ranks are at most FB_MAX_RANK.
 *  - Ops that need scratch take (workspace, workspace_bytes); the matching
 *    fb_*_workspace_bytes() says how much.  Scratch contents are undefined
 *    before and after a call; two calls that share scratch must not overlap.
 */
#ifndef FERRO_B200_H
#define FERRO_B200_H

#include <stdint.h>

#include "ferro_b200_kinds.h"

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define FB_API
#else
#define FB_API __attribute__((visibility("default")))
#endif

#define FB_MAX_RANK 16
#define FB_VERSION 1

typedef struct CUstream_st* fb_stream_t; /* cudaStream_t */

/* ---- library ----------------------------------------------------------- */
FB_API int fb_version(void);
/* Message of the last failing call on this thread ("" if none).  Plays the
 * role of cuda_err()'s text, crates/ferro-cuda/src/lib.rs:55-60. */
FB_API const char* fb_last_error(void);
/* Number of kernels this library has launched in this process; the
 * counterpart of pointwise_launch_counts(), crates/ferro-cuda/src/lib.rs:425-447. */
FB_API uint64_t fb_launch_count(void);

/* Kernels that stage rows with asynchronous bulk copies wait on completion
 * barriers with a bounded spin; a wait that gives up makes the kernel return
 * early and bumps a device-side counter instead of hanging the GPU.  This call
 * synchronises the device, returns the counter for the current device (0 on a
 * healthy run, -1 if it cannot be read) and clears it when `reset` is set.
 * After a non-zero reading, everything written by the pipelined LayerNorm /
 * RMS-norm kernels launched since the previous reading is undefined: the
 * rows a CTA had not reached are missing from y / dx, and its partial
 * dweight / dbias row was not written although the finalize still summed it.
 * Inputs are never modified.  A host layer should read this word wherever it
 * synchronises (the mirrors in ferro_b200/backend.py and host/ferro_b200.hpp
 * do, in synchronize() and before every read-back) and fail the step.
 * The reference reports device trouble as recorded driver errors,
 * crates/ferro-cuda/src/lib.rs:1938-1946. */
FB_API int fb_device_faults(int reset);
/* Self-test of that reporting path (no counterpart in the reference): launches
 * one warp that waits, with the same bounded wait the pipelined kernels use,
 * on a barrier nothing completes; after `limit_ms` (1 .. 1000) the wait gives
 * up, the kernel returns and fb_device_faults() reads 1.  The context stays
 * usable: nothing traps, nothing spins without a limit. */
FB_API int fb_selftest_bounded_wait(fb_stream_t stream, uint32_t limit_ms);

/* ---- contiguous elementwise --------------------------------------------- */
/* Backend::unary_dev, dispatch.rs:285; launch_elementwise lib.rs:476-501. */
FB_API int fb_unary(fb_stream_t stream, int kind, float p0, float p1, const float* x, float* out,
                    uint64_t n);
/* Backend::binary_dev, dispatch.rs:289; lib.rs:1082-1099.  `out` may alias
 * `a` or `b` (same-index combination only). */
FB_API int fb_binary(fb_stream_t stream, int kind, float p0, float p1, const float* a,
                     const float* b, float* out, uint64_t n);
/* Backend::binary_bc_dev, dispatch.rs:332; lib.rs:1132-1169: `a` and `b` are
 * whole contiguous buffers of shapes sa / sb that broadcast (numpy rules) to
 * out_shape. */
FB_API int fb_binary_bc(fb_stream_t stream, int kind, float p0, float p1, const float* a,
                        const uint64_t* sa, int rank_a, const float* b, const uint64_t* sb,
                        int rank_b, float* out, const uint64_t* out_shape, int rank_out);
/* New capability behind the same seam: operands addressed as ferro views
 * (storage, shape, stride, offset in elements; tensor.rs:213-227), so a
 * transposed / sliced / broadcast device tensor is computed in place instead
 * of taking the download path of tensor.rs:1692-1700.  `out` is row-major
 * over `shape`.  `x_len` / `a_len` / `b_len` are the storage lengths used to
 * bounds-check the views before launch. */
FB_API int fb_unary_strided(fb_stream_t stream, int kind, float p0, float p1, const float* x,
                            uint64_t x_len, const int64_t* x_strides, int64_t x_offset,
                            const uint64_t* shape, int rank, float* out);
FB_API int fb_binary_strided(fb_stream_t stream, int kind, float p0, float p1, const float* a,
                             uint64_t a_len, const int64_t* a_strides, int64_t a_offset,
                             const float* b, uint64_t b_len, const int64_t* b_strides,
                             int64_t b_offset, const uint64_t* shape, int rank, float* out);
/* Backend::materialize_dev, dispatch.rs:625; lib.rs:1589-1624. */
FB_API int fb_materialize(fb_stream_t stream, const float* x, uint64_t x_len,
                          const int64_t* strides, int64_t offset, const uint64_t* shape, int rank,
                          float* out);

/* ---- fused pointwise programs -------------------------------------------- */
/* Backend::chain_dev, dispatch.rs:349; launch_chain lib.rs:819-872,
 * generator kernels.rs:177-235.  One launch evaluates a small program per
 * output element over up to FB_CHAIN_MAX_OPERANDS strided operands.  The
 * program is a list of fb_chain_step for a two-register machine: V is the
 * running value (ferro's chain seed threaded through the steps), T a
 * temporary that lets an operand pass through unary steps before it meets V
 * (ferro's ChainStepRef, dispatch.rs:107-121, is the subset that never
 * touches T).  The result is V after the last step. */
#define FB_CHAIN_MAX_STEPS 32
#define FB_CHAIN_MAX_OPERANDS 6
enum fb_chain_opcode {
  FB_CH_LOAD = 0,   /* dst = operand[src]                                  */
  FB_CH_UNARY = 1,  /* dst = unary(kind, p0, p1, dst)                      */
  FB_CH_BINARY = 2, /* dst = binary(kind, p0, p1, lhs, rhs); see `src`     */
  FB_CH_IMM = 3     /* dst = p0                                            */
};
enum fb_chain_reg { FB_CH_V = 0, FB_CH_T = 1 };
/* Where FB_CH_BINARY takes its right-hand side (left is always dst), or,
 * with FB_CH_SWAP added, its left-hand side (right is then dst). */
enum fb_chain_src {
  FB_CH_SRC_OTHER_REG = 0, /* the register that is not dst */
  FB_CH_SRC_IMM = 1,       /* p1 is the operand; kinds that need p1 cannot use this */
  FB_CH_SRC_OPERAND0 = 8,  /* FB_CH_SRC_OPERAND0 + k loads operand k directly */
  FB_CH_SWAP = 64
};
typedef struct fb_chain_step {
  int32_t opcode; /* fb_chain_opcode */
  int32_t dst;    /* fb_chain_reg */
  int32_t kind;   /* fb_unary_kind / fb_binary_kind */
  int32_t src;    /* FB_CH_LOAD: operand index; FB_CH_BINARY: fb_chain_src */
  float p0, p1;
} fb_chain_step;
typedef struct fb_chain_operand {
  const float* ptr;
  uint64_t len;                 /* storage length, for bounds checking */
  int64_t offset;               /* element offset of the view */
  int64_t strides[FB_MAX_RANK]; /* element strides over the output shape, 0 = broadcast */
} fb_chain_operand;
FB_API int fb_chain(fb_stream_t stream, const fb_chain_step* steps, int n_steps,
                    const fb_chain_operand* operands, int n_operands, const uint64_t* shape,
                    int rank, float* out);
/* Chains listed in the build-time catalogue (csrc/chain_programs.def) run as
 * compiled straight-line programs; any other chain runs on an interpreter of
 * the same step list.  ferro compiles every chain at run time through nvrtc
 * (kernels.rs:177-235); this switch turns the compiled forms off (0) or on
 * (non-zero, the default) for the whole process and returns the previous
 * setting, so that the two runners can be compared on one chain.  Results
 * are identical either way. */
FB_API int fb_chain_catalogue(int enable);

/* ---- in-place family (dispatch.rs:448-549; lib.rs:1346-1451) ---------------- */
/* Backend::fill_dev / fill_inplace_dev, dispatch.rs:428, 511. */
FB_API int fb_fill(fb_stream_t stream, float* dst, float value, uint64_t n);
/* Backend::affine_inplace_dev, dispatch.rs:515: dst = dst * mul + add. */
FB_API int fb_affine_inplace(fb_stream_t stream, float* dst, float mul, float add, uint64_t n);
/* Backend::binary_inplace_dev, dispatch.rs:520: dst = dst kind src; dst may be src. */
FB_API int fb_binary_inplace(fb_stream_t stream, int kind, float* dst, const float* src,
                             uint64_t n);
/* Backend::axpy_inplace_dev, dispatch.rs:529: dst += alpha * src. */
FB_API int fb_axpy_inplace(fb_stream_t stream, float alpha, float* dst, const float* src,
                           uint64_t n);
/* Backend::copy_into_dev / copy_dev, dispatch.rs:540-549 (kernel copy, so it
 * records into a graph like copy_source, kernels.rs:375-383). */
FB_API int fb_copy(fb_stream_t stream, float* dst, const float* src, uint64_t n);
/* Backend::gather_rows_dev, dispatch.rs:656; lib.rs:1656-1706:
 * out[o, :] = w[idx[o], :] for n i64 indices over a [dim_size, inner] table.
 * An index outside [0, dim_size) writes zeros for that row and stores
 * 1 + its position into *bad_index (device i64, may be NULL; the caller
 * zeroes it), never a trap. */
FB_API int fb_gather_rows(fb_stream_t stream, const float* w, const int64_t* idx, uint64_t n,
                          uint64_t dim_size, uint64_t inner, float* out, int64_t* bad_index);

/* ---- reductions ------------------------------------------------------------ */
/* Backend::reduce_dev, dispatch.rs:358; lib.rs:1185-1230.  out is one f32.
 * n == 0: Sum writes 0, Mean writes NaN (lib.rs:1191-1199). */
FB_API uint64_t fb_reduce_workspace_bytes(uint64_t n);
FB_API int fb_reduce(fb_stream_t stream, int kind, const float* x, uint64_t n, float* out,
                     void* workspace, uint64_t workspace_bytes);
/* Backend::sum_dim_dev, dispatch.rs:417; lib.rs:1232-1258: x is row-major
 * [outer, red, inner]; out is [outer, inner] (the keepdim layout).
 * fb_mean_dim multiplies the sum by (1/red as f32), ops_ext/mean_dim.rs:24-30.
 * fb_max_dim has no trait method today (axis extrema exist only as the host
 * loop of ops_ext/argmax.rs:42-63); values and/or i64 indices may be NULL. */
FB_API uint64_t fb_reduce_dim_workspace_bytes(uint64_t outer, uint64_t red, uint64_t inner);
FB_API int fb_sum_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red,
                      uint64_t inner, float* out, void* workspace, uint64_t workspace_bytes);
FB_API int fb_mean_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red,
                       uint64_t inner, float* out, void* workspace, uint64_t workspace_bytes);
FB_API int fb_max_dim(fb_stream_t stream, const float* x, uint64_t outer, uint64_t red,
                      uint64_t inner, float* values, int64_t* indices, void* workspace,
                      uint64_t workspace_bytes);

/* ---- softmax family (rows x cols, last dim) ---------------------------------- */
/* Backend::softmax_dev / log_softmax_dev, dispatch.rs:396, 406; run_row_softmax
 * lib.rs:606-640.  One launch, one read of x. */
FB_API int fb_softmax_fwd(fb_stream_t stream, const float* x, uint64_t rows, uint64_t cols,
                          float* y);
FB_API int fb_log_softmax_fwd(fb_stream_t stream, const float* x, uint64_t rows, uint64_t cols,
                              float* y);
/* The backward closures ops_ext/softmax.rs:33-38 (dx = y * (g - sum(g*y))) and
 * ops_ext/log_softmax.rs:33-37 (dx = g - exp(y) * sum(g)), each as one launch
 * instead of four. dx may alias g. */
FB_API int fb_softmax_bwd(fb_stream_t stream, const float* g, const float* y, uint64_t rows,
                          uint64_t cols, float* dx);
FB_API int fb_log_softmax_bwd(fb_stream_t stream, const float* g, const float* y, uint64_t rows,
                              uint64_t cols, float* dx);
/* Softmax over a prologue: y = softmax(act(x + bias) * scale) along the last
 * dim, bias [cols] broadcast over rows (may be NULL), act = identity or relu
 * (`relu` != 0).  The fused form of add -> relu -> mul -> softmax
 * (ops.rs:19-28, 99-109, 44-58; ops_ext/softmax.rs:15-56). */
FB_API int fb_bias_act_scale_softmax_fwd(fb_stream_t stream, const float* x, const float* bias,
                                         int relu, float scale, uint64_t rows, uint64_t cols,
                                         float* y);
/* Its backward: dx = relu_backward((y * (g - sum(g*y))) * scale, x + bias),
 * and, when dbias != NULL, dbias[c] = sum over rows of dx[:, c] (the
 * unbroadcast of tensor.rs:2173-2185).  Scratch (only needed for dbias):
 * fb_softmax_fused_bwd_workspace_bytes(rows, cols). */
FB_API uint64_t fb_softmax_fused_bwd_workspace_bytes(uint64_t rows, uint64_t cols);
FB_API int fb_bias_act_scale_softmax_bwd(fb_stream_t stream, const float* g, const float* y,
                                         const float* x, const float* bias, int relu, float scale,
                                         uint64_t rows, uint64_t cols, float* dx, float* dbias,
                                         void* workspace, uint64_t workspace_bytes);

/* Fused log_softmax + NLL over i64 class ids, mean reduction: what
 * nn::cross_entropy_indices (crates/ferro-core/src/nn.rs:793-814) computes
 * through a host-built one-hot matrix (nn.rs:403-432) and four device ops.
 *   loss      [1]      = -(1/rows) * sum_r logp[r, targets[r]]
 *   row_max   [rows], row_lse [rows]  saved for the backward (lse = ln sum exp(x - max))
 *   argmax    [rows] i64, optional: first NaN wins, ties keep the lowest index
 *                      (ops_ext/argmax.rs:42-63)
 *   bad_target [1] i64 device word, optional, caller-zeroed: set to 1 + row of a
 *                      target outside [0, cols); that row contributes 0 loss.
 * Masked logits (-inf beside finite ones) give finite statistics, loss and
 * gradient: the target's log-probability is gathered, as in ferro's Python
 * functional.cross_entropy (crates/ferro-py/python/ferro/nn/functional.py:419-444).
 * The one-hot composition of nn.rs:380-400 would multiply -inf by the zeros of
 * the one-hot matrix and report NaN for the whole batch; a row that is -inf
 * throughout is NaN in both.
 * Scratch: fb_nll_workspace_bytes(rows). */
FB_API uint64_t fb_nll_workspace_bytes(uint64_t rows);
FB_API int fb_log_softmax_nll_fwd(fb_stream_t stream, const float* logits, const int64_t* targets,
                                  uint64_t rows, uint64_t cols, float* loss, float* row_max,
                                  float* row_lse, int64_t* argmax, int64_t* bad_target,
                                  void* workspace, uint64_t workspace_bytes);
/* dlogits[r, k] = (exp(x - max - lse) - [k == targets[r]]) * (grad_scale / rows);
 * grad_scale is the upstream gradient of the scalar loss (1 for loss.backward()). */
FB_API int fb_log_softmax_nll_bwd(fb_stream_t stream, const float* logits, const int64_t* targets,
                                  const float* row_max, const float* row_lse, float grad_scale,
                                  uint64_t rows, uint64_t cols, float* dlogits);

/* ---- index-driven ops ----------------------------------------------------------------- */
/* Tensor::gather (crates/ferro-core/src/ops_ext/gather.rs:12-111, a host loop
 * over to_vec() copies whatever the device): out[c] = x[c with c[dim] replaced
 * by index[c]] for every coordinate c of the index tensor.  x is whole and
 * row-major over in_shape, index (i64) and out are whole over out_shape, same
 * rank, out_shape[d] <= in_shape[d] for d != dim (gather.rs:38-48).  An index
 * outside [0, in_shape[dim]) writes 0 and stores 1 + its flat position into
 * *bad_index (device i64, may be NULL; the caller zeroes it), never a trap. */
FB_API int fb_gather_dim(fb_stream_t stream, const float* x, const uint64_t* in_shape, const int64_t* index,
                         const uint64_t* out_shape, int rank, int dim, float* out, int64_t* bad_index);
/* Its backward (gather.rs:103-110): gx = 0, then gx[position gathered from] += g
 * for every element of g, duplicates accumulating.  No float atomics: the
 * thread that owns a column of gx walks the index along `dim` in order, so
 * additions happen in the order of the host loop and the result equals it bit
 * for bit.  gx is whole over in_shape and is written in full. */
FB_API int fb_scatter_add_dim(fb_stream_t stream, const float* g, const int64_t* index, const uint64_t* in_shape,
                              const uint64_t* out_shape, int rank, int dim, float* gx, int64_t* bad_index);
/* Segment algebra over a CSR topology (crates/ferro-core/src/segment.rs;
 * device plan and kernel crates/ferro-cuda/src/segment.rs:20-89, segment.cu:1-40).
 * csr is the device table ferro's plan uploads: groups + 1 offsets followed by
 * the edge ids of every group in ascending edge order; fb_segment_csr_build
 * fills the same table in HOST memory from one segment id per edge (an id
 * >= groups is FB_ERR_INVALID_SHAPE).  x is [edges, width]:
 *   fb_segment_sum          out[s, f] = sum over the edges of group s (edge order: bit-identical
 *                           to the CPU loop of segment.rs:132-141); empty groups are 0
 *   fb_segment_sum_bwd      dx[e, f] = g[group of e, f]
 *   fb_segment_softmax_fwd  per group and feature, softmax over the group's edges; *not_finite
 *                           (device int, caller-zeroed, may be NULL) is set to 1 when an input is not
 *                           finite, which ferro reports as an error (segment.rs:222-225)
 *   fb_segment_softmax_bwd  dx = y * (g - sum over the group of g * y)
 * A group is owned by one warp (a slice of a warp when width < 32), lanes along the features. */
FB_API int fb_segment_csr_build(const uint64_t* ids, uint64_t edges, uint64_t groups, int64_t* csr_host);
FB_API int fb_segment_sum(fb_stream_t stream, const float* x, const int64_t* csr, uint64_t groups, uint64_t edges,
                          uint64_t width, float* out);
FB_API int fb_segment_sum_bwd(fb_stream_t stream, const float* g, const int64_t* csr, uint64_t groups,
                              uint64_t edges, uint64_t width, float* dx);
FB_API int fb_segment_softmax_fwd(fb_stream_t stream, const float* x, const int64_t* csr, uint64_t groups,
                                  uint64_t edges, uint64_t width, float* y, int* not_finite);
FB_API int fb_segment_softmax_bwd(fb_stream_t stream, const float* g, const float* y, const int64_t* csr,
                                  uint64_t groups, uint64_t edges, uint64_t width, float* dx);

/* ---- reductions and softmax on views ------------------------------------------------ */
/* A ferro tensor view: storage, shape, element strides (0 = broadcast, negative
 * allowed) and element offset (crates/ferro-core/src/tensor.rs:213-227).  The
 * view is bounds-checked against `len` before anything is launched. */
typedef struct fb_view {
  const float* ptr;              /* storage base */
  uint64_t len;                  /* storage length in elements */
  int64_t offset;                /* element offset of the view's first element */
  int32_t rank;                  /* 1 .. FB_MAX_RANK */
  uint64_t shape[FB_MAX_RANK];
  int64_t strides[FB_MAX_RANK];
} fb_view;
/* sum / mean / max over one dim of a view.  try_raw_sum_dim downloads every
 * device tensor that is not whole and contiguous and reduces it on the host
 * (tensor.rs:2057-2104); these keep a transposed, sliced or broadcast input on
 * the GPU.  `out` is row-major over the view's shape with `dim` set to 1 (the
 * keepdim layout of Backend::sum_dim_dev, dispatch.rs:417); mean multiplies by
 * (1/n as f32) (ops_ext/mean_dim.rs:24-30); max follows ops_ext/argmax.rs:42-63
 * (first NaN wins, ties keep the lowest index), values and/or indices may be
 * NULL.  A whole contiguous view takes the kernels of fb_sum_dim / fb_max_dim,
 * which is what the scratch is for: fb_reduce_view_workspace_bytes. */
FB_API uint64_t fb_reduce_view_workspace_bytes(const fb_view* x, int dim);
FB_API int fb_sum_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* out, void* workspace,
                           uint64_t workspace_bytes);
FB_API int fb_mean_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* out, void* workspace,
                            uint64_t workspace_bytes);
FB_API int fb_max_dim_view(fb_stream_t stream, const fb_view* x, int dim, float* values, int64_t* indices,
                           void* workspace, uint64_t workspace_bytes);
/* softmax / log_softmax over any dim of a view, and their backward.
 * raw_row_softmax (tensor.rs:2124-2140) declines unless the tensor is whole,
 * contiguous and reduced over its last dim, which sends every other case to
 * the host loops of ops_ext/softmax.rs:68-109 and log_softmax.rs:57-100; here
 * they stay on the device.  Outputs are row-major over the view's shape.  The
 * backward takes the upstream gradient and the saved forward result as two
 * views of the same shape (their strides may differ). */
FB_API int fb_softmax_view_fwd(fb_stream_t stream, const fb_view* x, int dim, float* y);
FB_API int fb_log_softmax_view_fwd(fb_stream_t stream, const fb_view* x, int dim, float* y);
FB_API int fb_softmax_view_bwd(fb_stream_t stream, const fb_view* g, const fb_view* y, int dim, float* dx);
FB_API int fb_log_softmax_view_bwd(fb_stream_t stream, const fb_view* g, const fb_view* y, int dim, float* dx);

/* ---- LayerNorm ------------------------------------------------------------------ */
/* Backend::layer_norm_dev / layer_norm_output_dev, dispatch.rs:369-380;
 * lib.rs:1260-1314; kernel layer_norm.cu:1-42.  weight / bias are [cols] or
 * NULL.  y is required; h (normalised input), stds, mean, rstd are each
 * written when non-NULL (ferro saves h and stds; mean and rstd = 1/std are
 * the compact statistics for fb_layer_norm_bwd). */
FB_API int fb_layer_norm_fwd(fb_stream_t stream, const float* x, const float* weight,
                             const float* bias, uint64_t rows, uint64_t cols, float eps, float* y,
                             float* h, float* stds, float* mean, float* rstd);
/* The backward closure ops_ext/layer_norm.rs:127-139 (host form :28-68) as
 * one pass: dxh = g*w; dx = (dxh - mean(dxh) - h*mean(dxh*h)) / std;
 * dweight = sum_rows g*h; dbias = sum_rows g.  Either pass the saved h and
 * stds (x = mean = rstd = NULL), or x with mean and rstd (h = stds = NULL).
 * dweight / dbias may be NULL.  Scratch: fb_layer_norm_bwd_workspace_bytes,
 * 16-byte aligned; it may be NULL only when neither dweight nor dbias is
 * asked for and the row has a fused form (cols a multiple of 4, at most 16384,
 * 16-byte aligned buffers): rows outside that take two kernels that pass
 * per-row statistics through the scratch. */
FB_API uint64_t fb_layer_norm_bwd_workspace_bytes(uint64_t rows, uint64_t cols);
FB_API int fb_layer_norm_bwd(fb_stream_t stream, const float* g, const float* h,
                             const float* stds, const float* x, const float* mean,
                             const float* rstd, const float* weight, uint64_t rows, uint64_t cols,
                             float* dx, float* dweight, float* dbias, void* workspace,
                             uint64_t workspace_bytes);

/* LayerNorm of a sum: y = layer_norm(x + residual) * weight + bias, which is
 * Tensor::residual_layernorm (host loops today, crates/ferro-core/src/
 * fused_ops.rs:106-231).  Outputs as fb_layer_norm_fwd; the backward is
 * fb_layer_norm_bwd on the saved (h, stds), or on (sum_out, mean, rstd) when
 * sum_out (optional, [rows, cols]) is requested: its dx is the gradient of
 * both x and residual (fused_ops.rs:222-226).  Rows up to 8192 columns add
 * on the fly (x and residual read once, nothing else moved); wider or
 * unaligned rows take one extra pass for the sum. */
FB_API int fb_residual_layer_norm_fwd(fb_stream_t stream, const float* x, const float* residual,
                                      const float* weight, const float* bias, uint64_t rows,
                                      uint64_t cols, float eps, float* y, float* h, float* stds,
                                      float* mean, float* rstd, float* sum_out);

/* RMS normalisation over the last dimension: y = x * rstd * weight with
 * rstd = 1 / sqrt(mean(x^2) + eps).  ferro's RmsNorm module composes it from
 * mul, mean_dim, add, sqrt, div and mul (crates/ferro-core/src/nn.rs:255-283:
 * six launches and five intermediates forward, the autograd chain of those
 * backward); here it is one kernel each way, the LayerNorm kernels run without
 * their mean.  weight may be NULL; rstd is [rows] and is what the backward
 * needs besides x.  Backward: dx, and dweight[c] = sum over rows of
 * g * x * rstd when dweight is non-NULL; scratch as for fb_layer_norm_bwd
 * (fb_layer_norm_bwd_workspace_bytes). */
FB_API int fb_rms_norm_fwd(fb_stream_t stream, const float* x, const float* weight, uint64_t rows,
                           uint64_t cols, float eps, float* y, float* rstd);
FB_API int fb_rms_norm_bwd(fb_stream_t stream, const float* g, const float* x, const float* rstd,
                           const float* weight, uint64_t rows, uint64_t cols, float* dx,
                           float* dweight, void* workspace, uint64_t workspace_bytes);

/* LayerNorm backward that allocates nothing and takes no scratch argument.
 * No counterpart in the reference.  It exists for callers that cannot provide
 * device scratch at the call site: a step whose memory pool is frozen (graph
 * replay, real-time loops), a plug-in without access to the host's allocator,
 * a process that must not grow.  Same arguments and results as
 * fb_layer_norm_bwd; the partial column sums live in a fixed device array of
 * FB_LN_STATIC_SCRATCH_BYTES inside the library image, which every GPU that
 * loads the library keeps until the process exits.  Limits and rules:
 *  - a problem whose fb_layer_norm_bwd_workspace_bytes(rows, cols) exceeds
 *    FB_LN_STATIC_SCRATCH_BYTES is refused with FB_ERR_WORKSPACE (nothing is
 *    launched); [32768, 4096] needs about 14.5 MB and fits;
 *  - the first call on each device looks up the array's device address (a
 *    host-side runtime query, done with that device current and cached), so
 *    make that first call before starting any stream capture;
 *  - every call on a device shares the one array and it keeps the previous
 *    call's contents; nothing in it needs clearing, but two calls that can
 *    run at the same time on one GPU (different streams) race on it: keep
 *    them on one stream or order them with events. */
#define FB_LN_STATIC_SCRATCH_BYTES (16u << 20)
FB_API int fb_layer_norm_bwd_static(fb_stream_t stream, const float* g, const float* h,
                                    const float* stds, const float* x, const float* mean,
                                    const float* rstd, const float* weight, uint64_t rows,
                                    uint64_t cols, float* dx, float* dweight, float* dbias);

/* ---- optimizers ---------------------------------------------------------------------- */
/* Backend::sgd_step_dev, dispatch.rs:551; lib.rs:1453-1496; math dispatch.rs:477-483. */
FB_API int fb_sgd_step(fb_stream_t stream, float* p, float* v, const float* g, uint64_t n,
                       float lr, float momentum, int nesterov);
/* Backend::adamw_step_dev, dispatch.rs:563; lib.rs:1498-1547; math dispatch.rs:489-503.
 * Bitwise equal to the host loop. */
typedef struct fb_adamw_hparams {
  float lr, beta1, beta2, bc1, bc2, eps, weight_decay;
} fb_adamw_hparams; /* AdamWStep, dispatch.rs:92-100 */
FB_API int fb_adamw_step(fb_stream_t stream, float* p, float* m, float* v, const float* g,
                         uint64_t n, fb_adamw_hparams hp);
/* Backend::adamw_step_capturable_dev / scalar_increment_dev, dispatch.rs:581-604;
 * lib.rs:1721-1813: t is a 3-float device buffer [step, bc1, bc2]. */
FB_API int fb_adamw_step_capturable(fb_stream_t stream, float* p, float* m, float* v,
                                    const float* g, const float* t, uint64_t n, float lr,
                                    float beta1, float beta2, float eps, float weight_decay);
FB_API int fb_scalar_increment(fb_stream_t stream, float* t, float beta1, float beta2);
/* One launch for a whole parameter list (Adam::update loops over parameters
 * and launches once per tensor, crates/ferro-core/src/optim.rs:707-771).
 * `table` is a DEVICE array of n_tensors fb_tensor_quad records the caller
 * filled; every tensor takes the same hyper-parameters.  `g_scale` multiplies
 * each gradient on load: 1 leaves it unchanged; 1/world turns the sum an
 * all-reduce produced into the mean of crates/ferro-core/src/ddp.rs:138-157. */
typedef struct fb_tensor_quad {
  float* p;
  float* m; /* Adam first moment, or the SGD velocity */
  float* v; /* Adam second moment; unused by SGD */
  const float* g;
  uint64_t n;
} fb_tensor_quad;
FB_API int fb_adamw_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                          uint64_t total_elems, fb_adamw_hparams hp, float g_scale);
FB_API int fb_sgd_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                        uint64_t total_elems, float lr, float momentum, int nesterov,
                        float g_scale);

/* Global-norm gradient clipping without a host read-back.  ferro computes the
 * norm with one device reduction and one scalar download per parameter and
 * scales every gradient on the host's say-so (global_grad_norm / clip_scale,
 * crates/ferro-core/src/optim.rs:1395-1425).  Here the whole parameter list is
 * one reduction, the factor stays on the device, and the fused update reads it:
 *   fb_grad_sumsq_multi   sumsq[0] = sum over the table of (g * g_scale)^2
 *   fb_clip_scale         norm = sqrt(sumsq); scale = max/norm if norm > max
 *                         and norm > 0, else 1 (norm_out may be NULL)
 *   fb_*_multi_clipped    the multi-tensor update with every gradient
 *                         multiplied by g_scale and then by clip_scale[0]
 *                         (clip_scale NULL: same as the unclipped entry). */
FB_API uint64_t fb_grad_norm_workspace_bytes(void);
FB_API int fb_grad_sumsq_multi(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                               uint64_t total_elems, float g_scale, float* sumsq, void* workspace,
                               uint64_t workspace_bytes);
FB_API int fb_clip_scale(fb_stream_t stream, const float* sumsq, float max_norm, float* norm_out,
                         float* scale_out);
FB_API int fb_adamw_multi_clipped(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                                  uint64_t total_elems, fb_adamw_hparams hp, float g_scale,
                                  const float* clip_scale);
FB_API int fb_sgd_multi_clipped(fb_stream_t stream, const fb_tensor_quad* table, int n_tensors,
                                uint64_t total_elems, float lr, float momentum, int nesterov,
                                float g_scale, const float* clip_scale);

/* ---- MLP glue of the data-parallel step ------------------------------------------------ */
/* Linear::forward's `+ bias` (nn.rs:157-160) fused with the activation that
 * follows, which is also Tensor::bias_add_activation (a host loop today,
 * crates/ferro-core/src/fused_ops.rs:57-104): out = act(x + bias[cols]) over
 * [rows, cols].  `act` (fused_ops.rs:10-16): 0 identity, 1 relu, 2 gelu (tanh
 * form), 3 silu.  out may alias x. */
FB_API int fb_bias_act_fwd(fb_stream_t stream, const float* x, const float* bias, int act,
                           uint64_t rows, uint64_t cols, float* out);
/* Its backward (fused_ops.rs:88-103): dx = g * act'(z) with z = x + bias
 * recomputed from the pre-bias x (relu: the exact mask of ReluBackward;
 * identity: dx = g, x may be NULL), dbias[c] = sum_rows dx[:, c].  dx may
 * alias g; dx == NULL skips writing it (bias-only gradient).  Scratch:
 * fb_reduce_dim_workspace_bytes(1, rows, cols). */
FB_API int fb_bias_act_bwd(fb_stream_t stream, const float* g, const float* x, const float* bias,
                           int act, uint64_t rows, uint64_t cols, float* dx, float* dbias,
                           void* workspace, uint64_t workspace_bytes);
/* mse_loss forward and gradient in one pass (ops_ext/mse_loss.rs:9-11 =
 * sub -> square -> mean; square is a host round trip today, square.rs:16-19):
 * loss[0] = mean((pred-target)^2); dpred = grad_scale * 2 (pred-target) / n.
 * Scratch: fb_reduce_workspace_bytes(n). */
FB_API int fb_mse_fwd_bwd(fb_stream_t stream, const float* pred, const float* target, uint64_t n,
                          float grad_scale, float* loss, float* dpred, void* workspace,
                          uint64_t workspace_bytes);

/* ---- host-buffer entry ---------------------------------------------------------------- */
/* LayerNorm forward + backward for tensors that live in HOST memory: what a
 * ferro user gets from alloc_from_host -> layer_norm_dev -> backward ->
 * copy_to_host (crates/ferro-cuda/src/lib.rs:571-588, 674-686, 1260-1287), but
 * cut into row chunks and run as a three-stage pipeline (upload chunk k + 1,
 * compute chunk k, download chunk k - 1) so both directions of the host link
 * are busy at once.  Outputs: y, dx [rows, cols], mean, rstd [rows],
 * dweight_dbias [2, cols] (dweight then dbias), all in host memory.
 * The handle holds three streams and their events (created with the current
 * device current; the only allocation-like calls, made once); device staging is
 * the caller's: fb_host_ln_device_bytes(rows, cols, chunks) bytes, 256-byte
 * aligned; rows must divide by chunks.  fb_host_ln_run returns after enqueueing;
 * the host outputs are complete after fb_host_ln_synchronize.  Pin the host
 * buffers for full transfer speed. */
typedef struct fb_host_ln fb_host_ln;
FB_API int fb_host_ln_create(int chunks, fb_host_ln** out);
FB_API uint64_t fb_host_ln_device_bytes(uint64_t rows, uint64_t cols, int chunks);
FB_API int fb_host_ln_run(fb_host_ln* h, uint64_t rows, uint64_t cols, float eps, const float* x, const float* g,
                          const float* weight, const float* bias, float* y, float* dx, float* mean, float* rstd,
                          float* dweight_dbias, void* device_staging, uint64_t staging_bytes);
FB_API int fb_host_ln_synchronize(fb_host_ln* h);
FB_API int fb_host_ln_destroy(fb_host_ln* h);

/* ---- checkpoint wire format ---------------------------------------------------------- */
/* safetensors images written from and read into device buffers.  ferro's
 * to_safetensors_bytes / from_safetensors_bytes (crates/ferro-core/src/
 * safetensors.rs:36-94, 96-230) and the optimizer snapshots built on them
 * (Adam::snapshot, crates/ferro-core/src/optim.rs:828-847: flat f32 arrays
 * "m.i", "v.i" and a scalar "t.i" per parameter, prefixed "optim." by the
 * checkpoint; "velocity.i" for SGD) download every buffer into a Vec and
 * re-encode it value by value.  Here only the header text is built on the
 * host; tensor bytes travel straight between device memory and their place in
 * the caller's host image, one asynchronous copy per tensor on `stream` (pin
 * the image for full transfer speed; synchronise the stream before reading or
 * freeing it).  The bytes are exactly ferro's: header length, JSON entries in
 * the order given, space padding to a multiple of 8, little-endian data.
 *   fb_safetensors_image_bytes  size of the image; data_offsets (n + 1 slots, may be NULL)
 *                               receives every tensor's byte offset inside the image
 *   fb_safetensors_write        lays the header down and copies each sources[i]
 *                               (device pointers when sources_on_device, else host)
 *   fb_safetensors_count / _entry   walk a finished image: name, dtype, shape and the byte
 *                               range of entry `index` (header order; "__metadata__" skipped)
 *   fb_safetensors_read         copies tensor `tensor_name` to dst after checking dtype and size
 * A malformed image is FB_ERR_FORMAT with the reader's message (Error::Format in ferro). */
enum fb_st_dtype { FB_ST_F32 = 0, FB_ST_I64 = 1 };
typedef struct fb_st_entry {
  const char* name;
  int32_t dtype; /* fb_st_dtype */
  int32_t rank;
  uint64_t shape[FB_MAX_RANK];
} fb_st_entry;
FB_API uint64_t fb_safetensors_image_bytes(const fb_st_entry* entries, int n, uint64_t* data_offsets);
FB_API int fb_safetensors_write(fb_stream_t stream, const fb_st_entry* entries, int n, const void* const* sources,
                                int sources_on_device, void* image, uint64_t image_bytes);
FB_API int fb_safetensors_count(const void* image, uint64_t image_bytes);
FB_API int fb_safetensors_entry(const void* image, uint64_t image_bytes, int index, char* name_out,
                                uint64_t name_cap, fb_st_entry* entry_out, uint64_t* data_begin,
                                uint64_t* data_end);
FB_API int fb_safetensors_read(fb_stream_t stream, const void* image, uint64_t image_bytes,
                               const char* tensor_name, int dtype, uint64_t numel, void* dst, int dst_on_device);

/* ---- DLPack exchange ------------------------------------------------------------------- */
/* Device tensors handed to and taken from other libraries as DLPack "dltensor"
 * capsules, without host staging.  ferro's binding exports a CUDA tensor
 * zero-copy (kDLCUDA, base pointer + byte offset of the view) behind a host
 * synchronisation of the allocation's stream, and imports a kDLCUDA tensor
 * through the host: download, gather through the strides, upload
 * (crates/ferro-py/src/dlpack.rs:216-256, 355-511, 535-600;
 * crates/ferro-py/src/lib.rs:32-46, 2071-2103).  These entries keep both
 * directions on the device:
 *   fb_dlpack_export       builds a DLManagedTensor (kDLCUDA, f32 or i64, shape, optional
 *                          element strides, byte offset of a view) that borrows `data`; its
 *                          deleter calls release(owner) once and frees the descriptor.  No
 *                          CUDA call is made.
 *   fb_dlpack_handoff      what __dlpack__(stream) owes the consumer: work enqueued on
 *                          `producer` so far is ordered before whatever the consumer enqueues
 *                          next on its stream (an event, no host wait).  Consumer token as in
 *                          the protocol: absent or 1 = legacy default stream, 2 = per-thread
 *                          default stream, another positive value = a stream handle; 0
 *                          (ambiguous) and negative values (-1, no synchronisation, is not
 *                          offered) are FB_ERR_INVALID_ARG, as in ferro.
 *   fb_dlpack_describe     validates a DLManagedTensor the way dlpack.rs does (device type,
 *                          dtype f32 / i64, negative rank or extents, element-count overflow,
 *                          strides reaching outside the described span, null data,
 *                          misaligned offset; same messages) and reports pointer, shape and
 *                          element strides.
 *   fb_dlpack_import_into  copies the described tensor into a contiguous device buffer on
 *                          `stream`: one device-to-device copy when it is compact, the
 *                          strided-copy kernel (fb_materialize) for a strided f32 CUDA tensor;
 *                          a kDLCPU tensor is uploaded.  The caller got the capsule from
 *                          producer.__dlpack__(stream = its own stream), so the producer has
 *                          already ordered its work before this stream.
 *   fb_dlpack_delete       runs the capsule's deleter (the consumer's duty once it is done,
 *                          and the capsule destructor's for a capsule nobody consumed). */
typedef void (*fb_dlpack_release_fn)(void* owner);
typedef struct fb_dlpack_desc {
  void* data; /* first element (byte offset applied); NULL for an empty tensor */
  int32_t on_device; /* 1: kDLCUDA, 0: kDLCPU */
  int32_t device_id;
  int32_t dtype; /* fb_st_dtype */
  int32_t rank;
  int32_t contiguous; /* compact row-major (extents of 1 ignored) */
  int32_t reserved;
  uint64_t numel;
  uint64_t shape[FB_MAX_RANK];
  int64_t strides[FB_MAX_RANK]; /* elements; filled in when the producer left them out */
} fb_dlpack_desc;
FB_API int fb_dlpack_export(const void* data, uint64_t byte_offset, int dtype, int ndim, const int64_t* shape,
                            const int64_t* strides, int device_ordinal, void* owner, fb_dlpack_release_fn release,
                            void** managed_out);
FB_API int fb_dlpack_handoff(fb_stream_t producer, int has_consumer, int64_t consumer);
FB_API int fb_dlpack_describe(const void* managed, fb_dlpack_desc* out);
FB_API int fb_dlpack_import_into(fb_stream_t stream, const void* managed, void* dst, uint64_t dst_bytes);
FB_API void fb_dlpack_delete(void* managed);

/* ---- seeded inputs ------------------------------------------------------------------- */
/* ferro_core::Rng (crates/ferro-core/src/rng.rs:12-70): splitmix64-seeded
 * xorshift128+; uniform() = top 24 bits / 2^24; normal() = Box-Muller cosine
 * branch on two uniforms with u1 clamped to 1e-9.  Tensor::randn / rand fill
 * row-major on the host (crates/ferro-core/src/tensor.rs:365-372), so these
 * write HOST buffers: out[i] = shift + scale * draw, draws consumed in index
 * order.  fb_rng_fill_rowscaled_normal draws one uniform u per row first and
 * writes normal() * (lo + span * u) along the row; fb_rng_fill_index writes
 * floor(uniform() * classes) as i64 (ferro's generator has no integer draw).
 * Large fills use every host thread for the transcendental part; the values
 * do not depend on the thread count. */
typedef struct fb_rng { uint64_t s0, s1; } fb_rng; /* Rng::state(), rng.rs:28 */
FB_API void fb_rng_seed(fb_rng* rng, uint64_t seed);
/* Advances the state by `draws` uniforms (a normal takes two) without
 * producing values: how one rank of a sharded run reaches its rows of a
 * tensor that ferro would have filled in one piece. */
FB_API void fb_rng_skip(fb_rng* rng, uint64_t draws);
FB_API float fb_rng_uniform(fb_rng* rng);
FB_API float fb_rng_normal(fb_rng* rng);
FB_API int fb_rng_fill_uniform(fb_rng* rng, float* out, uint64_t n, float scale, float shift);
FB_API int fb_rng_fill_normal(fb_rng* rng, float* out, uint64_t n, float scale, float shift);
FB_API int fb_rng_fill_rowscaled_normal(fb_rng* rng, float* out, uint64_t rows, uint64_t cols, float lo,
                                        float span);
FB_API int fb_rng_fill_index(fb_rng* rng, int64_t* out, uint64_t n, uint64_t classes);

/* ---- data-parallel gradient exchange -------------------------------------------------- */
/* The collective behind Ddp::average (crates/ferro-core/src/ddp.rs:127-160,
 * the seam named at ddp.rs:9-13), which today downloads every replica's
 * gradients, sums them on the host and divides by the replica count.  Here
 * there is one process per GPU and the exchange is an NCCL all-reduce, over
 * NVLink, of flat f32 gradient buckets in place on the stream given (a side
 * stream, so that it overlaps the rest of backward).  NCCL is bound at run
 * time (the file named by the FB_NCCL_LIBRARY environment variable, else
 * "libnccl.so.2"), so the library loads without it and a world of one never
 * touches it.
 *
 *   fb_ddp_unique_id       rank 0 fills FB_DDP_UNIQUE_ID_BYTES bytes; the host
 *                          carries them to every rank by its own means
 *   fb_ddp_comm_init       every rank, with its GPU current: joins the world
 *                          and returns a handle (world == 1: id may be NULL)
 *   fb_ddp_allreduce_bucket   bucket[i] = sum over ranks, in place.  The mean is
 *                          the caller's: g_scale = 1/world in fb_adamw_multi /
 *                          fb_sgd_multi folds it into the update
 *   fb_ddp_allreduce_buckets  the same for a list of buckets as one NCCL group
 *   fb_ddp_average_bucket  sum, then an IEEE divide by the replica count:
 *                          exactly `s / n` of ddp.rs:154, for callers with no
 *                          fused optimizer behind the exchange
 *   fb_ddp_poll            FB_OK while the communicator is healthy; FB_ERR_COMM
 *                          (with NCCL's text) once ncclCommGetAsyncError or an
 *                          earlier call has reported a failure.  Cheap, host
 *                          only: call it between steps
 *   fb_ddp_comm_abort      tears a communicator down without waiting for
 *                          outstanding collectives (after a failure or when a
 *                          peer has left); fb_ddp_comm_destroy is the orderly
 *                          end.  Both free the handle.
 * Errors: a failed NCCL call returns FB_ERR_COMM and marks the handle broken;
 * every later exchange on it is refused before anything is enqueued.  No call
 * here waits on the device or on a peer. */
#define FB_DDP_UNIQUE_ID_BYTES 128
typedef struct fb_ddp_comm fb_ddp_comm;
FB_API int fb_ddp_unique_id(void* id);
FB_API int fb_ddp_comm_init(const void* id, int rank, int world, fb_ddp_comm** out);
FB_API int fb_ddp_rank(const fb_ddp_comm* comm);
FB_API int fb_ddp_world(const fb_ddp_comm* comm);
FB_API int fb_ddp_nccl_version(void); /* NCCL's version code, -1 if NCCL cannot be loaded */
FB_API int fb_ddp_allreduce_bucket(fb_ddp_comm* comm, fb_stream_t stream, float* bucket, uint64_t n);
FB_API int fb_ddp_allreduce_buckets(fb_ddp_comm* comm, fb_stream_t stream, float* const* buckets,
                                    const uint64_t* lens, int n_buckets);
FB_API int fb_ddp_average_bucket(fb_ddp_comm* comm, fb_stream_t stream, float* bucket, uint64_t n);
FB_API int fb_ddp_poll(fb_ddp_comm* comm);
FB_API int fb_ddp_comm_abort(fb_ddp_comm* comm);
FB_API int fb_ddp_comm_destroy(fb_ddp_comm* comm);

#ifdef __cplusplus
}
#endif
#endif
