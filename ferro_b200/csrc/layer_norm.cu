// Fused LayerNorm forward and backward over the last dimension.
//
// Roofline: HBM.  Algorithmic bytes per row of `cols` f32:
//   forward            read x, write y                      8 * cols  (+ 4 per saved statistic,
//                                                            + 4 * cols if the normalised input h is saved)
//   backward           read g and h (or x), write dx        12 * cols (+ the per-CTA partial
//                                                            dweight / dbias rows, about 2 %)
// Fast path (cols % 4 == 0, cols <= 131072 forward / 65536 backward, 16-byte
// aligned rows): the row lives in the registers of a group of G threads
// (row_cfg) or, for the widest rows, of a thread block cluster
// (layer_norm_cluster.cuh), so x is read from HBM exactly once; the mean is
// taken first, then the centred sum of squares, both from registers (the
// accuracy of a two-pass variance at one-pass traffic).  Values are shifted by the row's first element before anything is
// summed, which is what keeps rows with a huge common offset (1e8, 1e20)
// exact - the same device the reference kernel uses (layer_norm.cu:1-2, 12 of
// crates/ferro-cuda/src) with f64 sums; here the sums stay f32 because the
// shifted, centred values no longer cancel.
// Generic path (any cols, any alignment): one CTA per row, three sweeps over
// the row, the second and third served by L2.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "pipe.cuh"
#include "reduce.cuh"

namespace fb {

template <int G>
constexpr int ln_threads() { return G < 256 ? 256 : G; }

// ------------------------------------------------------------------ forward
// One row per group of G threads, ITEMS float4 per thread, one CTA per block
// of rows on a full grid (the hardware scheduler hands out row blocks in
// address order; see grid_full).  EXACT: cols == 4 * G * ITEMS, so every
// column test folds away.  The affine epilogue is one multiply by 1/std and
// one fused multiply-add per element.
// MODE 0: LayerNorm; 1: RMS normalisation (no shift, no mean); 2: LayerNorm of x + res, the sum
// optionally stored to sum_out (residual_layernorm, crates/ferro-core/src/fused_ops.rs:106-231).
template <int G, int ITEMS, bool EXACT, int MODE>
__global__ void __launch_bounds__(ln_threads<G>(), ((ITEMS > 4 || (MODE == 2 && ITEMS == 4)) ? 1024 : (ITEMS <= 2 && G >= 256 ? 2048 : 1536)) / ln_threads<G>())  // 4 float4: 42 registers, six 256-thread CTAs per SM (the residual form, which has two arrays in flight: 64 registers, four CTAs); 2 float4 of a 256-thread row: 32 registers, eight
ln_fwd_reg_kernel(const float* __restrict__ x, const float* __restrict__ w,
                  const float* __restrict__ b, uint64_t rows, uint32_t cols, float eps,
                  float* __restrict__ y, float* __restrict__ h, float* __restrict__ stds,
                  float* __restrict__ mean, float* __restrict__ rstd, const float* __restrict__ res,
                  float* __restrict__ sum_out) {
  constexpr bool RMS = MODE == 1;
  constexpr int T = ln_threads<G>();
  constexpr int R = T / G;  // rows per CTA per iteration
  __shared__ float red_a[T / 32], red_b[T / 32];
  const uint32_t cols4 = cols / 4;
  const int grp = threadIdx.x / G, lane = threadIdx.x % G;
  const uint64_t nblk = (rows + R - 1) / R;
  const float inv_d = 1.0f / (float)cols;
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t row = blk * R + grp;
    const bool live = R == 1 || row < rows;
    const float* xr = x + row * cols;
    float4 v[ITEMS];
    float x0 = (live && !RMS) ? __ldg(xr) : 0.0f;  // RMS normalisation: no shift, no mean
    if constexpr (MODE == 2) {
      if (live) x0 += __ldg(res + row * cols);
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      v[k] = (live && (EXACT || c < cols4)) ? ld_stream4(xr + c * 4) : make_float4(x0, x0, x0, x0);
    }
    if constexpr (MODE == 2) {
      float4 r[ITEMS];  // all residual loads issued before the first is used
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        r[k] = (live && (EXACT || c < cols4)) ? ld_stream4(res + row * cols + c * 4) : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (live && (EXACT || c < cols4)) {
          v[k].x += r[k].x; v[k].y += r[k].y; v[k].z += r[k].z; v[k].w += r[k].w;
          if (sum_out) st_stream4(sum_out + row * cols + c * 4, v[k]);
        }
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      v[k].x -= x0; v[k].y -= x0; v[k].z -= x0; v[k].w -= x0;
      s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float md = RMS ? 0.0f : group_sum<G>(s, red_a) * inv_d;  // mean of the shifted row
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      v[k].x -= md; v[k].y -= md; v[k].z -= md; v[k].w -= md;
      if (EXACT || c < cols4) q += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
    const float var = group_sum<G>(q, red_b) * inv_d;
    const float sd = sqrtf(var + eps);
    const float rs = 1.0f / sd;
    if (live) {
      if (lane == 0) {
        if (stds) stds[row] = sd;
        if (mean) mean[row] = x0 + md;
        if (rstd) rstd[row] = rs;
      }
      float* yr = y + row * cols;
      float* hr = h ? h + row * cols : nullptr;
      const float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f), zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (EXACT || c < cols4) {
          const float4 hv = make_float4(v[k].x * rs, v[k].y * rs, v[k].z * rs, v[k].w * rs);
          if (hr) st_stream4(hr + c * 4, hv);
          const float4 wv = w ? __ldg(reinterpret_cast<const float4*>(w) + c) : one;
          const float4 bv = b ? __ldg(reinterpret_cast<const float4*>(b) + c) : zero;
          st_stream4(yr + c * 4, make_float4(fmaf(hv.x, wv.x, bv.x), fmaf(hv.y, wv.y, bv.y),
                                             fmaf(hv.z, wv.z, bv.z), fmaf(hv.w, wv.w, bv.w)));
        }
      }
    }
  }
}

// The same kernel with the row on any number of warps (1 .. 16, not only a power of two) and any number of
// float4 per thread from 4 to 8, for widths the power-of-two geometries fit badly.  Those pad the row to
// 4 * G * ITEMS columns; the padding costs nothing in HBM traffic, but a kernel of this kind is bound by the
// bytes its resident warps keep in flight, and dead slots are bytes not in flight: with 2560 columns on 256 x 4
// (62 % of the slots used) the forward ran at 77 % of the copy rate, 640 columns on 32 x 8 at 78 %, 10240 on
// 512 x 8 at 76 %.  Here 2560 columns are 4 warps x 5 float4, 640 columns 1 warp x 5, 10240 columns
// 10 warps x 8: no dead slots (82 / 88 / 76 / 86 / 87 / 83 % at 640 / 768 / 1280 / 3072 / 5120 / 10240 columns,
// from 78 / 83 / 71 / 83 / 83 / 76 %).  blockDim.x = 32 * warps_per_row * rows per CTA, at most 512.
// (A named barrier per row - bar.sync 1 + row, 32 * wpr - instead of the CTA-wide one, so that the rows of a
// CTA do not wait for one another, was measured and is behind on balance: 1536 / 1600 columns 84 / 82 % of the
// copy rate against 80 / 79 %, but 1280 / 2560 / 3072 / 5120 columns 74 / 73 / 83 / 77 % against 77 / 78 / 86 / 87 %.)
__device__ __forceinline__ float warps_sum(float v, float* scratch, int wpr) {
  v = warp_sum(v);
  if (wpr > 1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int first = (warp / wpr) * wpr;
    v = warp_sum(lane < wpr ? scratch[first + lane] : 0.0f);
  }
  return v;
}

template <int ITEMS, bool EXACT, int MODE>
__device__ __forceinline__ void ln_fwd_warps_body(const float* __restrict__ x, const float* __restrict__ w,
                    const float* __restrict__ b, uint64_t rows, uint32_t cols, float eps,
                    float* __restrict__ y, float* __restrict__ h, float* __restrict__ stds,
                    float* __restrict__ mean, float* __restrict__ rstd, const float* __restrict__ res,
                    float* __restrict__ sum_out, int wpr) {
  constexpr bool RMS = MODE == 1;
  __shared__ float red_a[16], red_b[16];
  const int G = 32 * wpr, R = blockDim.x / G;  // threads per row, rows per CTA per iteration
  const uint32_t cols4 = cols / 4;
  const int grp = threadIdx.x / G, lane = threadIdx.x % G;
  const uint64_t nblk = (rows + R - 1) / R;
  const float inv_d = 1.0f / (float)cols;
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t row = blk * R + grp;
    const bool live = row < rows;
    const float* xr = x + row * cols;
    float4 v[ITEMS];
    float x0 = (live && !RMS) ? __ldg(xr) : 0.0f;
    if constexpr (MODE == 2) {
      if (live) x0 += __ldg(res + row * cols);
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      v[k] = (live && (EXACT || c < cols4)) ? ld_stream4(xr + c * 4) : make_float4(x0, x0, x0, x0);
    }
    if constexpr (MODE == 2) {
      float4 r[ITEMS];
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        r[k] = (live && (EXACT || c < cols4)) ? ld_stream4(res + row * cols + c * 4) : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (live && (EXACT || c < cols4)) {
          v[k].x += r[k].x; v[k].y += r[k].y; v[k].z += r[k].z; v[k].w += r[k].w;
          if (sum_out) st_stream4(sum_out + row * cols + c * 4, v[k]);
        }
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      v[k].x -= x0; v[k].y -= x0; v[k].z -= x0; v[k].w -= x0;
      s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float md = RMS ? 0.0f : warps_sum(s, red_a, wpr) * inv_d;
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      v[k].x -= md; v[k].y -= md; v[k].z -= md; v[k].w -= md;
      if (EXACT || c < cols4) q += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
    const float var = warps_sum(q, red_b, wpr) * inv_d;
    const float sd = sqrtf(var + eps);
    const float rs = 1.0f / sd;
    if (live) {
      if (lane == 0) {
        if (stds) stds[row] = sd;
        if (mean) mean[row] = x0 + md;
        if (rstd) rstd[row] = rs;
      }
      float* yr = y + row * cols;
      float* hr = h ? h + row * cols : nullptr;
      const float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f), zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (EXACT || c < cols4) {
          const float4 hv = make_float4(v[k].x * rs, v[k].y * rs, v[k].z * rs, v[k].w * rs);
          if (hr) st_stream4(hr + c * 4, hv);
          const float4 wv = w ? __ldg(reinterpret_cast<const float4*>(w) + c) : one;
          const float4 bv = b ? __ldg(reinterpret_cast<const float4*>(b) + c) : zero;
          st_stream4(yr + c * 4, make_float4(fmaf(hv.x, wv.x, bv.x), fmaf(hv.y, wv.y, bv.y),
                                             fmaf(hv.z, wv.z, bv.z), fmaf(hv.w, wv.w, bv.w)));
        }
      }
    }
  }
}

// 6 .. 8 float4 per thread run in 64 registers (two 512-thread CTAs' worth per SM); 4 and 5 fit 48 registers,
// which leaves room for a third more warps (640 / 1280 / 2560 columns 86 / 77 / 78 % of the copy rate against
// 82 / 76 / 78 % in 64 registers).
#define FB_LN_WARPS_ARGS                                                                                      \
  const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b, uint64_t rows,       \
      uint32_t cols, float eps, float *__restrict__ y, float *__restrict__ h, float *__restrict__ stds,       \
      float *__restrict__ mean, float *__restrict__ rstd, const float *__restrict__ res,                      \
      float *__restrict__ sum_out, int wpr
template <int ITEMS, bool EXACT, int MODE>
__global__ void __launch_bounds__(512, 2) ln_fwd_warps_kernel(FB_LN_WARPS_ARGS) {
  ln_fwd_warps_body<ITEMS, EXACT, MODE>(x, w, b, rows, cols, eps, y, h, stds, mean, rstd, res, sum_out, wpr);
}
template <int ITEMS, bool EXACT, int MODE>
__global__ void __maxnreg__(48) ln_fwd_warps48_kernel(FB_LN_WARPS_ARGS) {
  ln_fwd_warps_body<ITEMS, EXACT, MODE>(x, w, b, rows, cols, eps, y, h, stds, mean, rstd, res, sum_out, wpr);
}
#undef FB_LN_WARPS_ARGS

// (The same idea one level up - a CTA holding two or four rows of 1025 .. 8192 columns at a time, one
// barrier pair per group of rows - was measured and changes nothing: 85 / 92-94 / 84-85 % of the copy
// rate at 2048 / 4096 / 8192 columns with it, 85 / 94 / 85 % without.)
//
// Rows of at most 512 columns: several rows per warp at a time.  One 1 KB row per warp leaves the
// kernel bound by the latency of its own chain (load, two shuffle trees, square root, divide) with
// 1 KB per warp in flight: 71 % of the copy rate at 256 columns.  Here LPR lanes (4, 8, 16 or 32) hold
// one row, ITEMS float4 each, so a warp holds 32 / LPR rows side by side and takes RW such groups per
// step: it loads all of them before it touches any and runs their reductions interleaved; the shift
// is the first element of the row (a shuffle from the row's first lane, not a load), the affine
// vectors are loaded once per CTA, the row sums are taken transposed (lanes_transpose_sum) and the
// lane that ends with a row's sums computes and stores its statistics.  One CTA of 8 warps per block of 8 * RW * 32 / LPR rows on a full grid.  With 32 lanes
// per row and 4 rows per warp for every width (1 GB in, share of the copy rate) 32 / 64 / 96 / 128 /
// 192 columns ran at 22 / 42 / 58 / 78 / 79 %.
template <int LPR, int ITEMS, int RW, bool EXACT, bool RMS>
__global__ void __launch_bounds__(256, (ITEMS <= 2 && RW <= 4) ? 3 : 2)
ln_fwd_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                   uint64_t rows, uint32_t cols, float eps, float* __restrict__ y, float* __restrict__ h,
                   float* __restrict__ stds, float* __restrict__ mean, float* __restrict__ rstd) {
  constexpr int SUB = 32 / LPR, RPW = SUB * RW;
  const uint32_t cols4 = cols / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t nblk = (rows + 8 * RPW - 1) / (8 * RPW);
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t r0 = (blk * 8 + warp) * RPW;
    float4 v[RW][ITEMS];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        v[j][k] = (row < rows && (EXACT || c < cols4)) ? ld_stream4(x + row * cols + c * 4)
                                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    float4 wv[ITEMS], bv[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = l + k * LPR;
      const bool in = EXACT || c < cols4;
      wv[k] = (w && in) ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
      bv[k] = (b && in) ? __ldg(reinterpret_cast<const float4*>(b) + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float x0[RW], s[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      x0[j] = RMS ? 0.0f : __shfl_sync(0xffffffffu, v[j][0].x, sub * LPR);
      s[j] = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (EXACT || c < cols4) {
          v[j][k].x -= x0[j]; v[j][k].y -= x0[j]; v[j][k].z -= x0[j]; v[j][k].w -= x0[j];
          s[j] += (v[j][k].x + v[j][k].y) + (v[j][k].z + v[j][k].w);
        }
      }
    }
    // The statistics are computed transposed: lane l of a row's lanes takes group l / SPAN, so the square
    // root and the division run once per step instead of once per group; the groups' mean and reciprocal
    // come back by shuffle.
    constexpr int SPAN = LPR / RW;
    const int mine = l / SPAN, first = sub * LPR;
    float my_md = 0.0f, my_x0 = 0.0f;
    if constexpr (!RMS) {
#pragma unroll
      for (int j = 0; j < RW; ++j) my_x0 = mine == j ? x0[j] : my_x0;
      my_md = lanes_transpose_sum<LPR, RW>(s, l) * inv_d;
    }
    float md[RW], q[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      md[j] = RMS ? 0.0f : __shfl_sync(0xffffffffu, my_md, first + j * SPAN);
      q[j] = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (EXACT || c < cols4) {
          v[j][k].x -= md[j]; v[j][k].y -= md[j]; v[j][k].z -= md[j]; v[j][k].w -= md[j];
          q[j] += (v[j][k].x * v[j][k].x + v[j][k].y * v[j][k].y) + (v[j][k].z * v[j][k].z + v[j][k].w * v[j][k].w);
        }
      }
    }
    const float my_sd = sqrtf(lanes_transpose_sum<LPR, RW>(q, l) * inv_d + eps);
    const float my_rs = 1.0f / my_sd;
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
      const float rs = __shfl_sync(0xffffffffu, my_rs, first + j * SPAN);
      if (row < rows) {
        float* yr = y + row * cols;
        float* hr = h ? h + row * cols : nullptr;
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = l + k * LPR;
          if (EXACT || c < cols4) {
            const float4 hv = make_float4(v[j][k].x * rs, v[j][k].y * rs, v[j][k].z * rs, v[j][k].w * rs);
            if (hr) st_stream4(hr + c * 4, hv);
            st_stream4(yr + c * 4, make_float4(fmaf(hv.x, wv[k].x, bv[k].x), fmaf(hv.y, wv[k].y, bv[k].y),
                                               fmaf(hv.z, wv[k].z, bv[k].z), fmaf(hv.w, wv[k].w, bv[k].w)));
          }
        }
      }
    }
    if (l % SPAN == 0 && r0 + mine * SUB + sub < rows) {
      const uint64_t row = r0 + mine * SUB + sub;
      if (stds) stds[row] = my_sd;
      if (mean) mean[row] = my_x0 + my_md;
      if (rstd) rstd[row] = my_rs;
    }
  }
}

// Rows the register form does not take (longer than 32768, a width that is
// not a multiple of 4, unaligned buffers): one CTA per row on a full grid and
// three sweeps, mean, centred sum of squares, output.  The first sweep pulls
// the row from HBM with loads that leave it in L2, the other two re-read it
// from there, so DRAM sees the row once.  VEC = 4 needs 16-byte aligned rows.
template <int VEC>
__device__ __forceinline__ void ln_load(const float* p, float (&v)[VEC], bool last_use) {
  if constexpr (VEC == 4) {
    const float4 t = last_use ? __ldcs(reinterpret_cast<const float4*>(p)) : __ldcg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = last_use ? __ldcs(p) : __ldcg(p);
  }
}
template <int VEC>
__device__ __forceinline__ void ln_store(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) st_stream4(p, make_float4(v[0], v[1], v[2], v[3]));
  else st_stream(p, v[0]);
}

constexpr int kLnStreamThreads = 512;

template <int VEC>
__global__ void __launch_bounds__(kLnStreamThreads)
ln_fwd_stream_kernel(const float* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ b, uint64_t rows, uint64_t cols, float eps,
                     float* __restrict__ y, float* __restrict__ h, float* __restrict__ stds,
                     float* __restrict__ mean, float* __restrict__ rstd, int rms) {
  __shared__ float red[32];
  constexpr int T = kLnStreamThreads;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t nv = cols / VEC;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    const float x0 = rms ? 0.0f : __ldg(xr);
    float s[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) s[j] = 0.0f;
    uint64_t c = threadIdx.x;
    for (; c + T < nv; c += 2 * T) {  // two loads in flight
      float u[VEC], v[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
      ln_load<VEC>(xr + (c + T) * VEC, v, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) s[j] += (u[j] - x0) + (v[j] - x0);
    }
    for (; c < nv; c += T) {
      float u[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) s[j] += u[j] - x0;
    }
    float st = s[0];
#pragma unroll
    for (int j = 1; j < VEC; ++j) st += s[j];
    const float row_sum = block_sum(st, red);
    const float md = rms ? 0.0f : row_sum * inv_d;  // RMS: no mean
    float q[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) q[j] = 0.0f;
    for (c = threadIdx.x; c + T < nv; c += 2 * T) {
      float u[VEC], v[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
      ln_load<VEC>(xr + (c + T) * VEC, v, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float du = (u[j] - x0) - md, dv = (v[j] - x0) - md;
        q[j] += du * du + dv * dv;
      }
    }
    for (; c < nv; c += T) {
      float u[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float du = (u[j] - x0) - md;
        q[j] += du * du;
      }
    }
    float qt = q[0];
#pragma unroll
    for (int j = 1; j < VEC; ++j) qt += q[j];
    const float var = block_sum(qt, red) * inv_d;
    const float sd = sqrtf(var + eps);
    const float rs = 1.0f / sd;
    if (threadIdx.x == 0) {
      if (stds) stds[row] = sd;
      if (mean) mean[row] = x0 + md;
      if (rstd) rstd[row] = rs;
    }
    for (c = threadIdx.x; c < nv; c += T) {
      float u[VEC], wv[VEC], bv[VEC], o[VEC];
      ln_load<VEC>(xr + c * VEC, u, true);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        wv[j] = w ? __ldg(w + c * VEC + j) : 1.0f;
        bv[j] = b ? __ldg(b + c * VEC + j) : 0.0f;
        u[j] = ((u[j] - x0) - md) * rs;
        o[j] = fmaf(u[j], wv[j], bv[j]);
      }
      if (h) ln_store<VEC>(h + row * cols + c * VEC, u);
      ln_store<VEC>(y + row * cols + c * VEC, o);
    }
  }
}

// Two sweeps instead of three (rows of 8192 columns and more that no register form takes; for rows
// that have one, this kernel was measured behind it: 71 / 58 / 52 % of the copy rate at 32768 / 65536 /
// 131072 columns; spread over a cluster of 2 CTAs per row, the way the two-sweep softmax forward is,
// 64 / 73 / 66 % - it needs 51 registers, so two 512-thread CTAs per SM where the softmax has four).  Every thread folds its elements into (count, mean, M2) in one pass:
// values are taken relative to the row's first element (the common reference that keeps huge
// offsets exact) and, inside the thread, relative to the thread's own first value (its pivot), so
// that the thread's sum of squares does not cancel: the error of M2_t = q - s^2 / n is bounded by
// eps * n_t * (largest deviation)^2, which the row's M2 exceeds.  Threads, then warps, are merged
// like the partitions of a parallel variance: d = mB - mA, m = mA + d nB / n,
// M2 = M2A + M2B + d^2 nA nB / n.  The first sweep's loads leave the row in L2, the second sweep
// re-reads it from there and writes the outputs.
struct LnPart {
  float n, m, m2;
};
__device__ __forceinline__ LnPart ln_merge(LnPart a, LnPart b) {
  const float n = a.n + b.n;
  if (n == 0.0f) return a;
  const float d = b.m - a.m, fb_ = b.n / n;
  return LnPart{n, a.m + d * fb_, a.m2 + b.m2 + d * d * a.n * fb_};
}
__device__ __forceinline__ LnPart ln_shfl_xor(LnPart p, int o) {
  return LnPart{__shfl_xor_sync(0xffffffffu, p.n, o), __shfl_xor_sync(0xffffffffu, p.m, o),
                __shfl_xor_sync(0xffffffffu, p.m2, o)};
}

template <int VEC>
__global__ void __launch_bounds__(kLnStreamThreads)
ln_fwd_stream2_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                      uint64_t rows, uint64_t cols, float eps, float* __restrict__ y, float* __restrict__ h,
                      float* __restrict__ stds, float* __restrict__ mean, float* __restrict__ rstd, int rms,
                      int wb_vec) {
  constexpr int T = kLnStreamThreads;
  __shared__ LnPart red[T / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t nv = cols / VEC;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    const float x0 = rms ? 0.0f : __ldg(xr);
    uint64_t c = threadIdx.x;
    float pivot = 0.0f;
    if (!rms && c < nv) pivot = __ldcg(xr + c * VEC) - x0;
    float s[VEC], q[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) s[j] = q[j] = 0.0f;
    uint32_t cnt = 0;
    for (; c + 3 * T < nv; c += 4 * T, cnt += 4) {  // four loads in flight
      float u[VEC], v[VEC], u2[VEC], v2[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
      ln_load<VEC>(xr + (c + T) * VEC, v, false);
      ln_load<VEC>(xr + (c + 2 * T) * VEC, u2, false);
      ln_load<VEC>(xr + (c + 3 * T) * VEC, v2, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float du = (u[j] - x0) - pivot, dv = (v[j] - x0) - pivot;
        const float du2 = (u2[j] - x0) - pivot, dv2 = (v2[j] - x0) - pivot;
        s[j] += (du + dv) + (du2 + dv2);
        q[j] += (du * du + dv * dv) + (du2 * du2 + dv2 * dv2);
      }
    }
    for (; c < nv; c += T, ++cnt) {
      float u[VEC];
      ln_load<VEC>(xr + c * VEC, u, false);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float du = (u[j] - x0) - pivot;
        s[j] += du;
        q[j] += du * du;
      }
    }
    float st = s[0], qt = q[0];
#pragma unroll
    for (int j = 1; j < VEC; ++j) { st += s[j]; qt += q[j]; }
    LnPart p;
    p.n = (float)(cnt * VEC);
    if (rms) {  // no mean: M2 is the plain sum of squares, every partial mean 0
      p.m = 0.0f;
      p.m2 = qt;
    } else {
      const float ms = p.n > 0.0f ? st / p.n : 0.0f;
      p.m = pivot + ms;             // this thread's mean, relative to x0
      p.m2 = qt - st * ms;          // sum of squares about it
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) p = ln_merge(p, ln_shfl_xor(p, o));
    __syncthreads();  // red is read by the previous row's merge until here
    if (lane == 0) red[warp] = p;
    __syncthreads();
    LnPart t = lane < T / 32 ? red[lane] : LnPart{0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = ln_merge(t, ln_shfl_xor(t, o));
    const float md = rms ? 0.0f : t.m;
    const float var = t.m2 * inv_d;
    const float sd = sqrtf(var + eps);
    const float rs = 1.0f / sd;
    if (threadIdx.x == 0) {
      if (stds) stds[row] = sd;
      if (mean) mean[row] = x0 + md;
      if (rstd) rstd[row] = rs;
    }
    // wb_vec: weight and bias (when present) are 16-byte aligned, so their float4 loads are legal.
    auto emit = [&](uint64_t cc, const float (&xin)[VEC]) {
      float u[VEC], wv[VEC], bv[VEC], o[VEC];
      if (VEC == 4 && wb_vec) {
        const float4 w4 = w ? __ldg(reinterpret_cast<const float4*>(w) + cc) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        const float4 b4 = b ? __ldg(reinterpret_cast<const float4*>(b) + cc) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        wv[0] = w4.x; bv[0] = b4.x;
        if constexpr (VEC == 4) { wv[1] = w4.y; wv[2] = w4.z; wv[3] = w4.w; bv[1] = b4.y; bv[2] = b4.z; bv[3] = b4.w; }
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          wv[j] = w ? __ldg(w + cc * VEC + j) : 1.0f;
          bv[j] = b ? __ldg(b + cc * VEC + j) : 0.0f;
        }
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        u[j] = ((xin[j] - x0) - md) * rs;
        o[j] = fmaf(u[j], wv[j], bv[j]);
      }
      if (h) ln_store<VEC>(h + row * cols + cc * VEC, u);
      ln_store<VEC>(y + row * cols + cc * VEC, o);
    };
    c = threadIdx.x;
    for (; c + 3 * T < nv; c += 4 * T) {  // four loads in flight
      float u0[VEC], u1[VEC], u2[VEC], u3[VEC];
      ln_load<VEC>(xr + c * VEC, u0, true);
      ln_load<VEC>(xr + (c + T) * VEC, u1, true);
      ln_load<VEC>(xr + (c + 2 * T) * VEC, u2, true);
      ln_load<VEC>(xr + (c + 3 * T) * VEC, u3, true);
      emit(c, u0); emit(c + T, u1); emit(c + 2 * T, u2); emit(c + 3 * T, u3);
    }
    for (; c < nv; c += T) {
      float u0[VEC];
      ln_load<VEC>(xr + c * VEC, u0, true);
      emit(c, u0);
    }
  }
}

// ----------------------------------------------------------------- backward
// Partial dweight / dbias layout in scratch: [parts][2][cols], part p written
// by exactly one (CTA, row group); the finalize kernel adds the parts in
// index order, so the result does not depend on scheduling.
// MODE 0: saved (h, stds); 1: saved (x, mean, rstd); 2: RMS normalisation, saved (x, rstd), no mean.
template <int G, int ITEMS, int MODE, bool EXACT>
__global__ void __launch_bounds__(G)
ln_bwd_reg_kernel(const float* __restrict__ g, const float* __restrict__ hx,
                  const float* __restrict__ stat_a,  // stds (FROM_X: mean)
                  const float* __restrict__ stat_b,  // unused (FROM_X: rstd)
                  const float* __restrict__ w, uint64_t rows, uint32_t cols,
                  float* __restrict__ dx, float* __restrict__ part, int want_dw, int want_db) {
  constexpr bool FROM_X = MODE != 0, RMS = MODE == 2;
  __shared__ float red_a[G / 32], red_b[G / 32];
  const uint32_t cols4 = cols / 4;
  const int lane = threadIdx.x;
  const float inv_d = 1.0f / (float)cols;
  // The weights stay in registers across rows except in the 1024-thread form,
  // which has 64 registers per thread and none to spare.
  constexpr bool kHoistW = G < 1024;
  auto load_w = [&](int k) {
    const uint32_t c = lane + k * G;
    return (w && (EXACT || c < cols4)) ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(1, 1, 1, 1);
  };
  float4 aw[ITEMS], ab[ITEMS], wreg[kHoistW ? ITEMS : 1];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    aw[k] = ab[k] = make_float4(0, 0, 0, 0);
    if constexpr (kHoistW) wreg[k] = load_w(k);
  }
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    float4 gv[ITEMS], hv[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (EXACT || c < cols4) {
        gv[k] = ld_stream4(g + row * cols + c * 4);
        hv[k] = ld_stream4(hx + row * cols + c * 4);
      } else {
        gv[k] = hv[k] = make_float4(0, 0, 0, 0);
      }
    }
    float rs;
    if constexpr (FROM_X) {
      const float mu = RMS ? 0.0f : __ldg(stat_a + row);
      rs = __ldg(stat_b + row);
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = lane + k * G;
        if (EXACT || c < cols4) {
          hv[k].x = (hv[k].x - mu) * rs; hv[k].y = (hv[k].y - mu) * rs;
          hv[k].z = (hv[k].z - mu) * rs; hv[k].w = (hv[k].w - mu) * rs;
        }
      }
    } else {
      rs = 1.0f / __ldg(stat_a + row);
    }
    float s1 = 0.0f, s2 = 0.0f;
    float4 dh[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      float4 wv;
      if constexpr (kHoistW) wv = wreg[k]; else wv = load_w(k);
      dh[k] = make_float4(gv[k].x * wv.x, gv[k].y * wv.y, gv[k].z * wv.z, gv[k].w * wv.w);
      s1 += (dh[k].x + dh[k].y) + (dh[k].z + dh[k].w);
      s2 += (dh[k].x * hv[k].x + dh[k].y * hv[k].y) + (dh[k].z * hv[k].z + dh[k].w * hv[k].w);
      aw[k].x += gv[k].x * hv[k].x; aw[k].y += gv[k].y * hv[k].y;
      aw[k].z += gv[k].z * hv[k].z; aw[k].w += gv[k].w * hv[k].w;
      ab[k].x += gv[k].x; ab[k].y += gv[k].y; ab[k].z += gv[k].z; ab[k].w += gv[k].w;
    }
    const float m1 = RMS ? 0.0f : group_sum<G>(s1, red_a) * inv_d;
    const float m2 = group_sum<G>(s2, red_b) * inv_d;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (EXACT || c < cols4) {
        float4 o;
        o.x = (dh[k].x - m1 - hv[k].x * m2) * rs;
        o.y = (dh[k].y - m1 - hv[k].y * m2) * rs;
        o.z = (dh[k].z - m1 - hv[k].z * m2) * rs;
        o.w = (dh[k].w - m1 - hv[k].w * m2) * rs;
        st_stream4(dx + row * cols + c * 4, o);
      }
    }
  }
  if (want_dw | want_db) {
    float* pw = part + (uint64_t)blockIdx.x * 2 * cols;
    float* pb = pw + cols;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t c = lane + k * G;
      if (EXACT || c < cols4) {
        if (want_dw) *reinterpret_cast<float4*>(pw + c * 4) = aw[k];
        if (want_db) *reinterpret_cast<float4*>(pb + c * 4) = ab[k];
      }
    }
  }
}

// Backward for rows the register and pipelined forms do not take.  Two
// kernels, because neither the row nor its two column accumulators fit a CTA:
//   1. per row, m1 = mean(g*w) and m2 = mean(g*w*h), one CTA per row;
//   2. a column-tiled sweep (reduce.cuh) whose source computes dx from the
//      row's (m1, m2, 1/std), stores it, and hands g*h and g to the column
//      sums that become dweight and dbias.
// g and h are read twice, so this path moves 5 arrays where the fused forms
// move 3; it exists so that no shape falls off a cliff.
template <int VEC, bool FROM_X>
__global__ void __launch_bounds__(kLnStreamThreads)
ln_bwd_rowstats_kernel(const float* __restrict__ g, const float* __restrict__ hx,
                       const float* __restrict__ stat_a, const float* __restrict__ stat_b,
                       const float* __restrict__ w, uint64_t rows, uint64_t cols,
                       float* __restrict__ m12 /*[rows][2]*/) {
  __shared__ float red[32];
  constexpr int T = kLnStreamThreads;
  const float inv_d = 1.0f / (float)cols;
  const uint64_t nv = cols / VEC;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* gr = g + row * cols;
    const float* hr = hx + row * cols;
    float mu = 0.0f, rs = 1.0f;
    if constexpr (FROM_X) {
      mu = stat_a ? __ldg(stat_a + row) : 0.0f;  // no mean: RMS normalisation
      rs = __ldg(stat_b + row);
    }
    float s1 = 0.0f, s2 = 0.0f;
    auto fold = [&](const float (&gv)[VEC], const float (&hv)[VEC], uint64_t c) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float hh = FROM_X ? (hv[j] - mu) * rs : hv[j];
        const float d = w ? gv[j] * __ldg(w + c * VEC + j) : gv[j];
        s1 += d;
        s2 += d * hh;
      }
    };
    uint64_t c = threadIdx.x;
    for (; c + T < nv; c += 2 * T) {  // four loads in flight
      float g0[VEC], h0[VEC], g1[VEC], h1[VEC];
      ln_load<VEC>(gr + c * VEC, g0, true);
      ln_load<VEC>(hr + c * VEC, h0, true);
      ln_load<VEC>(gr + (c + T) * VEC, g1, true);
      ln_load<VEC>(hr + (c + T) * VEC, h1, true);
      fold(g0, h0, c);
      fold(g1, h1, c + T);
    }
    for (; c < nv; c += T) {
      float g0[VEC], h0[VEC];
      ln_load<VEC>(gr + c * VEC, g0, true);
      ln_load<VEC>(hr + c * VEC, h0, true);
      fold(g0, h0, c);
    }
    const float m1 = (!FROM_X || stat_a) ? block_sum(s1, red) * inv_d : 0.0f;  // RMS: no mean term
    const float m2 = block_sum(s2, red) * inv_d;
    if (threadIdx.x == 0) {
      m12[row * 2] = m1;
      m12[row * 2 + 1] = m2;
    }
  }
}

// Source of the column sweep: element (r, c) yields g*h and g, and dx is
// stored on the way.
template <bool FROM_X>
struct LnBwdColSrc {
  const float* g;
  const float* hx;
  const float* stat_a;
  const float* stat_b;
  const float* w;
  const float* m12;
  float* dx;
  uint64_t cols;
  template <int VEC>
  __device__ __forceinline__ void load(uint64_t, uint64_t r, uint64_t c, float (&v)[2][VEC]) const {
    const uint64_t off = r * cols + c;
    float gv[VEC], hv[VEC], o[VEC];
    ln_load<VEC>(g + off, gv, true);
    ln_load<VEC>(hx + off, hv, true);
    float mu = 0.0f, rs;
    if constexpr (FROM_X) {
      mu = stat_a ? __ldg(stat_a + r) : 0.0f;
      rs = __ldg(stat_b + r);
    } else {
      rs = 1.0f / __ldg(stat_a + r);
    }
    const float m1 = __ldg(m12 + r * 2), m2 = __ldg(m12 + r * 2 + 1);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float hh = FROM_X ? (hv[j] - mu) * rs : hv[j];
      const float d = w ? gv[j] * __ldg(w + c + j) : gv[j];
      o[j] = (d - m1 - hh * m2) * rs;
      v[0][j] = gv[j] * hh;
      v[1][j] = gv[j];
    }
    ln_store<VEC>(dx + off, o);
  }
};

// Backward for rows of at most 384 columns: several rows per warp at a time, like ln_fwd_rows_kernel.
// LPR lanes (8, 16 or 32) hold one row, ITEMS float4 each, so a warp holds 32 / LPR rows side by side and
// takes RW such groups per step: it loads all of their g and h (or x) before it touches any, takes the
// two row sums of every row with interleaved shuffles and keeps its own column accumulators.  At the
// end the warps (and the row halves of a warp) of a CTA are added in a fixed order through shared
// memory, one partial row per CTA.  Persistent grid: CTA b takes the blocks of 8 * RW * 32 / LPR rows
// b, b + gridDim.x, ...  Measured against one row per warp (1.6 GB, share of the copy rate): 64 columns
// 96 % from 44, 128 columns 95 % from 82, 192 columns 93 % from 84, 256 columns 96 % from 90.
template <int LPR, int ITEMS, int RW, int MODE>
__global__ void __launch_bounds__(256, 2)
ln_bwd_rows_kernel(const float* __restrict__ g, const float* __restrict__ hx, const float* __restrict__ stat_a,
                   const float* __restrict__ stat_b, const float* __restrict__ w, uint64_t rows, uint32_t cols,
                   float* __restrict__ dx, float* __restrict__ part, int want_dw, int want_db) {
  constexpr bool FROM_X = MODE != 0, RMS = MODE == 2;
  constexpr int SUB = 32 / LPR, RPW = SUB * RW, NACC = 8 * SUB, W4 = ITEMS * LPR;
  __shared__ float4 fold[2][NACC][W4];
  const uint32_t cols4 = cols / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const float inv_d = 1.0f / (float)cols;
  // The weights stay in registers across rows except with four float4 per lane, where there is no room:
  // that form fetches them (from L1) once per step.
  constexpr bool kHoistW = ITEMS < 4;
  auto load_w = [&](int k) {
    const uint32_t c = l + k * LPR;
    return (w && c < cols4) ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(1, 1, 1, 1);
  };
  float4 aw[ITEMS], ab[ITEMS], wv[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    aw[k] = ab[k] = make_float4(0, 0, 0, 0);
    if constexpr (kHoistW) wv[k] = load_w(k);
  }
  const uint64_t nblk = (rows + 8 * RPW - 1) / (8 * RPW);
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t r0 = (blk * 8 + warp) * RPW;
    float4 gv[RW][ITEMS], hv[RW][ITEMS];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (row < rows && c < cols4) {
          gv[j][k] = ld_stream4(g + row * cols + c * 4);
          hv[j][k] = ld_stream4(hx + row * cols + c * 4);
        } else {
          gv[j][k] = hv[j][k] = make_float4(0, 0, 0, 0);
        }
      }
    }
    if constexpr (!kHoistW) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) wv[k] = load_w(k);
    }
    // Lane t < RPW fetches the statistics of row r0 + t; the lanes of that row get them by shuffle.
    float my_a = 1.0f, my_b = 1.0f;
    if (lane < RPW && r0 + lane < rows) {
      my_a = __ldg(stat_a + r0 + lane);
      if constexpr (FROM_X) my_b = __ldg(stat_b + r0 + lane);
    }
    float rs[RW], s1[RW], s2[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const bool live = r0 + j * SUB + sub < rows;
      const float sa = __shfl_sync(0xffffffffu, my_a, j * SUB + sub), sb = __shfl_sync(0xffffffffu, my_b, j * SUB + sub);
      float mu = 0.0f;
      if constexpr (FROM_X) {
        mu = RMS ? 0.0f : sa;
        rs[j] = sb;
      } else {
        rs[j] = 1.0f / sa;
      }
      s1[j] = s2[j] = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (live && c < cols4) {
          if constexpr (FROM_X) {
            hv[j][k].x = (hv[j][k].x - mu) * rs[j]; hv[j][k].y = (hv[j][k].y - mu) * rs[j];
            hv[j][k].z = (hv[j][k].z - mu) * rs[j]; hv[j][k].w = (hv[j][k].w - mu) * rs[j];
          }
          aw[k].x += gv[j][k].x * hv[j][k].x; aw[k].y += gv[j][k].y * hv[j][k].y;
          aw[k].z += gv[j][k].z * hv[j][k].z; aw[k].w += gv[j][k].w * hv[j][k].w;
          ab[k].x += gv[j][k].x; ab[k].y += gv[j][k].y; ab[k].z += gv[j][k].z; ab[k].w += gv[j][k].w;
          // from here on gv holds g * w
          gv[j][k].x *= wv[k].x; gv[j][k].y *= wv[k].y; gv[j][k].z *= wv[k].z; gv[j][k].w *= wv[k].w;
          s1[j] += (gv[j][k].x + gv[j][k].y) + (gv[j][k].z + gv[j][k].w);
          s2[j] += (gv[j][k].x * hv[j][k].x + gv[j][k].y * hv[j][k].y) + (gv[j][k].z * hv[j][k].z + gv[j][k].w * hv[j][k].w);
        }
      }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
#pragma unroll
      for (int j = 0; j < RW; ++j) {
        s1[j] += __shfl_xor_sync(0xffffffffu, s1[j], o);
        s2[j] += __shfl_xor_sync(0xffffffffu, s2[j], o);
      }
    }
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
      if (row >= rows) continue;
      const float m1 = RMS ? 0.0f : s1[j] * inv_d, m2 = s2[j] * inv_d;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (c < cols4)
          st_stream4(dx + row * cols + c * 4,
                     make_float4((gv[j][k].x - m1 - hv[j][k].x * m2) * rs[j], (gv[j][k].y - m1 - hv[j][k].y * m2) * rs[j],
                                 (gv[j][k].z - m1 - hv[j][k].z * m2) * rs[j], (gv[j][k].w - m1 - hv[j][k].w * m2) * rs[j]));
      }
    }
  }
  if (want_dw | want_db) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      fold[0][warp * SUB + sub][k * LPR + l] = aw[k];
      fold[1][warp * SUB + sub][k * LPR + l] = ab[k];
    }
    __syncthreads();
    float* pw = part + (uint64_t)blockIdx.x * 2 * cols;
    for (uint32_t i = threadIdx.x; i < 2u * W4; i += 256) {
      const uint32_t which = i / W4, c = i % W4;
      if (c < cols4 && (which ? want_db : want_dw)) {
        float4 t = fold[which][0][c];
#pragma unroll
        for (int q = 1; q < NACC; ++q) {
          const float4 u = fold[which][q][c];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        *reinterpret_cast<float4*>(pw + (uint64_t)which * cols + c * 4) = t;
      }
    }
  }
}

// dweight[c] = sum_p part[p][0][c], dbias[c] = sum_p part[p][1][c].
// A CTA owns 8 columns (one 32-byte sector per partial row) and spreads the
// parts over 128 row lanes, each with up to 4 independent loads per output in
// flight, so the scratch (still in L2) is pulled in about one memory latency;
// the lanes are then added in lane order.  The order depends on `parts` only.
__global__ void __launch_bounds__(1024)
ln_bwd_finalize_kernel(const float* __restrict__ part, uint32_t parts, uint64_t cols,
                       float* __restrict__ dw, float* __restrict__ db) {
  __shared__ float lane_sum[2][128][9];
  pdl_wait();  // a dependent launch: resident while the backward drains, released when its partial rows are complete
  pdl_trigger();
  const int cx = threadIdx.x & 7, rl = threadIdx.x >> 3;
  const uint64_t c = (uint64_t)blockIdx.x * 8 + cx;
  float a = 0.0f, b = 0.0f;
  if (c < cols) {
    for (uint32_t p = rl; p < parts; p += 4 * 128) {
      float va[4], vb[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t pq = p + q * 128;
        const float* pp = part + (uint64_t)pq * 2 * cols;
        va[q] = (dw && pq < parts) ? pp[c] : 0.0f;
        vb[q] = (db && pq < parts) ? pp[cols + c] : 0.0f;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        a += va[q];
        b += vb[q];
      }
    }
  }
  lane_sum[0][rl][cx] = a;
  lane_sum[1][rl][cx] = b;
  __syncthreads();
  // Warp w < 16 finishes output (w / 8) of column (w % 8).
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (w < 16) {
    const int o = w >> 3, col = w & 7;
    float r = (lane_sum[o][l][col] + lane_sum[o][l + 32][col]) + (lane_sum[o][l + 64][col] + lane_sum[o][l + 96][col]);
    r = warp_sum(r);
    const uint64_t oc = (uint64_t)blockIdx.x * 8 + col;
    if (l == 0 && oc < cols) {
      if (o == 0 && dw) dw[oc] = r;
      if (o == 1 && db) db[oc] = r;
    }
  }
}

}  // namespace fb
#include "layer_norm_pipe.cuh"
#include "layer_norm_cluster.cuh"
namespace fb {

// Raises the dynamic shared memory limit of a kernel: a host-side attribute of
// the function on the current device, set once per (kernel, device) and
// remembered (allow_dyn_smem, common.cuh), not at every launch.
template <class K>
static cudaError_t allow_smem(K kernel, size_t bytes) {
  return allow_dyn_smem(reinterpret_cast<const void*>(kernel), bytes);
}

// FB_LN_CLUSTER in the environment: 0 keeps wide rows on the single-CTA kernels, 2 / 4 / 8 fixes
// the cluster size (for A/B measurements); anything else, or nothing, lets cluster_plan choose.
static int ln_cluster_choice() {
  static const int v = [] {
    const char* e = getenv("FB_LN_CLUSTER");
    if (!e || !*e) return -1;
    const int n = atoi(e);
    return (n == 0 || n == 2 || n == 4 || n == 8) ? n : -1;
  }();
  return v;
}
// FB_LN_ROWS=0 keeps rows of at most 512 columns on the one-row-per-warp kernel (for A/B measurements).
static bool ln_rows_enabled() {
  static const int on = [] {
    const char* e = getenv("FB_LN_ROWS");
    return (e && e[0] == '0') ? 0 : 1;
  }();
  return on != 0;
}
// FB_LN_FWD_SWEEPS=3: the three-sweep forward for rows no register form takes (A/B measurements).
static bool ln_fwd_three_sweeps() {
  static const int v = [] { const char* e = getenv("FB_LN_FWD_SWEEPS"); return (e && e[0] == '3') ? 1 : 0; }();
  return v != 0;
}
// Forward over a cluster with the slices in registers (ln_fwd_cluster_reg_kernel): rows wider than
// 32768 columns, slices of at most 16384.  Returns the cluster size, 0 if the shape does not take it.
static int ln_fwd_cluster_reg_plan(uint64_t cols, uint64_t* slice4) {
  const int choice = ln_cluster_choice();
  if (choice == 0 || (cols & 3) || cols <= 32768 || cols > 16384ull * kClusterMax) return 0;
  const uint64_t v4 = cols / 4;
  // Slices of at most 8192 columns (256 threads x 8 float4, four CTAs per SM) while 8 CTAs cover the row: 70.5 % of
  // the copy rate at 65536 columns and 64 % at 50000, against 67 % and 61.5 % for slices of 16384 on 512 threads.
  const uint64_t cap4 = v4 <= 8 * 2048 ? 2048 : 4096;
  const int cl = choice > 0 ? choice : (v4 <= 2 * cap4 ? 2 : (v4 <= 4 * cap4 ? 4 : 8));
  const uint64_t s4 = (v4 + cl - 1) / cl;
  if (s4 > 4096 || s4 * (uint64_t)(cl - 1) >= v4) return 0;
  *slice4 = s4;
  return cl;
}
// FB_LN_BWD_ROWS=0 keeps rows of at most 256 columns on the one-row-per-warp backward (A/B measurements).
static bool ln_bwd_rows_on() {
  static const int on = [] { const char* e = getenv("FB_LN_BWD_ROWS"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}
// Widest row of the several-rows-per-warp backward.  Up to 384 columns (32 lanes x 3 float4) it is ahead of
// the staged pipeline (320 / 384 columns 94 / 93 % of the copy rate against 79 / 86 %); with four float4 per
// lane it runs out of registers and is behind (448 / 512 columns 85 / 88 % against 96 / 89 %).
// FB_LN_BWD_ROWS_MAX=<columns, at most 512> moves the limit (A/B measurements).
static uint64_t ln_bwd_rows_max() {
  static const uint64_t v = [] { const char* e = getenv("FB_LN_BWD_ROWS_MAX"); return e ? (uint64_t)atoll(e) : 384ull; }();
  return v > 512 ? 512 : v;
}
static ClusterPlan ln_cluster_plan(uint64_t cols, int narr) {
  const int c = ln_cluster_choice();
  if (c == 0) return ClusterPlan{0, 0, 0, 0, 0, 0, 0};
  return cluster_plan(cols, narr, c < 0 ? 0 : c);
}


// Backward geometry: at most 4 float4 per thread (8 only for the widest rows)
// so the two column accumulators stay in registers.
static RowCfg ln_bwd_cfg(uint64_t cols) {
  RowCfg c{0, 0};
  if (cols == 0 || (cols & 3)) return c;
  const uint64_t v = cols / 4;
  for (int g = 32; g <= 1024; g <<= 1) {
    const int cap = (g == 1024) ? 8 : 4;
    if (v <= (uint64_t)g * cap) {
      uint64_t it = (v + g - 1) / g;
      int p = 1;
      while ((uint64_t)p < it) p <<= 1;
      c.group = g;
      c.items = p;
      return c;
    }
  }
  return c;
}

// CTAs per SM the backward launches (a fixed table, so scratch sizing and the
// launch always agree).
static int ln_bwd_ctas_per_sm(const RowCfg& c) {
  if (c.group == 0) return 4;  // generic kernel, 256 threads
  const int threads_per_sm = c.items >= 8 ? 1024 : (c.items == 4 ? 768 : 1024);
  int n = threads_per_sm / c.group;
  return n < 1 ? 1 : n;
}

static uint32_t ln_bwd_parts(uint64_t rows, uint64_t cols) {
  const RowCfg c = ln_bwd_cfg(cols);
  const uint64_t cap = (uint64_t)device_info().sm_count * ln_bwd_ctas_per_sm(c);
  return (uint32_t)(rows < cap ? rows : cap);
}

// Upper bound of the partial rows over every path the backward may take
// (register, generic, pipelined): what the scratch is sized for.
static uint32_t ln_bwd_max_parts(uint64_t rows, uint64_t cols) {
  const uint32_t a = ln_bwd_parts(rows, cols);  // register and generic kernels
  const uint32_t c = pipe_plan(rows, cols, 2).grid;
  const uint32_t d = cluster_plan_max_clusters(ln_cluster_plan(cols, 2));
  const uint32_t m = a > c ? a : c;
  return m > d ? m : d;
}

// Forward geometry: at most 4 float4 per thread (8 only for the widest rows).
// The forward carries little state besides the row, so the short form keeps
// six CTAs of 256 threads on an SM, which is what covers the load latency.
static bool ln_fwd_wide512() {
  static const int on = [] { const char* e = getenv("FB_LN_FWD_W"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}
static RowCfg ln_fwd_cfg(uint64_t cols) {
  // 8 float4 per thread (eight loads in flight, fewer threads per row, four 256-thread CTAs per SM) where it was
  // measured ahead of 2 or 4 per thread: 1025 .. 2048 columns on 64 threads (90 % of the copy rate at 2048 against
  // 85 %, 78 against 70 % at 1536), 4097 .. 8192 columns on 256 threads (97 against 85 % at 8192, 85 against 76 % at
  // 6000).  Not 2049 .. 4096: 128 threads x 8 run at 90 % where 256 x 4 reach 94-95 %.
  if ((cols & 3) == 0 && cols > 1024 && cols <= 2048) return RowCfg{64, 8};
  if ((cols & 3) == 0 && cols > 4096 && cols <= 8192) return RowCfg{256, 8};
  // 8193 .. 16384 columns: 512 threads x 8 float4, two CTAs per SM (64 registers), loads straight from global
  // memory: 90 % of the copy rate at 16384 columns and 81 % at 12288, against 71 % and 69 % for the staged
  // 1024-thread pipeline.  FB_LN_FWD_W=0 restores that form for A/B measurements.
  if (ln_fwd_wide512() && cols > 8192 && cols <= 16384 && (cols & 3) == 0) return RowCfg{512, 8};
  // Up to 1024 columns a warp holds the row (8 float4 per lane at most): both reductions are shuffles, no barrier.
  if (cols > 512 && cols <= 1024 && (cols & 3) == 0) return RowCfg{32, 8};
  return ln_bwd_cfg(cols);
}

template <int G, int ITEMS>
static void launch_ln_fwd(cudaStream_t s, unsigned grid, const float* x, const float* w,
                          const float* b, uint64_t rows, uint32_t cols, float eps, float* y,
                          float* h, float* stds, float* mean, float* rstd, int mode, const float* res,
                          float* sum_out) {
#define FB_LN_FWD_REG(EX, MD) \
  ln_fwd_reg_kernel<G, ITEMS, EX, MD><<<grid, ln_threads<G>(), 0, s>>>(x, w, b, rows, cols, eps, y, h, stds, mean, rstd, res, sum_out)
  if (cols == 4u * G * ITEMS) {
    if (mode == 2) FB_LN_FWD_REG(true, 2); else if (mode == 1) FB_LN_FWD_REG(true, 1); else FB_LN_FWD_REG(true, 0);
  } else {
    if (mode == 2) FB_LN_FWD_REG(false, 2); else if (mode == 1) FB_LN_FWD_REG(false, 1); else FB_LN_FWD_REG(false, 0);
  }
#undef FB_LN_FWD_REG
}

// Geometry of ln_fwd_warps_kernel for `cols`, or false where the power-of-two geometry already fits (at least
// 94 % of its slots used), the width is out of range (513 .. 10240 columns, a multiple of 4) or the CTA size
// that follows leaves fewer than 960 threads resident per SM at 64 registers (12288 columns on 12 warps: 72 %
// of the copy rate against 81 % for 512 x 8 with a quarter of its slots dead).  Among 8 .. 4 float4 per
// thread the one with the fewest dead slots wins, more float4 per thread on a tie.  (Choosing by the bytes of
// row data resident per SM instead, with 40 / 48 registers for 5 / 6 float4 per thread, was measured and is
// behind: it spills, and 640 / 768 / 1280 / 1536 columns ran at 83 / 79 / 68 / 74 % against 82 / 88 / 76 / 81 %.)
// FB_LN_FWD_WARPS=0 switches the form off (A/B measurements).
// FB_LN_FWD_WARPS48=0 runs 4 and 5 float4 per thread in 64 registers too (A/B measurements).
static bool ln_fwd_warps48() {
  static const int on = [] { const char* e = getenv("FB_LN_FWD_WARPS48"); return (e && e[0] == '0') ? 0 : 1; }();
  return on != 0;
}
struct WarpsCfg { int wpr, items, rows_per_cta; };
static bool ln_fwd_warps_cfg(uint64_t cols, WarpsCfg* out) {
  static const int on = [] { const char* e = getenv("FB_LN_FWD_WARPS"); return (e && e[0] == '0') ? 0 : 1; }();
  if (!on || (cols & 3) || cols <= 512 || cols > 10240) return false;
  const uint64_t c4 = cols / 4;
  const RowCfg cur = ln_fwd_cfg(cols);
  if (cur.group && c4 * 100 >= (uint64_t)cur.group * cur.items * 94) return false;
  uint64_t best = ~0ull;
  for (int items = 8; items >= 4; --items) {
    const uint64_t wpr = (c4 + 32ull * items - 1) / (32ull * items);
    if (wpr > 10) continue;  // 16 warps x 6 or 7 float4: 76 / 78 % at 12288 / 14336 columns against 81 / 84 % for 512 x 8
    const int r = wpr >= 8 ? 1 : 8 / (int)wpr;  // rows per CTA: 160 .. 320 threads
    const int t = 32 * (int)wpr * r;
    if (t * (1024 / t) < 960) continue;
    const uint64_t dead = wpr * 32 * items - c4;
    if (dead < best) { best = dead; *out = WarpsCfg{(int)wpr, items, r}; }
  }
  return best != ~0ull;
}

template <int ITEMS>
static void launch_ln_fwd_warps(cudaStream_t s, int wpr, int r, const float* x, const float* w, const float* b,
                                uint64_t rows, uint32_t cols, float eps, float* y, float* h, float* stds,
                                float* mean, float* rstd, int mode, const float* res, float* sum_out) {
  const unsigned threads = 32u * wpr * r, grid = grid_full((rows + r - 1) / r);
#define FB_LN_FWD_WARPS(EX, MD)                                                                                       \
  {                                                                                                                   \
    if (ITEMS <= 5 && ln_fwd_warps48())                                                                               \
      ln_fwd_warps48_kernel<(ITEMS <= 5 ? ITEMS : 5), EX, MD><<<grid, threads, 0, s>>>(x, w, b, rows, cols, eps, y, h, stds, mean, rstd, nullptr, nullptr, wpr); \
    else                                                                                                              \
      ln_fwd_warps_kernel<ITEMS, EX, MD><<<grid, threads, 0, s>>>(x, w, b, rows, cols, eps, y, h, stds, mean, rstd, nullptr, nullptr, wpr); \
  }
  // (The LayerNorm of x + residual stays on the power-of-two geometries: with 7 or 8 float4 per thread of two
  // arrays this kernel does not fit 64 registers.)
  (void)res; (void)sum_out;
  if (cols == 128u * wpr * ITEMS) {
    if (mode == 1) FB_LN_FWD_WARPS(true, 1) else FB_LN_FWD_WARPS(true, 0)
  } else {
    if (mode == 1) FB_LN_FWD_WARPS(false, 1) else FB_LN_FWD_WARPS(false, 0)
  }
#undef FB_LN_FWD_WARPS
}

template <int G, int ITEMS>
static void launch_ln_bwd(cudaStream_t s, unsigned grid, int mode, const float* g,
                          const float* hx, const float* sa, const float* sb, const float* w,
                          uint64_t rows, uint32_t cols, float* dx, float* part, int wdw, int wdb) {
  const bool exact = cols == 4u * G * ITEMS;
#define FB_LN_BWD_REG(MD, EX) \
  ln_bwd_reg_kernel<G, ITEMS, MD, EX><<<grid, G, 0, s>>>(g, hx, sa, sb, w, rows, cols, dx, part, wdw, wdb)
  if (mode == 2) {
    if (exact) FB_LN_BWD_REG(2, true); else FB_LN_BWD_REG(2, false);
  } else if (mode == 1) {
    if (exact) FB_LN_BWD_REG(1, true); else FB_LN_BWD_REG(1, false);
  } else {
    if (exact) FB_LN_BWD_REG(0, true); else FB_LN_BWD_REG(0, false);
  }
#undef FB_LN_BWD_REG
}

}  // namespace fb

using namespace fb;

extern "C" {

// res != NULL: normalise x + res (sum_out, optional, receives the sum).  Only the register
// kernel adds on the fly; for every other path the caller (fb_residual_layer_norm_fwd) has
// formed the sum first and passes it as x with res = NULL.
static int ln_fwd_impl(fb_stream_t stream, const float* x, const float* weight, const float* bias,
                       uint64_t rows, uint64_t cols, float eps, float* y, float* h, float* stds,
                       float* mean, float* rstd, int rms, const float* res = nullptr,
                       float* sum_out = nullptr) {
  uint64_t total;
  if (cols == 0) return fail(FB_ERR_INVALID_SHAPE, "fb_layer_norm_fwd: last dimension must be nonempty");
  if (mul_overflows(rows, cols, &total) || total > (UINT64_MAX >> 3))
    return fail(FB_ERR_INVALID_SHAPE, "fb_layer_norm_fwd: rows * cols overflows");
  if (rows == 0) return FB_OK;
  if (!x || !y) return fail(FB_ERR_INVALID_ARG, "fb_layer_norm_fwd: null buffer");
  const RowCfg c = ln_fwd_cfg(cols);
  uint64_t clreg_slice4 = 0;
  const bool fast = (c.group != 0 || ln_fwd_cluster_reg_plan(cols, &clreg_slice4) != 0) && aligned16(x) && aligned16(y) && (!h || aligned16(h)) &&
                    (!weight || aligned16(weight)) && (!bias || aligned16(bias));
  if (!fast) {
    const bool v4 = cols % 4 == 0 && aligned16(x) && aligned16(y) && (!h || aligned16(h));
    const int wb_vec = (!weight || aligned16(weight)) && (!bias || aligned16(bias));
    // Two sweeps pay from about 8192 columns (10001 columns: 3.81 against 3.52 TB/s, 33001: 4.26 against 3.49,
    // 262144: 3.32 against 2.62); on shorter rows the merge of the threads' partial variances costs more than the
    // third sweep (4097 columns: 2.44 against 3.05 TB/s).
    if (ln_fwd_three_sweeps() || cols < 8192) {
      if (v4)
        ln_fwd_stream_kernel<4><<<grid_full(rows), kLnStreamThreads, 0, stream>>>(x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, rms);
      else
        ln_fwd_stream_kernel<1><<<grid_full(rows), kLnStreamThreads, 0, stream>>>(x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, rms);
    } else {
      if (v4)
        ln_fwd_stream2_kernel<4><<<grid_full(rows), kLnStreamThreads, 0, stream>>>(x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, rms, wb_vec);
      else
        ln_fwd_stream2_kernel<1><<<grid_full(rows), kLnStreamThreads, 0, stream>>>(x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, rms, 0);
    }
    FB_LAUNCHED("fb_layer_norm_fwd");
    return FB_OK;
  }
  if (res && (!fast || cols > 8192))
    return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_fwd: the fused residual form needs the register kernel");
  const uint32_t cc = (uint32_t)cols;
  // More than 32768 columns: a cluster of CTAs per row, slices in registers (layer_norm_cluster.cuh).
  {
    uint64_t slice4 = 0;
    const int cl = res ? 0 : ln_fwd_cluster_reg_plan(cols, &slice4);
    if (cl) {
      unsigned int* faults = fault_word();
      cudaError_t le = cudaErrorInvalidValue;
      int fit = 0;
#define FB_LN_FWD_CLR(TT, I, R)                                                                                     \
  {                                                                                                             \
    auto k = ln_fwd_cluster_reg_kernel<TT, I, R>;                                                               \
    FB_CUDA(resident_clusters(reinterpret_cast<const void*>(k), TT, 0, cl, &fit));                              \
    const uint64_t ncl = rows < (uint64_t)fit ? rows : (uint64_t)fit;                                           \
    le = launch_cluster(k, (unsigned)(ncl * cl), TT, 0, cl, false, stream, x, weight, bias,                     \
                        rows, cc, (uint32_t)cl, (uint32_t)slice4, eps, y, h, stds, mean, rstd, faults);         \
  }
      if (slice4 <= 2048) { if (rms) FB_LN_FWD_CLR(256, 8, true) else FB_LN_FWD_CLR(256, 8, false) }
      else { if (rms) FB_LN_FWD_CLR(512, 8, true) else FB_LN_FWD_CLR(512, 8, false) }
#undef FB_LN_FWD_CLR
      FB_CUDA(le);
      count_launch();
      return FB_OK;
    }
  }
  // 8193 .. 16384 columns with FB_LN_FWD_W=0 only: the staged 1024-thread pipeline (2-3 rows in flight per CTA;
  // 71 % of the copy rate at 16384 columns against 63 % for the 1024-thread register form and 90 % for 512 x 8).
  const PipePlan pp = pipe_plan(rows, cols, 1);
  if (cols > 8192 && pp.threads && rows >= 2 * (uint64_t)pp.grid && !(c.group == 512 && c.items == 8)) {
    unsigned int* faults = fault_word();
#define FB_LN_FWD_PIPE(TT, I)                                                                      \
  if (pp.threads == TT && pp.items == I) {                                                         \
    if (rms) {                                                                                     \
      FB_CUDA(allow_smem(ln_fwd_pipe_kernel<TT, I, true>, pp.smem));                               \
      ln_fwd_pipe_kernel<TT, I, true><<<pp.grid, TT, pp.smem, stream>>>(x, weight, bias, rows, cc, pp.stages, eps, \
                                                                        y, h, stds, mean, rstd, faults); \
    } else {                                                                                       \
      FB_CUDA(allow_smem(ln_fwd_pipe_kernel<TT, I, false>, pp.smem));                              \
      ln_fwd_pipe_kernel<TT, I, false><<<pp.grid, TT, pp.smem, stream>>>(x, weight, bias, rows, cc, pp.stages, eps, \
                                                                         y, h, stds, mean, rstd, faults); \
    }                                                                                              \
  } else
    FB_LN_FWD_PIPE(1024, 4) {
      return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_fwd: no pipelined kernel for %d threads x %d", pp.threads, pp.items);
    }
#undef FB_LN_FWD_PIPE
    FB_LAUNCHED("fb_layer_norm_fwd");
    return FB_OK;
  }
  if (!res && c.group == 32 && c.items <= 4 && ln_rows_enabled()) {
    // At most 512 columns.  Lanes per row x float4 per lane, by the row's float4 count: 4 x 2 (up to 8), 8 x 2
    // (16), 8 x 3 (24), 16 x 2 (32), 16 x 3 (48), 32 x 2 (64), 32 x 3 (96), 32 x 4 (128), four groups of rows per
    // step.  Never one float4 per lane: the work per row (shift, mean, reciprocal, their shuffles, the row's
    // addresses) is then paid per 16 bytes, and 32 / 64 / 128 columns run at 86 % of the copy rate, with eight
    // groups per step, where two float4 per lane reach the figures of 256 columns.
    const uint32_t c4 = cc / 4;
#define FB_LN_ROWS_K(L, I, R, EX, RM)                                                                              \
  {                                                                                                                \
    const uint64_t per = 8 * R * (32 / L);                                                                         \
    ln_fwd_rows_kernel<L, I, R, EX, RM><<<grid_full((rows + per - 1) / per), 256, 0, stream>>>(x, weight, bias, rows, cc, eps, \
                                                                                              y, h, stds, mean, rstd); \
  }
#define FB_LN_ROWS(L, I, R)                                                                                        \
  {                                                                                                                \
    const bool exact = c4 == (uint32_t)(L * I);                                                                    \
    if (rms) { if (exact) FB_LN_ROWS_K(L, I, R, true, true) else FB_LN_ROWS_K(L, I, R, false, true) }              \
    else { if (exact) FB_LN_ROWS_K(L, I, R, true, false) else FB_LN_ROWS_K(L, I, R, false, false) }                \
  }
    if (c4 <= 8) FB_LN_ROWS(4, 2, 4)
    else if (c4 <= 16) FB_LN_ROWS(8, 2, 4)
    else if (c4 <= 24) FB_LN_ROWS(8, 3, 4)
    else if (c4 <= 32) FB_LN_ROWS(16, 2, 4)
    else if (c4 <= 48) FB_LN_ROWS(16, 3, 4)
    else if (c4 <= 64) FB_LN_ROWS(32, 2, 4)
    else if (c4 <= 96) FB_LN_ROWS(32, 3, 4)
    else FB_LN_ROWS(32, 4, 4)
#undef FB_LN_ROWS
#undef FB_LN_ROWS_K
    FB_LAUNCHED("fb_layer_norm_fwd");
    return FB_OK;
  }
  WarpsCfg wc;
  if (!res && ln_fwd_warps_cfg(cols, &wc)) {
    const int mode = rms;
    switch (wc.items) {
      case 4: launch_ln_fwd_warps<4>(stream, wc.wpr, wc.rows_per_cta, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, mode, res, sum_out); break;
      case 5: launch_ln_fwd_warps<5>(stream, wc.wpr, wc.rows_per_cta, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, mode, res, sum_out); break;
      case 6: launch_ln_fwd_warps<6>(stream, wc.wpr, wc.rows_per_cta, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, mode, res, sum_out); break;
      case 7: launch_ln_fwd_warps<7>(stream, wc.wpr, wc.rows_per_cta, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, mode, res, sum_out); break;
      default: launch_ln_fwd_warps<8>(stream, wc.wpr, wc.rows_per_cta, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, mode, res, sum_out); break;
    }
    FB_LAUNCHED("fb_layer_norm_fwd");
    return FB_OK;
  }
  const int threads = c.group < 256 ? 256 : c.group;
  const int r = threads / c.group;
  const unsigned grid = grid_full((rows + r - 1) / r);
#define FB_LN_FWD(G, I)                                                                      \
  if (c.group == G && c.items == I) {                                                         \
    launch_ln_fwd<G, I>(stream, grid, x, weight, bias, rows, cc, eps, y, h, stds, mean, rstd, res ? 2 : rms, res, sum_out); \
  } else
  FB_LN_FWD(32, 1) FB_LN_FWD(32, 2) FB_LN_FWD(32, 4) FB_LN_FWD(32, 8) FB_LN_FWD(64, 4) FB_LN_FWD(128, 4)
  FB_LN_FWD(64, 8) FB_LN_FWD(128, 8) FB_LN_FWD(256, 8)
  FB_LN_FWD(256, 2) FB_LN_FWD(256, 4) FB_LN_FWD(512, 4) FB_LN_FWD(512, 8) FB_LN_FWD(1024, 4) FB_LN_FWD(1024, 8) {
    return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_fwd: no kernel for group %d items %d", c.group, c.items);
  }
#undef FB_LN_FWD
  FB_LAUNCHED("fb_layer_norm_fwd");
  return FB_OK;
}

int fb_layer_norm_fwd(fb_stream_t stream, const float* x, const float* weight, const float* bias,
                      uint64_t rows, uint64_t cols, float eps, float* y, float* h, float* stds,
                      float* mean, float* rstd) {
  return ln_fwd_impl(stream, x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, 0);
}

int fb_residual_layer_norm_fwd(fb_stream_t stream, const float* x, const float* residual,
                               const float* weight, const float* bias, uint64_t rows, uint64_t cols,
                               float eps, float* y, float* h, float* stds, float* mean, float* rstd,
                               float* sum_out) {
  const char* name = "fb_residual_layer_norm_fwd";
  uint64_t total;
  if (cols == 0) return fail(FB_ERR_INVALID_SHAPE, "%s: last dimension must be nonempty", name);
  if (mul_overflows(rows, cols, &total) || total > (UINT64_MAX >> 3))
    return fail(FB_ERR_INVALID_SHAPE, "%s: rows * cols overflows", name);
  if (rows == 0) return FB_OK;
  if (!x || !residual || !y) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const RowCfg c = ln_fwd_cfg(cols);
  const bool fused = c.group != 0 && cols <= 8192 && aligned16(x) && aligned16(residual) && aligned16(y) &&
                     (!h || aligned16(h)) && (!weight || aligned16(weight)) && (!bias || aligned16(bias)) &&
                     (!sum_out || aligned16(sum_out));
  if (fused) return ln_fwd_impl(stream, x, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, 0, residual, sum_out);
  // Rows the register kernel does not take: one extra pass forms the sum (in sum_out, or in y
  // and then normalised in place: every path reads a row completely before it writes it).
  float* sum = sum_out ? sum_out : y;
  if (int rc = fb_binary(stream, FB_BIN_ADD, 0.0f, 0.0f, x, residual, sum, total)) return rc;
  return ln_fwd_impl(stream, sum, weight, bias, rows, cols, eps, y, h, stds, mean, rstd, 0);
}

int fb_rms_norm_fwd(fb_stream_t stream, const float* x, const float* weight, uint64_t rows,
                    uint64_t cols, float eps, float* y, float* rstd) {
  return ln_fwd_impl(stream, x, weight, nullptr, rows, cols, eps, y, nullptr, nullptr, nullptr, rstd, 1);
}

// The split backward (row statistics, then a column-tiled sweep) serves the
// shapes the fused forms do not: decided by the shape alone, so the scratch
// query and the launch agree; buffers that turn out unaligned take it too.
static bool ln_bwd_split_shape(uint64_t cols) {
  const RowCfg c = ln_bwd_cfg(cols);
  return c.group == 0 || (c.group == 1024 && c.items == 8);
}
// Rows with a one-kernel backward (register, pipelined or cluster form), buffers permitting.
static bool ln_bwd_fused_shape(uint64_t cols) { return ln_cluster_plan(cols, 2).cl != 0 || !ln_bwd_split_shape(cols); }
static uint64_t ln_bwd_split_stats_bytes(uint64_t rows) { return ((rows * 2 * sizeof(float) + 15) / 16) * 16; }
static uint64_t ln_bwd_split_bytes(uint64_t rows, uint64_t cols) {
  const uint64_t a = col_scratch_bytes(col_plan(1, rows, cols, true), 1, cols, 2);
  const uint64_t b = col_scratch_bytes(col_plan(1, rows, cols, false), 1, cols, 2);
  return ln_bwd_split_stats_bytes(rows) + (a > b ? a : b);
}

uint64_t fb_layer_norm_bwd_workspace_bytes(uint64_t rows, uint64_t cols) {
  if (rows == 0 || cols == 0) return 0;
  const uint64_t fused = (uint64_t)ln_bwd_max_parts(rows, cols) * 2 * cols * sizeof(float);
  const uint64_t split = ln_bwd_split_bytes(rows, cols);
  // Unaligned buffers fall back to the split form whatever the shape, so the
  // scratch always covers it.
  return fused > split ? fused : split;
}

static int ln_bwd_impl(fb_stream_t stream, const float* g, const float* h, const float* stds,
                       const float* x, const float* mean, const float* rstd, const float* weight,
                       uint64_t rows, uint64_t cols, float* dx, float* dweight, float* dbias,
                       void* workspace, uint64_t workspace_bytes, int rms) {
  uint64_t total;
  if (cols == 0) return fail(FB_ERR_INVALID_SHAPE, "fb_layer_norm_bwd: last dimension must be nonempty");
  if (mul_overflows(rows, cols, &total) || total > (UINT64_MAX >> 3))
    return fail(FB_ERR_INVALID_SHAPE, "fb_layer_norm_bwd: rows * cols overflows");
  const bool from_x = x != nullptr;
  // RMS normalisation is the (x, mean, rstd) form without a mean: the kernels read a null mean as "none".
  if (rms ? (!x || !rstd || mean || h || stds)
          : (from_x ? (h || stds || !mean || !rstd) : (!h || !stds || mean || rstd)))
    return fail(FB_ERR_INVALID_ARG,
                "fb_layer_norm_bwd: pass either (h, stds) or (x, mean, rstd), not a mixture");
  if (rows == 0) {
    // No rows: the column sums are empty sums.
    if (dweight) { int rc = fb_fill(stream, dweight, 0.0f, cols); if (rc) return rc; }
    if (dbias) { int rc = fb_fill(stream, dbias, 0.0f, cols); if (rc) return rc; }
    return FB_OK;
  }
  if (!g || !dx) return fail(FB_ERR_INVALID_ARG, "fb_layer_norm_bwd: null buffer");
  const int wdw = dweight != nullptr, wdb = dbias != nullptr;
  uint32_t parts = ln_bwd_parts(rows, cols);
  const RowCfg c = ln_bwd_cfg(cols);
  const ClusterPlan cp = ln_cluster_plan(cols, 2);
  const bool fast = ln_bwd_fused_shape(cols) && aligned16(g) && aligned16(from_x ? x : h) && aligned16(dx) &&
                    (!weight || aligned16(weight));
  if ((wdw | wdb) || !fast) {
    const uint64_t need = fb_layer_norm_bwd_workspace_bytes(rows, cols);
    if (!workspace || workspace_bytes < need || !aligned16(workspace))
      return fail(FB_ERR_WORKSPACE, "fb_layer_norm_bwd: needs %llu bytes of 16-byte aligned scratch",
                  (unsigned long long)need);
  }
  float* part = static_cast<float*>(workspace);
  const float* hx = from_x ? x : h;
  const float* sa = from_x ? mean : stds;
  const float* sb = from_x ? rstd : nullptr;
  const PipePlan pp = pipe_plan(rows, cols, 2);
  const int mode = rms ? 2 : (from_x ? 1 : 0);
  if (!fast) {
    float* m12 = static_cast<float*>(workspace);
    void* col_ws = static_cast<char*>(workspace) + ln_bwd_split_stats_bytes(rows);
    const uint64_t col_ws_bytes = workspace_bytes - ln_bwd_split_stats_bytes(rows);
    const bool v4 = cols % 4 == 0 && aligned16(g) && aligned16(hx) && aligned16(dx);
#define FB_LN_SPLIT(VEC, FX)                                                                                  \
  {                                                                                                           \
    ln_bwd_rowstats_kernel<VEC, FX><<<grid_full(rows), kLnStreamThreads, 0, stream>>>(g, hx, sa, sb, weight,   \
                                                                                     rows, cols, m12);         \
    FB_LAUNCHED("fb_layer_norm_bwd");                                                                         \
    const LnBwdColSrc<FX> src{g, hx, sa, sb, weight, m12, dx, cols};                                           \
    return run_col_sum<2>(stream, src, 1, rows, cols, VEC == 4, wdw ? dweight : nullptr,                       \
                          wdb ? dbias : nullptr, 1.0f, col_ws, col_ws_bytes, "fb_layer_norm_bwd");             \
  }
    if (v4) {
      if (from_x) FB_LN_SPLIT(4, true) else FB_LN_SPLIT(4, false)
    } else {
      if (from_x) FB_LN_SPLIT(1, true) else FB_LN_SPLIT(1, false)
    }
#undef FB_LN_SPLIT
  } else if (cp.cl) {
    const uint32_t cc = (uint32_t)cols;
    unsigned int* faults = fault_word();
    cudaError_t le = cudaErrorInvalidValue;
    int fit = 0;
#define FB_LN_BWD_CL_K(TT, I, MD)                                                                       \
  {                                                                                                     \
    auto k = ln_bwd_cluster_kernel<TT, I, MD>;                                                          \
    FB_CUDA(allow_smem(k, cp.smem));                                                                    \
    FB_CUDA(resident_clusters(reinterpret_cast<const void*>(k), TT, cp.smem, cp.cl, &fit));             \
    const uint32_t cap = cluster_plan_max_clusters(cp);                                                 \
    uint64_t ncl = rows < (uint64_t)fit ? rows : (uint64_t)fit;                                         \
    if (ncl > cap) ncl = cap; /* the scratch is sized for `cap` partial rows */                         \
    parts = (uint32_t)ncl;                                                                              \
    le = launch_cluster(k, (unsigned)(ncl * cp.cl), TT, cp.smem, cp.cl, true, stream, g, hx, sa, sb,    \
                        weight, rows, cc, (uint32_t)cp.cl, cp.slice4, cp.stages, dx, part, wdw, wdb,     \
                        faults);                                                                                  \
  }
#define FB_LN_BWD_CL(TT, I)                                                    \
  if (cp.threads == TT && cp.items == I) {                                     \
    if (mode == 2) FB_LN_BWD_CL_K(TT, I, 2)                                    \
    else if (mode == 1) FB_LN_BWD_CL_K(TT, I, 1)                               \
    else FB_LN_BWD_CL_K(TT, I, 0)                                              \
  } else
    FB_LN_BWD_CL(256, 2) FB_LN_BWD_CL(512, 2) FB_LN_BWD_CL(512, 4) {
      return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_bwd: no cluster kernel for %d threads x %d", cp.threads, cp.items);
    }
#undef FB_LN_BWD_CL
#undef FB_LN_BWD_CL_K
    FB_CUDA(le);
  } else if (ln_bwd_rows_on() && c.group == 32 && cols <= ln_bwd_rows_max()) {
    // Lanes per row x float4 per lane: 8 x 1 up to 32 columns, 16 x 1 up to 64, 8 x 3 up to 96, 32 x 1 up to
    // 128, 16 x 3 up to 192, 32 x 2 up to 256, 32 x 3 up to 384, 32 x 4 beyond.
    const uint32_t cc = (uint32_t)cols, c4 = cc / 4;
    const uint32_t room = ln_bwd_parts(rows, cols);  // the scratch holds at least this many partial rows
#define FB_LN_BWD_ROWS_K(L, I, R, MD)                                                                           \
  {                                                                                                             \
    const uint64_t per = 8 * R * (32 / L), nblk = (rows + per - 1) / per;                                       \
    const uint64_t cap = (uint64_t)device_info().sm_count * 2;                                                  \
    parts = (uint32_t)(nblk < cap ? nblk : cap);                                                                \
    if (parts > room) parts = room;                                                                             \
    ln_bwd_rows_kernel<L, I, R, MD><<<parts, 256, 0, stream>>>(g, hx, sa, sb, weight, rows, cc, dx, part, wdw, wdb); \
  }
#define FB_LN_BWD_ROWS(L, I, R)                                                                                 \
  {                                                                                                             \
    if (mode == 2) FB_LN_BWD_ROWS_K(L, I, R, 2) else if (mode == 1) FB_LN_BWD_ROWS_K(L, I, R, 1)                \
    else FB_LN_BWD_ROWS_K(L, I, R, 0)                                                                           \
  }
    if (c4 <= 8) FB_LN_BWD_ROWS(8, 1, 4)
    else if (c4 <= 16) FB_LN_BWD_ROWS(16, 1, 4)
    else if (c4 <= 24) FB_LN_BWD_ROWS(8, 3, 2)
    else if (c4 <= 32) FB_LN_BWD_ROWS(32, 1, 4)
    else if (c4 <= 48) FB_LN_BWD_ROWS(16, 3, 2)
    else if (c4 <= 64) FB_LN_BWD_ROWS(32, 2, 4)
    else if (c4 <= 96) FB_LN_BWD_ROWS(32, 3, 2)
    else FB_LN_BWD_ROWS(32, 4, 2)
#undef FB_LN_BWD_ROWS
#undef FB_LN_BWD_ROWS_K
  } else if (pp.threads && rows >= 2 * (uint64_t)pp.grid) {
    const uint32_t cc = (uint32_t)cols;
    unsigned int* faults = fault_word();
    parts = pp.grid;
#define FB_LN_BWD_PIPE_MODE(TT, I, MD)                                                               \
  {                                                                                                  \
    FB_CUDA(allow_smem(ln_bwd_pipe_kernel<TT, I, MD>, pp.smem));                                     \
    FB_CUDA(launch_pdl(ln_bwd_pipe_kernel<TT, I, MD>, dim3(pp.grid), dim3(TT), pp.smem, stream, g, hx, sa, sb, \
                       weight, rows, cc, pp.stages, dx, part, wdw, wdb, faults));                    \
  }
#define FB_LN_BWD_PIPE(TT, I)                                                                        \
  if (pp.threads == TT && pp.items == I) {                                                           \
    if (mode == 2) FB_LN_BWD_PIPE_MODE(TT, I, 2)                                                     \
    else if (mode == 1) FB_LN_BWD_PIPE_MODE(TT, I, 1)                                                \
    else FB_LN_BWD_PIPE_MODE(TT, I, 0)                                                               \
  } else
    FB_LN_BWD_PIPE(64, 2) FB_LN_BWD_PIPE(128, 2) FB_LN_BWD_PIPE(256, 2) FB_LN_BWD_PIPE(256, 4) FB_LN_BWD_PIPE(512, 2) FB_LN_BWD_PIPE(512, 4) FB_LN_BWD_PIPE(1024, 4)
    FB_LN_BWD_PIPE(320, 2) FB_LN_BWD_PIPE(384, 2) FB_LN_BWD_PIPE(320, 4) FB_LN_BWD_PIPE(384, 4) FB_LN_BWD_PIPE(640, 4) FB_LN_BWD_PIPE(768, 4) {
      return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_bwd: no pipelined kernel for %d threads x %d", pp.threads, pp.items);
    }
#undef FB_LN_BWD_PIPE
#undef FB_LN_BWD_PIPE_MODE
  } else {
    const uint32_t cc = (uint32_t)cols;
#define FB_LN_BWD(G, I)                                                                          \
  if (c.group == G && c.items == I) {                                                            \
    launch_ln_bwd<G, I>(stream, parts, mode, g, hx, sa, sb, weight, rows, cc, dx, part, wdw, wdb); \
  } else
    FB_LN_BWD(32, 1) FB_LN_BWD(32, 2) FB_LN_BWD(32, 4) FB_LN_BWD(64, 4) FB_LN_BWD(128, 4)
    FB_LN_BWD(256, 4) FB_LN_BWD(512, 4) FB_LN_BWD(1024, 4) FB_LN_BWD(1024, 8) {
      return fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_bwd: no kernel for group %d items %d", c.group, c.items);
    }
#undef FB_LN_BWD
  }
  FB_LAUNCHED("fb_layer_norm_bwd");
  if (wdw | wdb) {
    FB_CUDA(launch_pdl(ln_bwd_finalize_kernel, dim3((unsigned)((cols + 7) / 8)), dim3(1024), 0, stream,
                       (const float*)part, parts, cols, wdw ? dweight : (float*)nullptr, wdb ? dbias : (float*)nullptr));
    FB_LAUNCHED("fb_layer_norm_bwd finalize");
  }
  return FB_OK;
}

int fb_layer_norm_bwd(fb_stream_t stream, const float* g, const float* h, const float* stds,
                      const float* x, const float* mean, const float* rstd, const float* weight,
                      uint64_t rows, uint64_t cols, float* dx, float* dweight, float* dbias,
                      void* workspace, uint64_t workspace_bytes) {
  return ln_bwd_impl(stream, g, h, stds, x, mean, rstd, weight, rows, cols, dx, dweight, dbias, workspace,
                     workspace_bytes, 0);
}

int fb_rms_norm_bwd(fb_stream_t stream, const float* g, const float* x, const float* rstd,
                    const float* weight, uint64_t rows, uint64_t cols, float* dx, float* dweight,
                    void* workspace, uint64_t workspace_bytes) {
  return ln_bwd_impl(stream, g, nullptr, nullptr, x, nullptr, rstd, weight, rows, cols, dx, dweight, nullptr,
                     workspace, workspace_bytes, 1);
}

}  // extern "C"

// ------------------------------------------------- allocation-free variant
// Some hosts of this library cannot hand out scratch: code running inside a
// CUDA-graph-replayed step or a real-time loop that has frozen its memory
// pool, a plug-in whose host allocator is not reachable from the call site,
// or a process that is at its memory limit and must not grow.  For them the
// LayerNorm backward is also offered with its scratch living in the library
// image itself: a fixed device array that every GPU loading the library holds
// until the process exits.
#include <mutex>

static __device__ __align__(256) unsigned char g_ln_static_scratch[FB_LN_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_ln_static_scratch per device ordinal.  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel may
// use, so the address is asked for once per device (with that device current)
// and remembered.
void* g_ln_static_ptr[64];
bool g_ln_static_ready[64];
std::mutex g_ln_static_mu;

int ln_static_scratch(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fb::cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fb::fail(FB_ERR_UNSUPPORTED, "fb_layer_norm_bwd_static: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_ln_static_mu);
  if (!g_ln_static_ready[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ln_static_scratch);
    if (e != cudaSuccess) return fb::cuda_fail(e, "cudaGetSymbolAddress(g_ln_static_scratch)");
    if (!p) return fb::fail(FB_ERR_CUDA, "fb_layer_norm_bwd_static: the scratch symbol has no device address");
    g_ln_static_ptr[dev] = p;
    g_ln_static_ready[dev] = true;
  }
  *out = g_ln_static_ptr[dev];
  return FB_OK;
}
}  // namespace

extern "C" int fb_layer_norm_bwd_static(fb_stream_t stream, const float* g, const float* h,
                                        const float* stds, const float* x, const float* mean,
                                        const float* rstd, const float* weight, uint64_t rows,
                                        uint64_t cols, float* dx, float* dweight, float* dbias) {
  // Scratch is needed for the column sums and, whatever the outputs, by the
  // two-kernel form that rows without a fused form take (the same condition
  // as in ln_bwd_impl), so a dx-only call on such a shape is refused here,
  // with this entry's own message, when it is too large.
  const float* rows_in = x ? x : h;
  const bool fused_form = ln_bwd_fused_shape(cols) && fb::aligned16(g) && fb::aligned16(rows_in) &&
                          fb::aligned16(dx) && (!weight || fb::aligned16(weight));
  const uint64_t need =
      (rows && cols && (dweight || dbias || !fused_form)) ? fb_layer_norm_bwd_workspace_bytes(rows, cols) : 0;
  if (need > FB_LN_STATIC_SCRATCH_BYTES)
    return fb::fail(FB_ERR_WORKSPACE,
                    "fb_layer_norm_bwd_static: rows %llu x cols %llu needs %llu bytes of scratch, the built-in "
                    "buffer holds %llu; use fb_layer_norm_bwd with caller scratch",
                    (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)need,
                    (unsigned long long)FB_LN_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (int rc = ln_static_scratch(&scratch)) return rc;
  // Nothing in the scratch has to start at zero: every partial row the
  // finalize step reads is written in full by the pass before it.
  return fb_layer_norm_bwd(stream, g, h, stds, x, mean, rstd, weight, rows, cols, dx, dweight, dbias,
                           scratch, FB_LN_STATIC_SCRATCH_BYTES);
}
