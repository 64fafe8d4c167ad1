// Softmax / log_softmax forward and backward for rows shorter than 256 columns: several rows per
// warp.  One row per warp leaves most lanes of a short row idle and pays the row's reductions, its
// reciprocal and its addresses per 16 bytes: the forward ran at 23 / 44 / 62 / 78 % of the copy rate
// at 32 / 64 / 96 / 128 columns, the backward at 40 / 74 / 90 % at 32 / 64 / 96.  Here LPR lanes (4, 8
// or 16) hold one row, ITEMS (2 .. 4) float4 each, so a warp holds 32 / LPR rows side by side and
// takes RW such groups per step: every load of the step is issued before any value is used, the
// rows' reductions run transposed (lanes_transpose_reduce) and the exact max-then-sum order of the
// wide kernels is kept.  One CTA of 8 warps per block of 8 * RW * 32 / LPR rows on a full grid.
#pragma once
#include "common.cuh"

namespace fb {

template <int LPR, int ITEMS, int RW, bool LOG>
__global__ void __launch_bounds__(256, ITEMS <= 2 ? 3 : 2)
softmax_fwd_rows_kernel(const float* __restrict__ x, uint64_t rows, uint32_t cols, float* __restrict__ y) {
  constexpr int SUB = 32 / LPR, RPW = SUB * RW, SPAN = LPR / RW;
  const uint32_t cols4 = cols / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const int first = sub * LPR;
  const uint64_t nblk = (rows + 8 * RPW - 1) / (8 * RPW);
  pdl_wait();
  pdl_trigger();
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t r0 = (blk * 8 + warp) * RPW;
    float4 v[RW][ITEMS];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        v[j][k] = (row < rows && c < cols4) ? ld_stream4(x + row * cols + c * 4)
                                            : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
    }
    float m[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      m[j] = -INFINITY;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) m[j] = fmaxf(m[j], fmaxf(fmaxf(v[j][k].x, v[j][k].y), fmaxf(v[j][k].z, v[j][k].w)));
    }
    const float my_m = lanes_transpose_max<LPR, RW>(m, l);
    float s[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const float mj = __shfl_sync(0xffffffffu, my_m, first + j * SPAN);
      s[j] = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        float4 e;
        v[j][k].x -= mj; v[j][k].y -= mj; v[j][k].z -= mj; v[j][k].w -= mj;
        e.x = __expf(v[j][k].x); e.y = __expf(v[j][k].y); e.z = __expf(v[j][k].z); e.w = __expf(v[j][k].w);
        if (c < cols4) s[j] += (e.x + e.y) + (e.z + e.w);
        if constexpr (!LOG) v[j][k] = e;
      }
    }
    const float my_s = lanes_transpose_sum<LPR, RW>(s, l);
    const float my_f = LOG ? logf(my_s) : 1.0f / my_s;  // what the outputs of this lane's row need
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
      const float f = __shfl_sync(0xffffffffu, my_f, first + j * SPAN);
      if (row < rows) {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = l + k * LPR;
          if (c < cols4) {
            float4 o;
            if constexpr (LOG) o = make_float4(v[j][k].x - f, v[j][k].y - f, v[j][k].z - f, v[j][k].w - f);
            else o = make_float4(v[j][k].x * f, v[j][k].y * f, v[j][k].z * f, v[j][k].w * f);
            st_stream4(y + row * cols + c * 4, o);
          }
        }
      }
    }
  }
}

// dx = y * (g - sum(g * y)) (softmax) or g - exp(y) * sum(g) (log_softmax), as in softmax_bwd_reg_kernel.
template <int LPR, int ITEMS, int RW, bool LOG>
__global__ void __launch_bounds__(256, 2)
softmax_bwd_rows_kernel(const float* __restrict__ g, const float* __restrict__ y, uint64_t rows, uint32_t cols,
                        float* __restrict__ dx) {
  constexpr int SUB = 32 / LPR, RPW = SUB * RW, SPAN = LPR / RW;
  const uint32_t cols4 = cols / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const int first = sub * LPR;
  const uint64_t nblk = (rows + 8 * RPW - 1) / (8 * RPW);
  pdl_wait();
  pdl_trigger();
  for (uint64_t blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
    const uint64_t r0 = (blk * 8 + warp) * RPW;
    float4 gv[RW][ITEMS], yv[RW][ITEMS];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const uint32_t c = l + k * LPR;
        if (row < rows && c < cols4) {
          gv[j][k] = ld_stream4(g + row * cols + c * 4);
          yv[j][k] = ld_stream4(y + row * cols + c * 4);
        } else {
          gv[j][k] = yv[j][k] = make_float4(0, 0, 0, 0);
        }
      }
    }
    float s[RW];
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      s[j] = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        if constexpr (LOG) s[j] += (gv[j][k].x + gv[j][k].y) + (gv[j][k].z + gv[j][k].w);
        else s[j] += (gv[j][k].x * yv[j][k].x + gv[j][k].y * yv[j][k].y) + (gv[j][k].z * yv[j][k].z + gv[j][k].w * yv[j][k].w);
      }
    }
    const float my_s = lanes_transpose_sum<LPR, RW>(s, l);
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      const uint64_t row = r0 + j * SUB + sub;
      const float t = __shfl_sync(0xffffffffu, my_s, first + j * SPAN);
      if (row < rows) {
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
          const uint32_t c = l + k * LPR;
          if (c < cols4) {
            float4 o;
            if constexpr (LOG) {
              o.x = gv[j][k].x - __expf(yv[j][k].x) * t; o.y = gv[j][k].y - __expf(yv[j][k].y) * t;
              o.z = gv[j][k].z - __expf(yv[j][k].z) * t; o.w = gv[j][k].w - __expf(yv[j][k].w) * t;
            } else {
              o.x = yv[j][k].x * (gv[j][k].x - t); o.y = yv[j][k].y * (gv[j][k].y - t);
              o.z = yv[j][k].z * (gv[j][k].z - t); o.w = yv[j][k].w * (gv[j][k].w - t);
            }
            st_stream4(dx + row * cols + c * 4, o);
          }
        }
      }
    }
  }
}

}  // namespace fb
