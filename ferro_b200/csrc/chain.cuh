// Device side of the strided pointwise engine (see chain.cu for the overview).
// Every kernel is a template over a Runner: the thing that evaluates the
// program on the N elements a thread holds.
//   Interp        interprets the step list at run time (any program);
//   Static<PROG>  (chain_static.cu) is the same program unrolled at compile
//                 time: no dispatch, constant kinds, and the compiler can fold
//                 work that is identical for all N elements (an operand that
//                 is broadcast along the row).
#pragma once
#include "common.cuh"
#include "math.cuh"

namespace fb {

constexpr int kMaxOps = FB_CHAIN_MAX_OPERANDS;
constexpr int kMaxSteps = FB_CHAIN_MAX_STEPS;
constexpr int kChThreads = 256;

// n / d for n < 2^31 with one multiply-high (d >= 1).
struct FastDiv {
  uint32_t d, magic, shift;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d;
  uint32_t shift = 0;
  while (shift < 32 && (1ull << shift) < d) ++shift;
  f.shift = shift;
  f.magic = (uint32_t)(((1ull << 32) * ((1ull << shift) - d)) / d + 1);
  return f;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) {
  return (uint32_t)(((uint64_t)__umulhi(n, f.magic) + n) >> f.shift);
}

struct Step {
  int8_t opcode, dst, kind, swap;  // kind: public or internal (math.cuh) code
  int16_t src;                     // LOAD: operand; BINARY: 0 other reg, 1 immediate, 8+k operand k
  float p0, p1;
};

struct ChainParams {
  int n_steps, n_ops, rank;
  uint64_t n;                    // output elements
  uint64_t shape[FB_MAX_RANK];   // collapsed, outermost first
  FastDiv div[FB_MAX_RANK];      // flat kernel, narrow path (innermost in vec units)
  const float* ptr[kMaxOps];     // already advanced by the view offset
  int64_t stride[kMaxOps][FB_MAX_RANK];
  Step steps[kMaxSteps];
};

template <int N>
__device__ __forceinline__ void unary_vec(int kind, float p0, float p1, float (&x)[N]) {
#define FB_CASE(K)                                                   \
  case K:                                                            \
    _Pragma("unroll") for (int j = 0; j < N; ++j) x[j] = unary_apply(K, p0, p1, x[j]); \
    break;
  switch (kind) {
    FB_CASE(FB_UN_NEG) FB_CASE(FB_UN_RELU) FB_CASE(FB_UN_EXP) FB_CASE(FB_UN_SIGMOID)
    FB_CASE(FB_UN_TANH) FB_CASE(FB_UN_SQRT) FB_CASE(FB_UN_ABS) FB_CASE(FB_UN_SIGN)
    FB_CASE(FB_UN_LOG) FB_CASE(FB_UN_POWF) FB_CASE(FB_UN_CLAMP) FB_CASE(FB_UN_GTZ)
    FB_CASE(FB_UN_GELU) FB_CASE(FB_UN_GELU_ERF) FB_CASE(FB_UN_GELU_ERF_GRAD) FB_CASE(FB_UN_SILU)
    FB_CASE(FBI_POWF_SQRT) FB_CASE(FBI_POWF_RSQRT) FB_CASE(FBI_POWF_RCP) FB_CASE(FBI_POWF_RSQ)
    FB_CASE(FBI_POWF_SQ) FB_CASE(FBI_POWF_CUBE) FB_CASE(FBI_POWF_1_5) FB_CASE(FBI_POWF_GENERIC)
    FB_CASE(FBI_CLAMP_ORDERED)
    default: break;
  }
#undef FB_CASE
}

// a = a (kind) b, or b (kind) a when swap.
template <int N>
__device__ __forceinline__ void binary_vec(int kind, bool swap, float p0, float p1, float (&a)[N],
                                           const float (&b)[N]) {
#define FB_CASE(K)                                                                     \
  case K:                                                                              \
    if (swap) {                                                                        \
      _Pragma("unroll") for (int j = 0; j < N; ++j) a[j] = binary_apply(K, p0, p1, b[j], a[j]); \
    } else {                                                                           \
      _Pragma("unroll") for (int j = 0; j < N; ++j) a[j] = binary_apply(K, p0, p1, a[j], b[j]); \
    }                                                                                  \
    break;
  switch (kind) {
    FB_CASE(FB_BIN_ADD) FB_CASE(FB_BIN_SUB) FB_CASE(FB_BIN_MUL) FB_CASE(FB_BIN_DIV)
    FB_CASE(FB_BIN_RELU_BACKWARD) FB_CASE(FB_BIN_TANH_BWD) FB_CASE(FB_BIN_SIGMOID_BWD)
    FB_CASE(FB_BIN_SQRT_BWD) FB_CASE(FB_BIN_ABS_BWD) FB_CASE(FB_BIN_LOG_BWD)
    FB_CASE(FB_BIN_POWF_BWD) FB_CASE(FB_BIN_CLAMP_BWD)
    default: break;
  }
#undef FB_CASE
}

// One step acting in place on register R, with O the other register.
template <int N, class Fetch>
__device__ __forceinline__ void exec_step(const Step& st, float (&R)[N], const float (&O)[N], Fetch& fetch) {
  switch (st.opcode) {
    case FB_CH_LOAD: fetch(st.src, R); break;
    case FB_CH_IMM:
#pragma unroll
      for (int j = 0; j < N; ++j) R[j] = st.p0;
      break;
    case FB_CH_UNARY: unary_vec<N>(st.kind, st.p0, st.p1, R); break;
    case FB_CH_BINARY: {
      if (st.src == FB_CH_SRC_OTHER_REG) {
        binary_vec<N>(st.kind, st.swap != 0, st.p0, st.p1, R, O);
      } else {
        float other[N];
        if (st.src == FB_CH_SRC_IMM) {
#pragma unroll
          for (int j = 0; j < N; ++j) other[j] = st.p1;
        } else {
          fetch(st.src - FB_CH_SRC_OPERAND0, other);
        }
        binary_vec<N>(st.kind, st.swap != 0, st.p0, st.p1, R, other);
      }
      break;
    }
    default: break;
  }
}

// The run-time interpreter.  The step loop is warp-uniform; the two registers
// are addressed by (uniform) branching rather than by selects.  (A form that
// keeps one copy of every kind's code - registers trading places, one fetch
// site, operands exchanged for swapped steps - was measured slower, 2150 us
// against 1790 us on the [16384, 16384] gate-clamp chain: the interpreter is
// bound by the number of instructions it issues, about 180 per element there
// against 44 for the compiled program, not by the size of its code.)
struct Interp {
  static constexpr int kTileCtasPerSm = 2;  // register budget hint for the tile kernels
  template <int N, class Fetch>
  static __device__ __forceinline__ void run(const ChainParams& P, Fetch& fetch, float (&V)[N]) {
    float T[N];
#pragma unroll
    for (int j = 0; j < N; ++j) V[j] = T[j] = 0.0f;
#pragma unroll 1
    for (int s = 0; s < P.n_steps; ++s) {
      const Step st = P.steps[s];
      if (st.dst == 0) exec_step<N>(st, V, T, fetch);
      else exec_step<N>(st, T, V, fetch);
    }
  }
};

// ------------------------------------------------------------ segment kernel
// Work item = (outer index, run of 256 * VEC * U innermost elements).
// VEC = 4: every operand is unit-stride or broadcast along the innermost dim
// and float4-aligned; VEC = 1: arbitrary innermost strides.
template <int VEC, int U, class Runner>
__global__ void __launch_bounds__(kChThreads)
chain_seg_kernel(const __grid_constant__ ChainParams P, uint64_t nseg, float* __restrict__ out) {
  constexpr int N = VEC * U;
  const int last = P.rank - 1;
  const uint64_t inner = P.shape[last];
  const uint64_t outer = P.n / inner;
  const uint64_t items = outer * nseg;
  for (uint64_t it = blockIdx.x; it < items; it += gridDim.x) {
    const uint64_t o = it / nseg, sg = it - o * nseg;
    // Outer coordinates -> operand bases (uniform across the CTA).
    int64_t base[kMaxOps];
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) base[k] = 0;
    uint64_t rem = o;
    for (int d = last - 1; d >= 0; --d) {
      const uint64_t q = rem / P.shape[d], c = rem - q * P.shape[d];
      rem = q;
#pragma unroll
      for (int k = 0; k < kMaxOps; ++k)
        if (k < P.n_ops) base[k] += (int64_t)c * P.stride[k][d];
    }
    const uint64_t col0 = sg * (uint64_t)(kChThreads * N) + (uint64_t)threadIdx.x * VEC;
    auto fetch = [&](int k, float (&dst)[N]) {
      int64_t b = 0;
#pragma unroll
      for (int q = 0; q < kMaxOps; ++q)
        if (q == k) b = base[q];
      const int64_t si = P.stride[k][last];
      const float* p = P.ptr[k] + b;
      if (si == 0) {  // broadcast along the run: one scalar
        const float t = __ldg(p);
#pragma unroll
        for (int j = 0; j < N; ++j) dst[j] = t;
        return;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t col = col0 + (uint64_t)u * kChThreads * VEC;
        if constexpr (VEC == 4) {
          float4 t = make_float4(0, 0, 0, 0);
          if (col < inner) t = __ldg(reinterpret_cast<const float4*>(p + col));
          dst[u * 4 + 0] = t.x; dst[u * 4 + 1] = t.y; dst[u * 4 + 2] = t.z; dst[u * 4 + 3] = t.w;
        } else {
          dst[u] = col < inner ? __ldg(p + (int64_t)col * si) : 0.0f;
        }
      }
    };
    float V[N];
    Runner::template run<N>(P, fetch, V);
    float* orow = out + o * inner;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t col = col0 + (uint64_t)u * kChThreads * VEC;
      if (col < inner) {
        if constexpr (VEC == 4) st_stream4(orow + col, make_float4(V[u * 4], V[u * 4 + 1], V[u * 4 + 2], V[u * 4 + 3]));
        else st_stream(orow + col, V[u]);
      }
    }
  }
}

// --------------------------------------------------------------- flat kernel
// One work item (VEC adjacent innermost elements) per thread per iteration.
// WIDE = false: fewer than 2^31 items, 32-bit index math.
template <int VEC, bool WIDE>
__global__ void __launch_bounds__(kChThreads)
chain_flat_kernel(const __grid_constant__ ChainParams P, float* __restrict__ out) {
  const uint64_t items = P.n / VEC;
  const uint64_t stride = (uint64_t)gridDim.x * kChThreads;
  const int last = P.rank - 1;
  for (uint64_t it = (uint64_t)blockIdx.x * kChThreads + threadIdx.x; it < items; it += stride) {
    int64_t off[kMaxOps];
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) off[k] = 0;
    if constexpr (WIDE) {
      uint64_t rem = it;
      for (int d = last; d >= 0; --d) {
        const uint64_t ext = d == last ? P.shape[d] / VEC : P.shape[d];
        const uint64_t q = rem / ext, c = rem - q * ext;
        rem = q;
        const int64_t cc = (int64_t)(d == last ? c * VEC : c);
#pragma unroll
        for (int k = 0; k < kMaxOps; ++k)
          if (k < P.n_ops) off[k] += cc * P.stride[k][d];
      }
    } else {
      uint32_t rem = (uint32_t)it;
      for (int d = last; d >= 0; --d) {
        const uint32_t q = fdiv(rem, P.div[d]), c = rem - q * P.div[d].d;
        rem = q;
        const int64_t cc = (int64_t)(d == last ? (uint64_t)c * VEC : (uint64_t)c);
#pragma unroll
        for (int k = 0; k < kMaxOps; ++k)
          if (k < P.n_ops) off[k] += cc * P.stride[k][d];
      }
    }
    auto fetch = [&](int k, float (&dst)[VEC]) {
      int64_t o = 0;
#pragma unroll
      for (int q = 0; q < kMaxOps; ++q)
        if (q == k) o = off[q];
      const float* p = P.ptr[k] + o;
      if constexpr (VEC == 4) {
        if (P.stride[k][last] == 1) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(p));
          dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
        } else {
          const float t = __ldg(p);
          dst[0] = dst[1] = dst[2] = dst[3] = t;
        }
      } else {
        dst[0] = __ldg(p);
      }
    };
    float V[VEC];
    Interp::run<VEC>(P, fetch, V);
    if constexpr (VEC == 4) st_stream4(out + it * 4, make_float4(V[0], V[1], V[2], V[3]));
    else out[it] = V[0];
  }
}

// -------------------------------------------------------------- tile kernels
// Output viewed as [batch..., A, ..., B] with B innermost.  Operands flagged
// in `tmask` (at most two) are unit-stride along A and are staged through
// shared memory; the others are read directly with lanes along B.
enum { kOpDirect = 0, kOpBcastB = 1, kOpStaged = 2 };
struct TileParams {
  ChainParams c;
  uint32_t tmask;
  uint32_t modes;  // 2 bits per operand: direct (unit stride along B), broadcast along B, staged
  int tslot[kMaxOps];  // shared-memory slot of a staged operand
  uint32_t tiles_a, tiles_b;
  uint64_t batches;
  int dim_a;
  uint64_t ostride[FB_MAX_RANK];  // output (row-major) stride of every collapsed dim
};

constexpr int kTile = 64;
constexpr int kTileSlots = 2;

// Scalar form: any extents and alignments.  Thread (tx, ty) of 32 x 8 owns
// a = ty + 8m (m < 8), b = tx + 32h (h < 2); slots are [b][a] padded by one.
struct ScalarTile {
  static constexpr int kThreads = kChThreads, kMinCtas = 0;
  static constexpr int kSmemFloats = kTileSlots * kTile * (kTile + 1);
  template <class Runner>
  static __device__ __forceinline__ void run(const TileParams& TP, float* smem, const int64_t (&boff)[kMaxOps],
                                             uint64_t obatch, uint32_t ia, uint32_t ib, float* __restrict__ out) {
    const ChainParams& P = TP.c;
    constexpr int LD = kTile + 1;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int last = P.rank - 1, da = TP.dim_a;
    const uint64_t A = P.shape[da], B = P.shape[last];
    const uint64_t a0 = (uint64_t)ia * kTile, b0 = (uint64_t)ib * kTile;
    __syncthreads();  // the previous tile's readers are done with the slots
    for (int k = 0; k < P.n_ops; ++k) {
      if (!((TP.tmask >> k) & 1)) continue;
      int64_t o = 0;
#pragma unroll
      for (int q = 0; q < kMaxOps; ++q)
        if (q == k) o = boff[q];
      const float* p = P.ptr[k] + o;
      const int64_t sb = P.stride[k][last];
      float* slot = smem + TP.tslot[k] * kTile * LD;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const int bl = ty + 8 * m;
        const uint64_t b = b0 + bl;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int al = tx + 32 * h;
          const uint64_t a = a0 + al;
          slot[bl * LD + al] = (a < A && b < B) ? __ldg(p + (int64_t)a + (int64_t)b * sb) : 0.0f;
        }
      }
    }
    __syncthreads();
    auto fetch = [&](int k, float (&dst)[16]) {
      int64_t o = 0;
#pragma unroll
      for (int q = 0; q < kMaxOps; ++q)
        if (q == k) o = boff[q];
      if ((TP.tmask >> k) & 1) {
        const float* slot = smem + TP.tslot[k] * kTile * LD;
#pragma unroll
        for (int m = 0; m < 8; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) dst[m * 2 + h] = slot[(tx + 32 * h) * LD + ty + 8 * m];
      } else {
        const float* p = P.ptr[k] + o;
        const int64_t sa = P.stride[k][da], sb = P.stride[k][last];
#pragma unroll
        for (int m = 0; m < 8; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t a = a0 + ty + 8 * m, b = b0 + tx + 32 * h;
            dst[m * 2 + h] = (a < A && b < B) ? __ldg(p + (int64_t)a * sa + (int64_t)b * sb) : 0.0f;
          }
      }
    };
    float V[16];
    Runner::template run<16>(P, fetch, V);
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint64_t a = a0 + ty + 8 * m, b = b0 + tx + 32 * h;
        if (a < A && b < B) st_stream(out + obatch + a * TP.ostride[da] + b, V[m * 2 + h]);
      }
  }
};

// Vector form: A and B multiples of 4 and every access float4-aligned.
// Thread t owns a = t/16 + 16m (m < 4) and the four columns b = 4*(t%16)..+3.
// A staged operand is read with float4 along A and scattered into a [a][b]
// slot whose 4-column groups are XOR-swizzled by (a/4)%8, which makes the
// float4 reads of the compute phase conflict-free (writes are 2-way).
//
// MODES >= 0 fixes every operand's class (TileParams::modes) at compile time:
// the class tests fold, and with a compiled program the four equal lanes of an
// operand that is broadcast along B are one value to the compiler, so a
// sub-chain on such an operand is evaluated once per row instead of once per
// element.  MODES < 0 reads the classes from the launch parameters.
template <int MODES>
struct VectorTile {
  static constexpr int kThreads = kChThreads, kMinCtas = 0;
  static constexpr int kSmemFloats = kTileSlots * kTile * kTile;
  static __device__ __forceinline__ int swz(int a, int b) { return b ^ (((a >> 2) & 7) << 2); }
  static __device__ __forceinline__ int mode(const TileParams& TP, int k) {
    return (int)(((MODES >= 0 ? (uint32_t)MODES : TP.modes) >> (2 * k)) & 3u);
  }
  template <class Runner>
  static __device__ __forceinline__ void run(const TileParams& TP, float* smem, const int64_t (&boff)[kMaxOps],
                                             uint64_t obatch, uint32_t ia, uint32_t ib, float* __restrict__ out) {
    const ChainParams& P = TP.c;
    const int t16 = threadIdx.x & 15, q16 = threadIdx.x >> 4;
    const int last = P.rank - 1, da = TP.dim_a;
    const uint64_t A = P.shape[da], B = P.shape[last];
    const uint64_t a0 = (uint64_t)ia * kTile, b0 = (uint64_t)ib * kTile;
    // Extents are multiples of 4, so a float4 is inside or outside as a whole.
    // Bit m of rows_a: row a0 + q16 + 16m exists; of rows_b: row b0 + q16 + 16m.
    uint32_t rows_a = 0, rows_b = 0;
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      rows_a |= (uint32_t)(a0 + q16 + 16 * m < A) << m;
      rows_b |= (uint32_t)(b0 + q16 + 16 * m < B) << m;
    }
    const bool col_a = a0 + 4 * t16 < A, col_b = b0 + 4 * t16 < B;
    __syncthreads();  // the previous tile's readers are done with the slots
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) {
      if (mode(TP, k) != kOpStaged) continue;
      const int64_t sb = P.stride[k][last];
      const float* p = P.ptr[k] + boff[k] + (int64_t)(a0 + 4 * t16) + (int64_t)(b0 + q16) * sb;
      float* slot = smem + TP.tslot[k] * kTile * kTile;
      const int al = 4 * t16;
      float4 v[4];
#pragma unroll
      for (int m = 0; m < 4; ++m)
        v[m] = (col_a && ((rows_b >> m) & 1)) ? __ldg(reinterpret_cast<const float4*>(p + (int64_t)(16 * m) * sb))
                                              : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int c = swz(al, q16 + 16 * m);  // the swizzle term is the same for al .. al + 3
        slot[(al + 0) * kTile + c] = v[m].x;
        slot[(al + 1) * kTile + c] = v[m].y;
        slot[(al + 2) * kTile + c] = v[m].z;
        slot[(al + 3) * kTile + c] = v[m].w;
      }
    }
    __syncthreads();
    const int bl = 4 * t16;
    auto fetch = [&](int k, float (&dst)[16]) {
      int64_t o = 0;
#pragma unroll
      for (int q = 0; q < kMaxOps; ++q)
        if (q == k) o = boff[q];
      const int md = mode(TP, k);
      if (md == kOpStaged) {
        const float* slot = smem + TP.tslot[k] * kTile * kTile;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const int al = q16 + 16 * m;
          const float4 t = *reinterpret_cast<const float4*>(slot + al * kTile + swz(al, bl));
          dst[m * 4 + 0] = t.x; dst[m * 4 + 1] = t.y; dst[m * 4 + 2] = t.z; dst[m * 4 + 3] = t.w;
        }
      } else if (md == kOpBcastB) {
        const int64_t sa = P.stride[k][da];
        const float* p = P.ptr[k] + o + (int64_t)(a0 + q16) * sa;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float s = ((rows_a >> m) & 1) ? __ldg(p + (int64_t)(16 * m) * sa) : 0.0f;
          dst[m * 4 + 0] = s; dst[m * 4 + 1] = s; dst[m * 4 + 2] = s; dst[m * 4 + 3] = s;
        }
      } else {
        const int64_t sa = P.stride[k][da];
        const float* p = P.ptr[k] + o + (int64_t)(a0 + q16) * sa + (int64_t)(b0 + bl);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float4 t = (col_b && ((rows_a >> m) & 1)) ? __ldg(reinterpret_cast<const float4*>(p + (int64_t)(16 * m) * sa))
                                                          : make_float4(0, 0, 0, 0);
          dst[m * 4 + 0] = t.x; dst[m * 4 + 1] = t.y; dst[m * 4 + 2] = t.z; dst[m * 4 + 3] = t.w;
        }
      }
    };
    float V[16];
    Runner::template run<16>(P, fetch, V);
    float* po = out + obatch + (a0 + q16) * TP.ostride[da] + b0 + bl;
#pragma unroll
    for (int m = 0; m < 4; ++m)
      if (col_b && ((rows_a >> m) & 1))
        st_stream4(po + (uint64_t)(16 * m) * TP.ostride[da], make_float4(V[m * 4], V[m * 4 + 1], V[m * 4 + 2], V[m * 4 + 3]));
  }
};

// Interior form for compiled programs.  Requirements, checked on the host:
// collapsed rank 2 (one batch), both extents multiples of the tile, every
// operand offset inside a tile below 2^31 elements.  Nothing is predicated,
// in-tile offsets are 32-bit, and a thread owns RPT rows of 4 columns
// (RPT = 8: 128 threads per tile, 32 elements per thread), so that what a
// thread spends per tile on decoding, addresses and barriers is shared by
// twice as many elements as in VectorTile.  A staged operand is loaded with
// float4 along A for four adjacent b, transposed in registers and written with
// float4 stores along B into the same XOR-swizzled [a][b] slot VectorTile
// uses: 4 vector stores where that form issues 16 scalar ones.
template <int MODES, int RPT>
struct FullTile {
  static constexpr int kQ = kTile / RPT;       // row groups per tile: thread rows are q + kQ * m
  static constexpr int kThreads = 16 * kQ;
  static constexpr int kMinCtas = RPT == 8 ? 5 : 0;
  static constexpr int kN = 4 * RPT;
  static constexpr int kSmemFloats = kTileSlots * kTile * kTile;
  static __device__ __forceinline__ int swz(int a, int b) { return b ^ (((a >> 2) & 7) << 2); }
  static constexpr int mode(int k) { return (MODES >> (2 * k)) & 3; }
  template <class Runner>
  static __device__ __forceinline__ void run(const TileParams& TP, float* smem, const int64_t (&)[kMaxOps], uint64_t,
                                             uint32_t ia, uint32_t ib, float* __restrict__ out) {
    const ChainParams& P = TP.c;
    const int t16 = threadIdx.x & 15, q = threadIdx.x >> 4;
    const uint32_t a0 = ia * kTile, b0 = ib * kTile;
    __syncthreads();  // the previous tile's readers are done with the slots
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) {
      if (mode(k) != kOpStaged) continue;
      // Thread (t16, q): the four a = 4 * t16 .. + 3 of the b-groups q, q + kQ, ...; a b-group is four adjacent b.
      const int32_t sb = (int32_t)P.stride[k][1];
      const float* p = P.ptr[k] + (int64_t)(a0 + 4 * t16) + (int64_t)(b0 + 4 * q) * (int64_t)sb;
      float* slot = smem + TP.tslot[k] * kTile * kTile;
      constexpr int G = 16 / kQ;  // b-groups per thread
      float4 v[G][4];
#pragma unroll
      for (int u = 0; u < G; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) v[u][j] = __ldg(reinterpret_cast<const float4*>(p + (4 * kQ * u + j) * sb));
#pragma unroll
      for (int u = 0; u < G; ++u) {
        const int bl = 4 * (q + kQ * u), al = 4 * t16;
        const int c = swz(al, bl);  // the swizzle term is the same for al .. al + 3
        *reinterpret_cast<float4*>(slot + (al + 0) * kTile + c) = make_float4(v[u][0].x, v[u][1].x, v[u][2].x, v[u][3].x);
        *reinterpret_cast<float4*>(slot + (al + 1) * kTile + c) = make_float4(v[u][0].y, v[u][1].y, v[u][2].y, v[u][3].y);
        *reinterpret_cast<float4*>(slot + (al + 2) * kTile + c) = make_float4(v[u][0].z, v[u][1].z, v[u][2].z, v[u][3].z);
        *reinterpret_cast<float4*>(slot + (al + 3) * kTile + c) = make_float4(v[u][0].w, v[u][1].w, v[u][2].w, v[u][3].w);
      }
    }
    __syncthreads();
    const int bl = 4 * t16;
    auto fetch = [&](int k, float (&dst)[kN]) {
      // `k` is a compile-time constant at every call site of a compiled program; the chain below folds.
#pragma unroll
      for (int kk = 0; kk < kMaxOps; ++kk) {
        if (kk != k) continue;
        if (mode(kk) == kOpStaged) {
          const float* slot = smem + TP.tslot[kk] * kTile * kTile;
#pragma unroll
          for (int m = 0; m < RPT; ++m) {
            const int al = q + kQ * m;
            const float4 t = *reinterpret_cast<const float4*>(slot + al * kTile + swz(al, bl));
            dst[m * 4 + 0] = t.x; dst[m * 4 + 1] = t.y; dst[m * 4 + 2] = t.z; dst[m * 4 + 3] = t.w;
          }
        } else if (mode(kk) == kOpBcastB) {
          const int32_t sa = (int32_t)P.stride[kk][0];
          const float* p = P.ptr[kk] + (int64_t)(a0 + q) * (int64_t)sa;
#pragma unroll
          for (int m = 0; m < RPT; ++m) {
            const float s = __ldg(p + (kQ * m) * sa);
            dst[m * 4 + 0] = s; dst[m * 4 + 1] = s; dst[m * 4 + 2] = s; dst[m * 4 + 3] = s;
          }
        } else {
          const int32_t sa = (int32_t)P.stride[kk][0];
          const float* p = P.ptr[kk] + (int64_t)(a0 + q) * (int64_t)sa + (int64_t)(b0 + bl);
#pragma unroll
          for (int m = 0; m < RPT; ++m) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(p + (kQ * m) * sa));
            dst[m * 4 + 0] = t.x; dst[m * 4 + 1] = t.y; dst[m * 4 + 2] = t.z; dst[m * 4 + 3] = t.w;
          }
        }
      }
    };
    float V[kN];
    Runner::template run<kN>(P, fetch, V);
    const uint32_t os = (uint32_t)TP.ostride[0];
    float* po = out + (uint64_t)(a0 + q) * os + b0 + bl;
#pragma unroll
    for (int m = 0; m < RPT; ++m)
      st_stream4(po + (uint32_t)(kQ * m) * os, make_float4(V[m * 4], V[m * 4 + 1], V[m * 4 + 2], V[m * 4 + 3]));
  }
};

// Work items per batch: first the unordered off-diagonal pairs {i, j} of the
// square part of the tile grid (each item does tile (i, j) and then its mirror
// (j, i)), then the diagonal tiles, then the tiles outside the square.
template <class Tile, class Runner>
__global__ void __launch_bounds__(Tile::kThreads, Tile::kMinCtas ? Tile::kMinCtas : Runner::kTileCtasPerSm)
chain_tile_kernel(const __grid_constant__ TileParams TP, float* __restrict__ out) {
  const ChainParams& P = TP.c;
  __shared__ __align__(16) float sm[Tile::kSmemFloats];
  const int last = P.rank - 1, da = TP.dim_a;
  const uint32_t sq = TP.tiles_a < TP.tiles_b ? TP.tiles_a : TP.tiles_b;
  const uint64_t npairs = (uint64_t)sq * (sq - 1) / 2;
  const uint64_t rest = (uint64_t)TP.tiles_a * TP.tiles_b - (uint64_t)sq * sq;
  const uint64_t per_batch = npairs + sq + rest;
  const uint64_t total = per_batch * TP.batches;
  for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const uint64_t batch = TP.batches == 1 ? 0 : t / per_batch;
    const uint64_t w = t - batch * per_batch;
    int64_t boff[kMaxOps];
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) boff[k] = 0;
    uint64_t obatch = 0, rem = batch;
    for (int d = last - 1; d >= 0; --d) {
      if (d == da) continue;
      const uint64_t q = rem / P.shape[d], c = rem - q * P.shape[d];
      rem = q;
#pragma unroll
      for (int k = 0; k < kMaxOps; ++k)
        if (k < P.n_ops) boff[k] += (int64_t)c * P.stride[k][d];
      obatch += c * TP.ostride[d];
    }
    // The tile(s) of this work item; one call site for the tile body, so that its code (the whole
    // program unrolled over a thread's elements) exists once in the kernel.
    uint32_t ta[2], tb[2];
    int ntiles = 1;
    if (w < npairs) {
      // Triangular decode: w = j*(j-1)/2 + i with 0 <= i < j < sq.  sq < 2^16
      // (2^22 elements per side) keeps everything in 32 bits; the float guess
      // is off by at most one, which the two loops repair.
      uint32_t i, j;
      if (sq < 65536u) {
        const uint32_t w32 = (uint32_t)w;
        j = (uint32_t)((1.0f + sqrt_approx(1.0f + 8.0f * (float)w32)) * 0.5f);
        while (j > 1 && j * (j - 1) / 2 > w32) --j;
        while ((j + 1) * j / 2 <= w32) ++j;
        i = w32 - j * (j - 1) / 2;
      } else {
        j = (uint32_t)((1.0 + sqrt(1.0 + 8.0 * (double)w)) * 0.5);
        while (j > 1 && (uint64_t)j * (j - 1) / 2 > w) --j;
        while ((uint64_t)(j + 1) * j / 2 <= w) ++j;
        i = (uint32_t)(w - (uint64_t)j * (j - 1) / 2);
      }
      ta[0] = i; tb[0] = j;  // tile (i, j), then its mirror (j, i)
      ta[1] = j; tb[1] = i;
      ntiles = 2;
    } else if (w < npairs + sq) {
      ta[0] = tb[0] = (uint32_t)(w - npairs);
    } else {
      const uint64_t r = w - npairs - sq;
      if (TP.tiles_a > sq) {
        ta[0] = sq + (uint32_t)(r / TP.tiles_b);
        tb[0] = (uint32_t)(r % TP.tiles_b);
      } else {
        ta[0] = (uint32_t)(r / (TP.tiles_b - sq));
        tb[0] = sq + (uint32_t)(r % (TP.tiles_b - sq));
      }
    }
#pragma unroll 1
    for (int rep = 0; rep < ntiles; ++rep)
      Tile::template run<Runner>(TP, sm, boff, obatch, rep ? ta[1] : ta[0], rep ? tb[1] : tb[0], out);
  }
}

// ------------------------------------------------- compiled program catalogue
// chain_static.cu.  Returns true when the program in P matches a catalogue
// entry and the matching kernel has been launched.
enum StaticTarget { kStaticSeg44 = 0, kStaticVectorTile = 1 };
// The interpreted kernels live in translation units of their own (chain_interp_tile.cu,
// chain_interp_seg.cu): each instantiation unrolls every kind for 16 elements, and
// compiling them side by side is what keeps the build short.
void launch_interp_tile(cudaStream_t stream, const TileParams& TP, unsigned grid, bool vector, float* out);
void launch_interp_seg(cudaStream_t stream, const ChainParams& P, uint64_t nseg, unsigned grid, bool vec, int unroll,
                       float* out);
bool launch_static_seg(cudaStream_t stream, const ChainParams& P, uint64_t nseg, unsigned grid, float* out);
bool launch_static_vtile(cudaStream_t stream, const TileParams& TP, unsigned grid, float* out);
bool launch_static_ftile(cudaStream_t stream, const TileParams& TP, unsigned grid, float* out);

}  // namespace fb
