// The strided pointwise engine: one kernel family evaluates a small program
// per output element over up to six operands addressed as ferro views
// (pointer, element offset, element strides, stride 0 = broadcast).  It backs
// fb_chain and, with one- or two-step programs, fb_binary_bc,
// fb_unary_strided, fb_binary_strided, fb_materialize and fb_bias_act_fwd.
//
// Roofline: HBM.  Algorithmic bytes: 4 bytes per output element written plus
// 4 bytes per distinct operand element read (a broadcast operand counts once;
// the same storage reached through two views counts once).
//
// Host side: validate, bounds-check every view, drop size-1 dims and merge
// dims that are contiguous for every operand, then pick
//   - the row kernel (lanes along the innermost dim; float4 when every
//     operand is unit-stride or broadcast there and 16-byte aligned), or
//   - the tile kernel when an operand is unit-stride along ANOTHER dim (a
//     transposed view): 32x32 tiles staged through shared memory so both the
//     transposed read and the row-major write are coalesced.  Tiles (I, J)
//     and (J, I) are scheduled back to back in the same CTA, so when the same
//     storage is read both straight and transposed (f(a, a^T)) the second
//     touch of each tile is an L2 hit and `a` crosses HBM once.
// The reference decodes coordinates with one u32 div/mod pair per dim per
// element and cannot read non-contiguous views at all
// (crates/ferro-cuda/src/kernels.rs:114-142; crates/ferro-core/src/tensor.rs:1692-1700).
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
static FastDiv make_fastdiv(uint32_t d) {
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
  int8_t opcode, dst, kind, swap;
  int16_t src;  // LOAD: operand; BINARY: 0 other reg, 1 immediate, 8+k operand k
  float p0, p1;
};

struct ChainParams {
  int n_steps, n_ops, rank;
  uint64_t n;                    // output elements
  uint64_t shape[FB_MAX_RANK];   // collapsed, outermost first
  FastDiv div[FB_MAX_RANK];      // divisors for the narrow path (innermost is in vec units)
  const float* ptr[kMaxOps];     // already advanced by the view offset
  int64_t stride[kMaxOps][FB_MAX_RANK];
  Step steps[kMaxSteps];
};

template <int VEC>
__device__ __forceinline__ void unary_vec(int kind, float p0, float p1, float (&x)[VEC]) {
#define FB_CASE(K)                                                   \
  case K:                                                            \
    _Pragma("unroll") for (int j = 0; j < VEC; ++j) x[j] = unary_apply(K, p0, p1, x[j]); \
    break;
  switch (kind) {
    FB_CASE(FB_UN_NEG) FB_CASE(FB_UN_RELU) FB_CASE(FB_UN_EXP) FB_CASE(FB_UN_SIGMOID)
    FB_CASE(FB_UN_TANH) FB_CASE(FB_UN_SQRT) FB_CASE(FB_UN_ABS) FB_CASE(FB_UN_SIGN)
    FB_CASE(FB_UN_LOG) FB_CASE(FB_UN_POWF) FB_CASE(FB_UN_CLAMP) FB_CASE(FB_UN_GTZ)
    FB_CASE(FB_UN_GELU) FB_CASE(FB_UN_GELU_ERF) FB_CASE(FB_UN_GELU_ERF_GRAD) FB_CASE(FB_UN_SILU)
    default: break;
  }
#undef FB_CASE
}

template <int VEC>
__device__ __forceinline__ void binary_vec(int kind, float p0, float p1, const float (&a)[VEC],
                                           const float (&b)[VEC], float (&r)[VEC]) {
#define FB_CASE(K)                                                   \
  case K:                                                            \
    _Pragma("unroll") for (int j = 0; j < VEC; ++j) r[j] = binary_apply(K, p0, p1, a[j], b[j]); \
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

// Runs the program for VEC adjacent output elements.  `fetch(k, dst)` loads
// operand k for those elements.
template <int VEC, class Fetch>
__device__ __forceinline__ void run_program(const ChainParams& P, Fetch&& fetch, float (&V)[VEC]) {
  float T[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) V[j] = T[j] = 0.0f;
  for (int s = 0; s < P.n_steps; ++s) {
    const Step st = P.steps[s];
    const bool onT = st.dst != 0;
    float cur[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) cur[j] = onT ? T[j] : V[j];
    switch (st.opcode) {
      case FB_CH_LOAD: fetch(st.src, cur); break;
      case FB_CH_IMM:
#pragma unroll
        for (int j = 0; j < VEC; ++j) cur[j] = st.p0;
        break;
      case FB_CH_UNARY: unary_vec<VEC>(st.kind, st.p0, st.p1, cur); break;
      case FB_CH_BINARY: {
        float other[VEC];
        if (st.src == FB_CH_SRC_OTHER_REG) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) other[j] = onT ? V[j] : T[j];
        } else if (st.src == FB_CH_SRC_IMM) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) other[j] = st.p1;
        } else {
          fetch(st.src - FB_CH_SRC_OPERAND0, other);
        }
        float r[VEC];
        if (st.swap) binary_vec<VEC>(st.kind, st.p0, st.p1, other, cur, r);
        else binary_vec<VEC>(st.kind, st.p0, st.p1, cur, other, r);
#pragma unroll
        for (int j = 0; j < VEC; ++j) cur[j] = r[j];
        break;
      }
      default: break;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      if (onT) T[j] = cur[j];
      else V[j] = cur[j];
    }
  }
}

// Row kernel.  VEC = 4: every operand has innermost stride 0 or 1 and float4
// alignment.  VEC = 1: arbitrary strides (plain gathers).  WIDE = false:
// fewer than 2^31 work items, 32-bit index math with multiply-high division.
template <int VEC, bool WIDE>
__global__ void __launch_bounds__(kChThreads)
chain_row_kernel(const __grid_constant__ ChainParams P, float* __restrict__ out) {
  const uint64_t items = P.n / VEC;
  const uint64_t stride = (uint64_t)gridDim.x * kChThreads;
  for (uint64_t it = (uint64_t)blockIdx.x * kChThreads + threadIdx.x; it < items; it += stride) {
    int64_t off[kMaxOps];
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) off[k] = 0;
    if constexpr (WIDE) {
      uint64_t rem = it;
      for (int d = P.rank - 1; d >= 0; --d) {
        const uint64_t ext = d == P.rank - 1 ? P.shape[d] / VEC : P.shape[d];
        const uint64_t q = rem / ext, c = rem - q * ext;
        rem = q;
        const int64_t cc = (int64_t)(d == P.rank - 1 ? c * VEC : c);
#pragma unroll
        for (int k = 0; k < kMaxOps; ++k)
          if (k < P.n_ops) off[k] += cc * P.stride[k][d];
      }
    } else {
      uint32_t rem = (uint32_t)it;
      for (int d = P.rank - 1; d >= 0; --d) {
        const uint32_t q = fdiv(rem, P.div[d]), c = rem - q * P.div[d].d;
        rem = q;
        const int64_t cc = (int64_t)(d == P.rank - 1 ? (uint64_t)c * VEC : (uint64_t)c);
#pragma unroll
        for (int k = 0; k < kMaxOps; ++k)
          if (k < P.n_ops) off[k] += cc * P.stride[k][d];
      }
    }
    const int last = P.rank - 1;
    auto fetch = [&](int k, float (&dst)[VEC]) {
      // k is warp-uniform; select the offset without indexing registers dynamically.
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
    run_program<VEC>(P, fetch, V);
    if constexpr (VEC == 4) st_stream4(out + it * 4, make_float4(V[0], V[1], V[2], V[3]));
    else out[it] = V[0];
  }
}

// Tile kernel: output viewed as [batch..., A, ..., B] with B innermost;
// operands flagged in `tmask` are unit-stride along A (transposed) and are
// staged through shared memory; the others are read directly with lanes
// along B.  Collapsed rank is >= 2; the dims other than A and B form the batch.
struct TileParams {
  ChainParams c;
  uint32_t tmask;  // bit k: operand k is read transposed
  uint32_t tiles_a, tiles_b;
  uint64_t batches;
  int dim_a;             // which collapsed dim plays A
  uint64_t ostride_a;    // output stride of dim A
  uint64_t obatch_stride[FB_MAX_RANK];  // output stride of each dim
};

constexpr int kTile = 32;

// One 32x32 tile: stage the transposed operands, then run the program with
// lanes along B.
__device__ __forceinline__ void chain_tile(const TileParams& TP, float (&sm)[kMaxOps][kTile][kTile + 1],
                                           const int64_t (&boff)[kMaxOps], uint64_t obatch,
                                           uint32_t ia, uint32_t ib, float* __restrict__ out) {
  const ChainParams& P = TP.c;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int last = P.rank - 1, da = TP.dim_a;
  const uint64_t A = P.shape[da], B = P.shape[last];
  const uint64_t a0 = (uint64_t)ia * kTile, b0 = (uint64_t)ib * kTile;
  __syncthreads();  // the previous tile's readers are done with sm
  for (int k = 0; k < P.n_ops; ++k) {
    if (!((TP.tmask >> k) & 1)) continue;
    int64_t o = 0;
#pragma unroll
    for (int q = 0; q < kMaxOps; ++q)
      if (q == k) o = boff[q];
#pragma unroll
    for (int j = ty; j < kTile; j += 8) {
      const uint64_t a = a0 + tx, b = b0 + j;
      float v = 0.0f;
      if (a < A && b < B)
        v = __ldg(P.ptr[k] + o + (int64_t)a * P.stride[k][da] + (int64_t)b * P.stride[k][last]);
      sm[k][j][tx] = v;  // [b_local][a_local]
    }
  }
  __syncthreads();
#pragma unroll 1
  for (int j = ty; j < kTile; j += 8) {
    const uint64_t a = a0 + j, b = b0 + tx;
    if (a < A && b < B) {
      auto fetch = [&](int k, float (&dst)[1]) {
        if ((TP.tmask >> k) & 1) {
          dst[0] = sm[k][tx][j];
        } else {
          int64_t o = 0;
#pragma unroll
          for (int q = 0; q < kMaxOps; ++q)
            if (q == k) o = boff[q];
          dst[0] = __ldg(P.ptr[k] + o + (int64_t)a * P.stride[k][da] + (int64_t)b * P.stride[k][last]);
        }
      };
      float V[1];
      run_program<1>(P, fetch, V);
      st_stream(out + obatch + a * TP.ostride_a + b, V[0]);
    }
  }
}

// Work items per batch: first the unordered off-diagonal pairs {i, j} of the
// square part of the tile grid (each item does tile (i, j) then its mirror
// (j, i), so storage read both straight and transposed is fetched from HBM
// once and found in L2 the second time), then the diagonal tiles, then the
// tiles outside the square.
__global__ void __launch_bounds__(kChThreads)
chain_tile_kernel(const __grid_constant__ TileParams TP, float* __restrict__ out) {
  const ChainParams& P = TP.c;
  __shared__ float sm[kMaxOps][kTile][kTile + 1];
  const int last = P.rank - 1, da = TP.dim_a;
  const uint32_t sq = TP.tiles_a < TP.tiles_b ? TP.tiles_a : TP.tiles_b;
  const uint64_t npairs = (uint64_t)sq * (sq - 1) / 2;
  const uint64_t rest = (uint64_t)TP.tiles_a * TP.tiles_b - (uint64_t)sq * sq;
  const uint64_t per_batch = npairs + sq + rest;
  const uint64_t total = per_batch * TP.batches;
  for (uint64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const uint64_t batch = t / per_batch;
    const uint64_t w = t - batch * per_batch;
    int64_t boff[kMaxOps];
#pragma unroll
    for (int k = 0; k < kMaxOps; ++k) boff[k] = 0;
    uint64_t obatch = 0;
    uint64_t rem = batch;
    for (int d = last - 1; d >= 0; --d) {
      if (d == da) continue;
      const uint64_t q = rem / P.shape[d], c = rem - q * P.shape[d];
      rem = q;
#pragma unroll
      for (int k = 0; k < kMaxOps; ++k)
        if (k < P.n_ops) boff[k] += (int64_t)c * P.stride[k][d];
      obatch += c * TP.obatch_stride[d];
    }
    if (w < npairs) {
      // Triangular decode: w = j*(j-1)/2 + i with 0 <= i < j < sq.
      uint32_t j = (uint32_t)((1.0 + sqrt(1.0 + 8.0 * (double)w)) * 0.5);
      while ((uint64_t)j * (j - 1) / 2 > w) --j;
      while ((uint64_t)(j + 1) * j / 2 <= w) ++j;
      const uint32_t i = (uint32_t)(w - (uint64_t)j * (j - 1) / 2);
      chain_tile(TP, sm, boff, obatch, i, j, out);
      chain_tile(TP, sm, boff, obatch, j, i, out);
    } else if (w < npairs + sq) {
      const uint32_t d = (uint32_t)(w - npairs);
      chain_tile(TP, sm, boff, obatch, d, d, out);
    } else {
      const uint64_t r = w - npairs - sq;
      uint32_t ia, ib;
      if (TP.tiles_a > sq) {
        ia = sq + (uint32_t)(r / TP.tiles_b);
        ib = (uint32_t)(r % TP.tiles_b);
      } else {
        ia = (uint32_t)(r / (TP.tiles_b - sq));
        ib = sq + (uint32_t)(r % (TP.tiles_b - sq));
      }
      chain_tile(TP, sm, boff, obatch, ia, ib, out);
    }
  }
}

// ---------------------------------------------------------------- host side
struct View {
  const float* ptr;
  uint64_t len;
  int64_t offset;
  int64_t strides[FB_MAX_RANK];
};

static int validate_view(const char* name, int k, const View& v, const uint64_t* shape, int rank) {
  if (!v.ptr) return fail(FB_ERR_INVALID_ARG, "%s: operand %d is null", name, k);
  // Lowest and highest element index the view can touch (every dim non-empty here).
  __int128 lo = v.offset, hi = v.offset;
  for (int d = 0; d < rank; ++d) {
    const __int128 span = (__int128)(shape[d] - 1) * v.strides[d];
    if (span >= 0) hi += span;
    else lo += span;
  }
  if (lo < 0 || hi >= (__int128)v.len)
    return fail(FB_ERR_INVALID_SHAPE, "%s: operand %d view reaches outside its storage of %llu elements",
                name, k, (unsigned long long)v.len);
  return FB_OK;
}

static int run_chain(cudaStream_t stream, const char* name, const fb_chain_step* steps, int n_steps,
                     const View* ops, int n_ops, const uint64_t* shape, int rank, float* out) {
  if (rank < 0 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 0..%d", name, rank, FB_MAX_RANK);
  if (n_steps < 1 || n_steps > kMaxSteps) return fail(FB_ERR_INVALID_ARG, "%s: %d steps not in 1..%d", name, n_steps, kMaxSteps);
  if (n_ops < 0 || n_ops > kMaxOps) return fail(FB_ERR_INVALID_ARG, "%s: %d operands not in 0..%d", name, n_ops, kMaxOps);
  if (!steps || (n_ops && !ops) || (rank && !shape)) return fail(FB_ERR_INVALID_ARG, "%s: null argument", name);
  uint64_t n = 1;
  for (int d = 0; d < rank; ++d)
    if (mul_overflows(n, shape[d], &n) || n > (UINT64_MAX >> 3))
      return fail(FB_ERR_INVALID_SHAPE, "%s: shape overflows", name);
  // Program checks: registers are written before they are read.
  bool def[2] = {false, false};
  ChainParams P{};
  for (int s = 0; s < n_steps; ++s) {
    const fb_chain_step& st = steps[s];
    if (st.dst != FB_CH_V && st.dst != FB_CH_T) return fail(FB_ERR_INVALID_ARG, "%s: step %d: bad register", name, s);
    Step o{};
    o.opcode = (int8_t)st.opcode;
    o.dst = (int8_t)st.dst;
    o.kind = (int8_t)st.kind;
    o.p0 = st.p0;
    o.p1 = st.p1;
    switch (st.opcode) {
      case FB_CH_LOAD:
        if (st.src < 0 || st.src >= n_ops) return fail(FB_ERR_INVALID_ARG, "%s: step %d: operand %d out of range", name, s, st.src);
        o.src = (int16_t)st.src;
        break;
      case FB_CH_IMM: break;
      case FB_CH_UNARY:
        if (st.kind < 0 || st.kind >= FB_UN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "%s: step %d: unknown unary kind %d", name, s, st.kind);
        if (!def[st.dst]) return fail(FB_ERR_INVALID_ARG, "%s: step %d reads a register before it is written", name, s);
        break;
      case FB_CH_BINARY: {
        if (st.kind < 0 || st.kind >= FB_BIN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "%s: step %d: unknown binary kind %d", name, s, st.kind);
        if (!def[st.dst]) return fail(FB_ERR_INVALID_ARG, "%s: step %d reads a register before it is written", name, s);
        const int src = st.src & ~FB_CH_SWAP;
        o.swap = (st.src & FB_CH_SWAP) ? 1 : 0;
        if (src == FB_CH_SRC_OTHER_REG) {
          if (!def[1 - st.dst]) return fail(FB_ERR_INVALID_ARG, "%s: step %d reads a register before it is written", name, s);
        } else if (src == FB_CH_SRC_IMM) {
          if (st.kind == FB_BIN_CLAMP_BWD) return fail(FB_ERR_INVALID_ARG, "%s: step %d: kind needs p1, cannot take an immediate", name, s);
        } else if (src < FB_CH_SRC_OPERAND0 || src >= FB_CH_SRC_OPERAND0 + n_ops) {
          return fail(FB_ERR_INVALID_ARG, "%s: step %d: bad source %d", name, s, st.src);
        }
        o.src = (int16_t)src;
        break;
      }
      default: return fail(FB_ERR_INVALID_ARG, "%s: step %d: unknown opcode %d", name, s, st.opcode);
    }
    def[st.dst] = true;
    P.steps[s] = o;
  }
  if (!def[FB_CH_V]) return fail(FB_ERR_INVALID_ARG, "%s: the program never writes V", name);
  if (n == 0) return FB_OK;
  if (!out) return fail(FB_ERR_INVALID_ARG, "%s: null output", name);
  for (int k = 0; k < n_ops; ++k)
    if (int rc = validate_view(name, k, ops[k], shape, rank)) return rc;

  // Collapse: drop size-1 dims, merge dims contiguous for every operand.
  uint64_t cs[FB_MAX_RANK];
  int64_t cst[kMaxOps][FB_MAX_RANK];
  int cr = 0;
  for (int d = 0; d < rank; ++d) {
    if (shape[d] == 1) continue;
    bool merge = cr > 0;
    if (merge)
      for (int k = 0; k < n_ops; ++k)
        if (cst[k][cr - 1] != (int64_t)shape[d] * ops[k].strides[d]) { merge = false; break; }
    if (merge) {
      cs[cr - 1] *= shape[d];
      for (int k = 0; k < n_ops; ++k) cst[k][cr - 1] = ops[k].strides[d];
    } else {
      cs[cr] = shape[d];
      for (int k = 0; k < n_ops; ++k) cst[k][cr] = ops[k].strides[d];
      ++cr;
    }
  }
  if (cr == 0) {  // a single element
    cs[0] = 1;
    for (int k = 0; k < n_ops; ++k) cst[k][0] = 0;
    cr = 1;
  }
  P.n_steps = n_steps;
  P.n_ops = n_ops;
  P.rank = cr;
  P.n = n;
  for (int d = 0; d < cr; ++d) {
    P.shape[d] = cs[d];
    for (int k = 0; k < n_ops; ++k) P.stride[k][d] = cst[k][d];
  }
  for (int k = 0; k < n_ops; ++k) P.ptr[k] = ops[k].ptr + ops[k].offset;

  const int last = cr - 1;
  // Transposed operands: not unit/zero stride innermost, but unit stride along one other dim.
  uint32_t tmask = 0;
  int dim_a = -1;
  bool gather = false;
  for (int k = 0; k < n_ops; ++k) {
    const int64_t si = cst[k][last];
    if (si == 0 || si == 1) continue;
    int unit = -1;
    for (int d = 0; d < last; ++d)
      if (cst[k][d] == 1) unit = d;
    if (unit >= 0 && (dim_a < 0 || dim_a == unit)) {
      dim_a = unit;
      tmask |= 1u << k;
    } else {
      gather = true;
    }
  }
  if (tmask && !gather && cs[last] >= 8 && cs[dim_a] >= 8) {
    TileParams TP{};
    TP.c = P;
    TP.tmask = tmask;
    TP.dim_a = dim_a;
    TP.tiles_a = (uint32_t)((cs[dim_a] + kTile - 1) / kTile);
    TP.tiles_b = (uint32_t)((cs[last] + kTile - 1) / kTile);
    TP.batches = n / (cs[dim_a] * cs[last]);
    uint64_t ostr = 1;
    for (int d = cr - 1; d >= 0; --d) {
      TP.obatch_stride[d] = ostr;
      ostr *= cs[d];
    }
    TP.ostride_a = TP.obatch_stride[dim_a];
    const uint64_t sqt = TP.tiles_a < TP.tiles_b ? TP.tiles_a : TP.tiles_b;
    const uint64_t total = ((uint64_t)TP.tiles_a * TP.tiles_b - sqt * (sqt - 1) / 2) * TP.batches;
    chain_tile_kernel<<<grid_for(total, 8), kChThreads, 0, stream>>>(TP, out);
    FB_LAUNCHED(name);
    return FB_OK;
  }

  bool vec = aligned16(out) && cs[last] % 4 == 0;
  for (int k = 0; k < n_ops && vec; ++k) {
    const int64_t si = cst[k][last];
    if (si != 0 && si != 1) vec = false;
    if (si == 1) {
      if (!aligned16(P.ptr[k])) vec = false;
      for (int d = 0; d < last; ++d)
        if (cst[k][d] % 4 != 0) vec = false;
    }
  }
  const int V = vec ? 4 : 1;
  const uint64_t items = n / V;
  const bool wide = items >= (1ull << 31);
  if (!wide)
    for (int d = 0; d < cr; ++d) {
      const uint64_t ext = d == last ? cs[d] / V : cs[d];
      P.div[d] = make_fastdiv((uint32_t)ext);
    }
  const unsigned grid = grid_for((items + kChThreads - 1) / kChThreads, 8);
  if (vec) {
    if (wide) chain_row_kernel<4, true><<<grid, kChThreads, 0, stream>>>(P, out);
    else chain_row_kernel<4, false><<<grid, kChThreads, 0, stream>>>(P, out);
  } else {
    if (wide) chain_row_kernel<1, true><<<grid, kChThreads, 0, stream>>>(P, out);
    else chain_row_kernel<1, false><<<grid, kChThreads, 0, stream>>>(P, out);
  }
  FB_LAUNCHED(name);
  return FB_OK;
}

// Broadcast strides of a contiguous tensor of `shape` read as `out_shape`
// (dispatch.rs:823-835).  Returns false when the shapes do not broadcast.
static bool bc_strides(const uint64_t* shape, int rank, const uint64_t* out_shape, int rank_out,
                       int64_t* strides, uint64_t* len) {
  if (rank > rank_out) return false;
  const int pad = rank_out - rank;
  uint64_t acc = 1;
  int64_t own[FB_MAX_RANK];
  for (int i = rank - 1; i >= 0; --i) {
    own[i] = (int64_t)acc;
    acc *= shape[i];
  }
  *len = acc;
  for (int i = 0; i < rank_out; ++i) {
    if (i < pad) { strides[i] = 0; continue; }
    const uint64_t s = shape[i - pad];
    if (s == out_shape[i]) strides[i] = own[i - pad];
    else if (s == 1) strides[i] = 0;
    else return false;
  }
  return true;
}

static void contiguous_strides(const uint64_t* shape, int rank, int64_t* strides) {
  uint64_t acc = 1;
  for (int i = rank - 1; i >= 0; --i) {
    strides[i] = (int64_t)acc;
    acc *= shape[i];
  }
}

}  // namespace fb

using namespace fb;

extern "C" {

int fb_chain(fb_stream_t stream, const fb_chain_step* steps, int n_steps,
             const fb_chain_operand* operands, int n_operands, const uint64_t* shape, int rank,
             float* out) {
  if (n_operands < 0 || n_operands > kMaxOps) return fail(FB_ERR_INVALID_ARG, "fb_chain: %d operands not in 0..%d", n_operands, kMaxOps);
  if (rank < 0 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "fb_chain: rank %d not in 0..%d", rank, FB_MAX_RANK);
  if (n_operands && !operands) return fail(FB_ERR_INVALID_ARG, "fb_chain: null operand table");
  View v[kMaxOps];
  for (int k = 0; k < n_operands; ++k) {
    v[k].ptr = operands[k].ptr;
    v[k].len = operands[k].len;
    v[k].offset = operands[k].offset;
    for (int d = 0; d < rank; ++d) v[k].strides[d] = operands[k].strides[d];
  }
  return run_chain(stream, "fb_chain", steps, n_steps, v, n_operands, shape, rank, out);
}

int fb_binary_bc(fb_stream_t stream, int kind, float p0, float p1, const float* a, const uint64_t* sa,
                 int rank_a, const float* b, const uint64_t* sb, int rank_b, float* out,
                 const uint64_t* out_shape, int rank_out) {
  const char* name = "fb_binary_bc";
  if (kind < 0 || kind >= FB_BIN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "%s: unknown kind %d", name, kind);
  if (rank_out < 0 || rank_out > FB_MAX_RANK || rank_a < 0 || rank_b < 0)
    return fail(FB_ERR_INVALID_SHAPE, "%s: rank out of range", name);
  View v[2];
  v[0].ptr = a; v[0].offset = 0;
  v[1].ptr = b; v[1].offset = 0;
  if (!bc_strides(sa, rank_a, out_shape, rank_out, v[0].strides, &v[0].len) ||
      !bc_strides(sb, rank_b, out_shape, rank_out, v[1].strides, &v[1].len))
    return fail(FB_ERR_INVALID_SHAPE, "%s: operand shapes do not broadcast to the output shape", name);
  const fb_chain_step prog[2] = {{FB_CH_LOAD, FB_CH_V, 0, 0, 0.0f, 0.0f},
                                 {FB_CH_BINARY, FB_CH_V, kind, FB_CH_SRC_OPERAND0 + 1, p0, p1}};
  return run_chain(stream, name, prog, 2, v, 2, out_shape, rank_out, out);
}

int fb_unary_strided(fb_stream_t stream, int kind, float p0, float p1, const float* x, uint64_t x_len,
                     const int64_t* x_strides, int64_t x_offset, const uint64_t* shape, int rank,
                     float* out) {
  const char* name = "fb_unary_strided";
  if (kind < 0 || kind >= FB_UN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "%s: unknown kind %d", name, kind);
  if (rank < 0 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 0..%d", name, rank, FB_MAX_RANK);
  if (rank && !x_strides) return fail(FB_ERR_INVALID_ARG, "%s: null strides", name);
  View v[1];
  v[0].ptr = x; v[0].len = x_len; v[0].offset = x_offset;
  for (int d = 0; d < rank; ++d) v[0].strides[d] = x_strides[d];
  const fb_chain_step prog[2] = {{FB_CH_LOAD, FB_CH_V, 0, 0, 0.0f, 0.0f}, {FB_CH_UNARY, FB_CH_V, kind, 0, p0, p1}};
  return run_chain(stream, name, prog, 2, v, 1, shape, rank, out);
}

int fb_binary_strided(fb_stream_t stream, int kind, float p0, float p1, const float* a, uint64_t a_len,
                      const int64_t* a_strides, int64_t a_offset, const float* b, uint64_t b_len,
                      const int64_t* b_strides, int64_t b_offset, const uint64_t* shape, int rank,
                      float* out) {
  const char* name = "fb_binary_strided";
  if (kind < 0 || kind >= FB_BIN_KIND_COUNT) return fail(FB_ERR_INVALID_ARG, "%s: unknown kind %d", name, kind);
  if (rank < 0 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 0..%d", name, rank, FB_MAX_RANK);
  if (rank && (!a_strides || !b_strides)) return fail(FB_ERR_INVALID_ARG, "%s: null strides", name);
  View v[2];
  v[0].ptr = a; v[0].len = a_len; v[0].offset = a_offset;
  v[1].ptr = b; v[1].len = b_len; v[1].offset = b_offset;
  for (int d = 0; d < rank; ++d) {
    v[0].strides[d] = a_strides[d];
    v[1].strides[d] = b_strides[d];
  }
  const fb_chain_step prog[2] = {{FB_CH_LOAD, FB_CH_V, 0, 0, 0.0f, 0.0f},
                                 {FB_CH_BINARY, FB_CH_V, kind, FB_CH_SRC_OPERAND0 + 1, p0, p1}};
  return run_chain(stream, name, prog, 2, v, 2, shape, rank, out);
}

int fb_materialize(fb_stream_t stream, const float* x, uint64_t x_len, const int64_t* strides,
                   int64_t offset, const uint64_t* shape, int rank, float* out) {
  const char* name = "fb_materialize";
  if (rank < 0 || rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: rank %d not in 0..%d", name, rank, FB_MAX_RANK);
  if (rank && !strides) return fail(FB_ERR_INVALID_ARG, "%s: null strides", name);
  View v[1];
  v[0].ptr = x; v[0].len = x_len; v[0].offset = offset;
  for (int d = 0; d < rank; ++d) v[0].strides[d] = strides[d];
  const fb_chain_step prog[1] = {{FB_CH_LOAD, FB_CH_V, 0, 0, 0.0f, 0.0f}};
  return run_chain(stream, name, prog, 1, v, 1, shape, rank, out);
}

int fb_bias_act_fwd(fb_stream_t stream, const float* x, const float* bias, int relu, uint64_t rows,
                    uint64_t cols, float* out) {
  const char* name = "fb_bias_act_fwd";
  uint64_t n;
  if (mul_overflows(rows, cols, &n)) return fail(FB_ERR_INVALID_SHAPE, "%s: rows * cols overflows", name);
  if (n == 0) return FB_OK;
  if (!x || !out) return fail(FB_ERR_INVALID_ARG, "%s: null buffer", name);
  const uint64_t shape[2] = {rows, cols};
  View v[2];
  v[0].ptr = x; v[0].len = n; v[0].offset = 0;
  contiguous_strides(shape, 2, v[0].strides);
  v[1].ptr = bias; v[1].len = cols; v[1].offset = 0;
  v[1].strides[0] = 0; v[1].strides[1] = 1;
  fb_chain_step prog[3];
  int ns = 0;
  prog[ns++] = {FB_CH_LOAD, FB_CH_V, 0, 0, 0.0f, 0.0f};
  if (bias) prog[ns++] = {FB_CH_BINARY, FB_CH_V, FB_BIN_ADD, FB_CH_SRC_OPERAND0 + 1, 0.0f, 0.0f};
  if (relu) prog[ns++] = {FB_CH_UNARY, FB_CH_V, FB_UN_RELU, 0, 0.0f, 0.0f};
  return run_chain(stream, name, prog, ns, v, bias ? 2 : 1, shape, 2, out);
}

}  // extern "C"
