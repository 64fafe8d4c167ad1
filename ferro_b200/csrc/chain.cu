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
//   - the segment kernel (long innermost dim): a CTA owns one outer index and
//     a run of the innermost dim, decodes the outer coordinates once per run,
//     and every thread evaluates the program on 16 elements at a time (four
//     float4 accesses per operand in flight), so neither index arithmetic nor
//     the interpreter's dispatch is paid per element;
//   - the tile kernel when an operand is unit-stride along ANOTHER dim (a
//     transposed view): 64x64 tiles staged through shared memory so both the
//     transposed read and the row-major write are coalesced.  Tiles (I, J)
//     and (J, I) are done back to back by the same CTA, so when the same
//     storage is read both straight and transposed (f(a, a^T)) the second
//     touch of each tile is an L2 hit and `a` crosses HBM once;
//   - the flat kernel (short innermost dim, unaligned or irregular strides):
//     one work item per thread with multiply-high index decoding.
// The reference decodes coordinates with one u32 div/mod pair per dim per
// element and cannot read non-contiguous views at all
// (crates/ferro-cuda/src/kernels.rs:114-142; crates/ferro-core/src/tensor.rs:1692-1700).
#include <atomic>
#include <cstdlib>

#include "chain.cuh"

namespace fb {

// Process-wide switch read by the launchers: when off, every chain runs on the
// interpreter even if the catalogue holds a compiled form (fb_chain_catalogue).
static std::atomic<int> g_catalogue_on{1};
static inline bool catalogue_on() { return g_catalogue_on.load(std::memory_order_relaxed) != 0; }
// FB_CHAIN_FULL=0 in the environment keeps compiled tile programs on the general vector tile
// (for A/B measurements of the interior form).
static bool full_tile_enabled() {
  static const int on = [] {
    const char* e = getenv("FB_CHAIN_FULL");
    return (e && e[0] == '0') ? 0 : 1;
  }();
  return on != 0;
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
        o.kind = (int8_t)resolve_unary_kind(st.kind, st.p0, st.p1);
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
  const uint64_t inner = cs[last];
  // Transposed operands: not unit/zero stride innermost, but unit stride along one other dim.
  uint32_t tmask = 0;
  int dim_a = -1, nt = 0;
  bool gather = false;
  for (int k = 0; k < n_ops; ++k) {
    const int64_t si = cst[k][last];
    if (si == 0 || si == 1) continue;
    int unit = -1;
    for (int d = 0; d < last; ++d)
      if (cst[k][d] == 1) unit = d;
    if (unit >= 0 && (dim_a < 0 || dim_a == unit) && nt < kTileSlots) {
      dim_a = unit;
      tmask |= 1u << k;
      ++nt;
    } else {
      gather = true;
    }
  }
  if (tmask && !gather && inner >= 16 && cs[dim_a] >= 16) {
    TileParams TP{};
    TP.c = P;
    TP.tmask = tmask;
    TP.dim_a = dim_a;
    int slot = 0;
    for (int k = 0; k < n_ops; ++k) {
      TP.tslot[k] = ((tmask >> k) & 1) ? slot++ : 0;
      const uint32_t md = ((tmask >> k) & 1) ? kOpStaged : (cst[k][last] == 0 ? kOpBcastB : kOpDirect);
      TP.modes |= md << (2 * k);
    }
    TP.tiles_a = (uint32_t)((cs[dim_a] + kTile - 1) / kTile);
    TP.tiles_b = (uint32_t)((inner + kTile - 1) / kTile);
    TP.batches = n / (cs[dim_a] * inner);
    uint64_t ostr = 1;
    for (int d = cr - 1; d >= 0; --d) {
      TP.ostride[d] = ostr;
      ostr *= cs[d];
    }
    const uint64_t sqt = TP.tiles_a < TP.tiles_b ? TP.tiles_a : TP.tiles_b;
    const uint64_t total = ((uint64_t)TP.tiles_a * TP.tiles_b - sqt * (sqt - 1) / 2) * TP.batches;
    const unsigned grid = grid_full(total);
    // Vector form: every access a float4.  Extents along A and B multiples of 4,
    // bases 16-byte aligned, every stride that is not the unit one a multiple of 4,
    // straight operands unit-stride or broadcast along B.
    bool vt = aligned16(out) && inner % 4 == 0 && cs[dim_a] % 4 == 0;
    for (int k = 0; k < n_ops && vt; ++k) {
      const bool staged = (tmask >> k) & 1;
      if ((staged || cst[k][last] == 1) && !aligned16(P.ptr[k])) vt = false;
      for (int d = 0; d < cr; ++d) {
        const int64_t st = cst[k][d];
        // A straight operand that is broadcast along B is read with scalar loads: no constraint.
        if (staged ? (d != dim_a && st % 4 != 0) : (cst[k][last] == 1 && d != last && st % 4 != 0)) vt = false;
      }
      if (!staged && cst[k][last] != 0 && cst[k][last] != 1) vt = false;
    }
    if (vt) {
      // The interior form of a compiled program: one batch, extents multiples of the tile, offsets
      // inside a tile within 32 bits.
      bool full = full_tile_enabled() && cr == 2 && dim_a == 0 && cs[0] % kTile == 0 && cs[1] % kTile == 0 && cs[0] <= (1u << 24) &&
                  cs[1] <= (1u << 24);
      for (int k = 0; k < n_ops && full; ++k)
        for (int d = 0; d < 2; ++d)
          if (cst[k][d] < 0 || cst[k][d] > (1 << 24)) full = false;
      if (!(catalogue_on() && ((full && launch_static_ftile(stream, TP, grid, out)) ||
                               launch_static_vtile(stream, TP, grid, out))))
        launch_interp_tile(stream, TP, grid, true, out);
    } else {
      launch_interp_tile(stream, TP, grid, false, out);
    }
    FB_LAUNCHED(name);
    return FB_OK;
  }

  bool vec = aligned16(out) && inner % 4 == 0;
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

  // Long rows: segment kernel.  A run covers 256 * V * U elements.
  if (inner >= (uint64_t)kChThreads * V) {
    const int U = inner >= (uint64_t)kChThreads * V * 3 ? 4 : 1;
    const uint64_t run = (uint64_t)kChThreads * V * U;
    const uint64_t nseg = (inner + run - 1) / run;
    const uint64_t items = (n / inner) * nseg;
    const unsigned grid = grid_full(items);
    if (!(vec && U == 4 && catalogue_on() && launch_static_seg(stream, P, nseg, grid, out)))
      launch_interp_seg(stream, P, nseg, grid, vec, U, out);
    FB_LAUNCHED(name);
    return FB_OK;
  }

  const uint64_t items = n / V;
  const bool wide = items >= (1ull << 31);
  if (!wide)
    for (int d = 0; d < cr; ++d) {
      const uint64_t ext = d == last ? cs[d] / V : cs[d];
      P.div[d] = make_fastdiv((uint32_t)ext);
    }
  const unsigned grid = grid_full((items + kChThreads - 1) / kChThreads);
  if (vec) {
    if (wide) chain_flat_kernel<4, true><<<grid, kChThreads, 0, stream>>>(P, out);
    else chain_flat_kernel<4, false><<<grid, kChThreads, 0, stream>>>(P, out);
  } else {
    if (wide) chain_flat_kernel<1, true><<<grid, kChThreads, 0, stream>>>(P, out);
    else chain_flat_kernel<1, false><<<grid, kChThreads, 0, stream>>>(P, out);
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

int fb_chain_catalogue(int enable) { return g_catalogue_on.exchange(enable ? 1 : 0, std::memory_order_relaxed); }

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

int fb_bias_act_fwd(fb_stream_t stream, const float* x, const float* bias, int act, uint64_t rows,
                    uint64_t cols, float* out) {
  const char* name = "fb_bias_act_fwd";
  if (act < 0 || act > 3) return fail(FB_ERR_INVALID_ARG, "%s: unknown activation %d", name, act);
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
  static const int kind_of[4] = {0, FB_UN_RELU, FB_UN_GELU, FB_UN_SILU};
  if (act) prog[ns++] = {FB_CH_UNARY, FB_CH_V, kind_of[act], 0, 0.0f, 0.0f};
  return run_chain(stream, name, prog, ns, v, bias ? 2 : 1, shape, 2, out);
}

}  // extern "C"
