// Compiled program catalogue of the strided pointwise engine.
//
// The interpreter of chain.cuh pays a few instructions per element per step
// for dispatch, cannot fold work that is the same for all of a thread's
// elements, and keeps kinds as data.  For chains that matter the same step
// list is also instantiated here as a compile-time program: each step becomes
// straight-line code with its kind a constant, and sub-chains on operands that
// are broadcast along the row collapse to one evaluation per thread.  Scalars
// (p0, p1, immediates) stay run-time values, so one entry serves every scale,
// clamp bound or bias.  A chain that is not in the catalogue still runs, on
// the interpreter.  The catalogue is the manifest chain_programs.def: this
// file turns every line of it into a program type and into the instantiations
// and match tests of the launch functions below.
//
// ferro fuses such chains at run time by generating and compiling CUDA source
// through nvrtc (crates/ferro-cuda/src/kernels.rs:177-235); this library is
// compiled ahead of time, so the fused forms are fixed at build time.
#include "chain.cuh"

namespace fb {

struct SS {
  int opcode, dst, kind, src, swap;
};

constexpr int kV = FB_CH_V, kT = FB_CH_T;
constexpr SS LoadV(int k) { return SS{FB_CH_LOAD, kV, 0, k, 0}; }
constexpr SS LoadT(int k) { return SS{FB_CH_LOAD, kT, 0, k, 0}; }
constexpr SS UnV(int kind) { return SS{FB_CH_UNARY, kV, kind, 0, 0}; }
constexpr SS UnT(int kind) { return SS{FB_CH_UNARY, kT, kind, 0, 0}; }
constexpr SS BinV(int kind, int src) { return SS{FB_CH_BINARY, kV, kind, src, 0}; }
constexpr SS BinT(int kind, int src) { return SS{FB_CH_BINARY, kT, kind, src, 0}; }
constexpr int kOther = FB_CH_SRC_OTHER_REG, kImm = FB_CH_SRC_IMM;
constexpr int Op(int k) { return FB_CH_SRC_OPERAND0 + k; }

#define FB_PROGRAM(NAME, ...)                                   \
  struct NAME {                                                 \
    static constexpr SS steps[] = {__VA_ARGS__};                \
    static constexpr int n = sizeof(steps) / sizeof(steps[0]);  \
  };

// The programs of the manifest.
#define FB_CHAIN_PROGRAM(NAME, ...) FB_PROGRAM(NAME, __VA_ARGS__)
#define FB_CHAIN_SEG(NAME)
#define FB_CHAIN_TILE(NAME, M0, M1, M2)
#include "chain_programs.def"
#undef FB_CHAIN_PROGRAM
#undef FB_CHAIN_SEG
#undef FB_CHAIN_TILE

template <int OP, int KIND, int SRC, int SWAP, int N, class Fetch>
__device__ __forceinline__ void static_step(float p0, float p1, float (&R)[N], const float (&O)[N], Fetch& fetch) {
  if constexpr (OP == FB_CH_LOAD) {
    fetch(SRC, R);
  } else if constexpr (OP == FB_CH_IMM) {
#pragma unroll
    for (int j = 0; j < N; ++j) R[j] = p0;
  } else if constexpr (OP == FB_CH_UNARY) {
#pragma unroll
    for (int j = 0; j < N; ++j) R[j] = unary_apply(KIND, p0, p1, R[j]);
  } else {
    if constexpr (SRC == FB_CH_SRC_OTHER_REG) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        R[j] = SWAP ? binary_apply(KIND, p0, p1, O[j], R[j]) : binary_apply(KIND, p0, p1, R[j], O[j]);
    } else if constexpr (SRC == FB_CH_SRC_IMM) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        R[j] = SWAP ? binary_apply(KIND, p0, p1, p1, R[j]) : binary_apply(KIND, p0, p1, R[j], p1);
    } else {
      float other[N];
      fetch(SRC - FB_CH_SRC_OPERAND0, other);
#pragma unroll
      for (int j = 0; j < N; ++j)
        R[j] = SWAP ? binary_apply(KIND, p0, p1, other[j], R[j]) : binary_apply(KIND, p0, p1, R[j], other[j]);
    }
  }
}

template <class PROG>
struct Static {
  // Compiled programs are short of warps to cover load latency, not of
  // registers: ask for four resident CTAs of 256 threads (64 registers each).
  static constexpr int kTileCtasPerSm = 4;
  template <int I, int N, class Fetch>
  static __device__ __forceinline__ void steps(const ChainParams& P, float (&V)[N], float (&T)[N], Fetch& fetch) {
    if constexpr (I < PROG::n) {
      constexpr SS s = PROG::steps[I];
      const float p0 = P.steps[I].p0, p1 = P.steps[I].p1;
      if constexpr (s.dst == 0) static_step<s.opcode, s.kind, s.src, s.swap, N>(p0, p1, V, T, fetch);
      else static_step<s.opcode, s.kind, s.src, s.swap, N>(p0, p1, T, V, fetch);
      steps<I + 1, N>(P, V, T, fetch);
    }
  }
  template <int N, class Fetch>
  static __device__ __forceinline__ void run(const ChainParams& P, Fetch& fetch, float (&V)[N]) {
    float T[N];
#pragma unroll
    for (int j = 0; j < N; ++j) V[j] = T[j] = 0.0f;
    steps<0, N>(P, V, T, fetch);
  }
};

template <class PROG>
static bool matches(const ChainParams& P) {
  if (P.n_steps != PROG::n) return false;
  for (int i = 0; i < PROG::n; ++i) {
    const Step& r = P.steps[i];
    const SS& s = PROG::steps[i];
    if (r.opcode != s.opcode || r.dst != s.dst) return false;
    if (s.opcode == FB_CH_LOAD && r.src != s.src) return false;
    if (s.opcode == FB_CH_UNARY && r.kind != s.kind) return false;
    if (s.opcode == FB_CH_BINARY && (r.kind != s.kind || r.src != s.src || r.swap != s.swap)) return false;
  }
  return true;
}

#define FB_TRY_SEG(PROG)                                                                        \
  if (matches<PROG>(P)) {                                                                       \
    chain_seg_kernel<4, 4, Static<PROG>><<<grid, kChThreads, 0, stream>>>(P, nseg, out);        \
    return true;                                                                                \
  }
// Operand classes of a tile instantiation, operand 0 first.
constexpr int modes(int m0, int m1 = 0, int m2 = 0) { return m0 | (m1 << 2) | (m2 << 4); }
// The classes of operands a program does not have are zero in the launch parameters.
template <class PROG>
constexpr int n_operands() {
  int n = 0;
  for (int i = 0; i < PROG::n; ++i) {
    const SS& s = PROG::steps[i];
    int k = -1;
    if (s.opcode == FB_CH_LOAD) k = s.src;
    if (s.opcode == FB_CH_BINARY && s.src >= FB_CH_SRC_OPERAND0) k = s.src - FB_CH_SRC_OPERAND0;
    if (k + 1 > n) n = k + 1;
  }
  return n;
}
template <class PROG>
constexpr int used_modes(int m0, int m1, int m2) {
  constexpr int n = n_operands<PROG>();
  return modes(n > 0 ? m0 : 0, n > 1 ? m1 : 0, n > 2 ? m2 : 0);
}
#define FB_TRY_VTILE(PROG, MODES)                                                                       \
  if (TP.modes == (uint32_t)(MODES) && matches<PROG>(TP.c)) {                                           \
    chain_tile_kernel<VectorTile<(MODES)>, Static<PROG>><<<grid, kChThreads, 0, stream>>>(TP, out);     \
    return true;                                                                                        \
  }
#define FB_TRY_FTILE(PROG, MODES)                                                                       \
  if (TP.modes == (uint32_t)(MODES) && matches<PROG>(TP.c)) {                                           \
    using Tile = FullTile<(MODES), 8>;                                                                  \
    chain_tile_kernel<Tile, Static<PROG>><<<grid, Tile::kThreads, 0, stream>>>(TP, out);                \
    return true;                                                                                        \
  }

bool launch_static_seg(cudaStream_t stream, const ChainParams& P, uint64_t nseg, unsigned grid, float* out) {
#define FB_CHAIN_PROGRAM(NAME, ...)
#define FB_CHAIN_SEG(NAME) FB_TRY_SEG(NAME)
#define FB_CHAIN_TILE(NAME, M0, M1, M2)
#include "chain_programs.def"
#undef FB_CHAIN_PROGRAM
#undef FB_CHAIN_SEG
#undef FB_CHAIN_TILE
  return false;
}

bool launch_static_vtile(cudaStream_t stream, const TileParams& TP, unsigned grid, float* out) {
#define FB_CHAIN_PROGRAM(NAME, ...)
#define FB_CHAIN_SEG(NAME)
#define FB_CHAIN_TILE(NAME, M0, M1, M2) FB_TRY_VTILE(NAME, (used_modes<NAME>(M0, M1, M2)))
#include "chain_programs.def"
#undef FB_CHAIN_PROGRAM
#undef FB_CHAIN_SEG
#undef FB_CHAIN_TILE
  return false;
}

// The interior form (FullTile): the caller has checked its requirements.
bool launch_static_ftile(cudaStream_t stream, const TileParams& TP, unsigned grid, float* out) {
#define FB_CHAIN_PROGRAM(NAME, ...)
#define FB_CHAIN_SEG(NAME)
#define FB_CHAIN_TILE(NAME, M0, M1, M2) FB_TRY_FTILE(NAME, (used_modes<NAME>(M0, M1, M2)))
#include "chain_programs.def"
#undef FB_CHAIN_PROGRAM
#undef FB_CHAIN_SEG
#undef FB_CHAIN_TILE
  return false;
}

}  // namespace fb
