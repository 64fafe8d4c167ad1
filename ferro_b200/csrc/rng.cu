// ferro's random generator for seeded inputs, on the host: `ferro_core::Rng`
// (crates/ferro-core/src/rng.rs:12-70) is a splitmix64-seeded xorshift128+
// whose draws fill tensors row-major on the CPU before they are uploaded
// (Tensor::randn / rand, crates/ferro-core/src/tensor.rs:365-372).  Runs that
// say "seed 0 via ferro Rng" need the same stream of values, so the library
// carries the generator; outputs are HOST buffers.
//
// The state advances strictly in sequence (one xorshift step per 24-bit
// uniform, two uniforms per normal), which costs about a nanosecond per draw;
// the expensive part of a normal is logf / sqrtf / cosf.  Large fills
// therefore run in blocks: one thread advances the state and stores the raw
// 24-bit draws of a block, then all host threads turn them into values.  The
// result does not depend on the thread count: every value is a pure function
// of its own draws, computed with the C library's single-precision routines
// (the ones Rust's f32::ln / sqrt / cos lower to on Linux).
#include <cmath>
#include <thread>
#include <vector>

#include "common.cuh"

namespace fb {

static inline uint64_t splitmix(uint64_t& z) {
  z += 0x9E3779B97F4A7C15ull;
  uint64_t x = z;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

static inline uint32_t next24(fb_rng* r) {  // the top 24 bits of one xorshift128+ step
  uint64_t x = r->s0;
  const uint64_t y = r->s1;
  r->s0 = y;
  x ^= x << 23;
  x ^= x >> 17;
  x ^= y ^ (y >> 26);
  r->s1 = x;
  return (uint32_t)((x + y) >> 40);
}

static inline float to_uniform(uint32_t bits24) { return (float)bits24 / 16777216.0f; }
static inline float to_normal(uint32_t a, uint32_t b) {
  const float u1 = fmaxf(to_uniform(a), 1e-9f);
  const float u2 = to_uniform(b);
  const float rad = sqrtf(-2.0f * logf(u1));
  return rad * cosf(6.28318530717958647692f * u2);
}

static unsigned host_threads() {
  unsigned n = std::thread::hardware_concurrency();
  if (n == 0) n = 1;
  return n > 32 ? 32 : n;
}

// Runs fn(begin, end) over [0, n) split across the host threads.
template <typename F>
static void parallel_for(uint64_t n, F fn) {
  const unsigned t = (n < 65536) ? 1 : host_threads();
  if (t == 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
  const uint64_t per = (n + t - 1) / t;
  for (unsigned i = 0; i < t; ++i) {
    const uint64_t b = (uint64_t)i * per, e = b + per < n ? b + per : n;
    if (b >= e) break;
    pool.emplace_back([=] { fn(b, e); });
  }
  for (auto& th : pool) th.join();
}

constexpr uint64_t kBlock = 1ull << 21;  // values per block

}  // namespace fb

using namespace fb;

extern "C" {

void fb_rng_seed(fb_rng* r, uint64_t seed) {
  if (!r) return;
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  r->s0 = splitmix(z) | 1ull;
  r->s1 = splitmix(z) | 1ull;
}

float fb_rng_uniform(fb_rng* r) { return to_uniform(next24(r)); }
float fb_rng_normal(fb_rng* r) {
  const uint32_t a = next24(r), b = next24(r);
  return to_normal(a, b);
}

void fb_rng_skip(fb_rng* r, uint64_t draws) {
  if (!r) return;
  for (uint64_t i = 0; i < draws; ++i) (void)next24(r);
}

int fb_rng_fill_uniform(fb_rng* r, float* out, uint64_t n, float scale, float shift) {
  if (!r || (n && !out)) return fail(FB_ERR_INVALID_ARG, "fb_rng_fill_uniform: null argument");
  std::vector<uint32_t> raw(n < kBlock ? n : kBlock);
  for (uint64_t base = 0; base < n; base += kBlock) {
    const uint64_t m = n - base < kBlock ? n - base : kBlock;
    for (uint64_t i = 0; i < m; ++i) raw[i] = next24(r);
    const uint32_t* rp = raw.data();
    float* op = out + base;
    parallel_for(m, [=](uint64_t b, uint64_t e) {
      for (uint64_t i = b; i < e; ++i) op[i] = shift + scale * to_uniform(rp[i]);
    });
  }
  return FB_OK;
}

int fb_rng_fill_normal(fb_rng* r, float* out, uint64_t n, float scale, float shift) {
  if (!r || (n && !out)) return fail(FB_ERR_INVALID_ARG, "fb_rng_fill_normal: null argument");
  std::vector<uint32_t> raw(2 * (n < kBlock ? n : kBlock));
  for (uint64_t base = 0; base < n; base += kBlock) {
    const uint64_t m = n - base < kBlock ? n - base : kBlock;
    for (uint64_t i = 0; i < 2 * m; ++i) raw[i] = next24(r);
    const uint32_t* rp = raw.data();
    float* op = out + base;
    parallel_for(m, [=](uint64_t b, uint64_t e) {
      for (uint64_t i = b; i < e; ++i) op[i] = shift + scale * to_normal(rp[2 * i], rp[2 * i + 1]);
    });
  }
  return FB_OK;
}

int fb_rng_fill_rowscaled_normal(fb_rng* r, float* out, uint64_t rows, uint64_t cols, float lo, float span) {
  if (!r || (rows && cols && !out)) return fail(FB_ERR_INVALID_ARG, "fb_rng_fill_rowscaled_normal: null argument");
  if (rows == 0 || cols == 0) return FB_OK;
  // One uniform per row (its scale), drawn before the row's normals.
  uint64_t rb = kBlock / cols;
  if (rb == 0) rb = 1;
  std::vector<uint32_t> raw((size_t)rb * (1 + 2 * cols));
  for (uint64_t r0 = 0; r0 < rows; r0 += rb) {
    const uint64_t m = rows - r0 < rb ? rows - r0 : rb;
    const uint64_t per = 1 + 2 * cols;
    for (uint64_t i = 0; i < m * per; ++i) raw[i] = next24(r);
    const uint32_t* rp = raw.data();
    float* op = out + r0 * cols;
    parallel_for(m * cols, [=](uint64_t b, uint64_t e) {
      for (uint64_t i = b; i < e; ++i) {
        const uint64_t row = i / cols, c = i % cols;
        const uint32_t* q = rp + row * per;
        const float sc = lo + span * to_uniform(q[0]);
        op[i] = to_normal(q[1 + 2 * c], q[2 + 2 * c]) * sc;
      }
    });
  }
  return FB_OK;
}

int fb_rng_fill_index(fb_rng* r, int64_t* out, uint64_t n, uint64_t classes) {
  if (!r || (n && !out) || classes == 0) return fail(FB_ERR_INVALID_ARG, "fb_rng_fill_index: bad argument");
  for (uint64_t i = 0; i < n; ++i) {
    int64_t t = (int64_t)floorf(to_uniform(next24(r)) * (float)classes);
    if (t >= (int64_t)classes) t = (int64_t)classes - 1;
    out[i] = t;
  }
  return FB_OK;
}

}  // extern "C"
