// Exercises ferro_b200/host/ferro_b200.hpp (the C++ mirror of ferro's Backend seam) end to end.
// Known answers are those of ferro's own tests: LayerNorm of [1,2,3] (crates/ferro-core/tests/op_layer_norm.rs:15-22),
// softmax rows sum to one (tests/op_softmax.rs:5-15), sum_dim of [[1,2,3],[4,5,6]] (tests/op_sum_dim.rs:5-16),
// argmax ties and NaN (tests/op_argmax.rs:20-27), first Adam step = -lr (tests/optim.rs:127-157),
// shape errors of layer_norm_dev (crates/ferro-cuda/tests/layer_norm_fused.rs:17-22).
#include <cmath>
#include <cstdio>

#include "../../ferro_b200/host/ferro_b200.hpp"

#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); return 1; } \
  } while (0)

int main() {
  fb::CudaBackend be(0);
  {
    auto x = be.alloc_from_host({1.f, 2.f, 3.f});
    auto y = be.copy_to_host(*be.layer_norm_output_dev(*x, nullptr, nullptr, 1, 3, 1e-5f));
    const float s = std::sqrt(1.5f);
    EXPECT(std::fabs(y[0] + s) < 1e-5f && std::fabs(y[1]) < 1e-5f && std::fabs(y[2] - s) < 1e-5f);
    bool threw = false;
    try { be.layer_norm_dev(*x, nullptr, nullptr, 2, 3, 1e-5f); } catch (const fb::InvalidShape&) { threw = true; }
    EXPECT(threw);
    auto [yy, h, sd] = be.layer_norm_dev(*x, nullptr, nullptr, 1, 3, 1e-5f);
    auto g = be.alloc_from_host({0.15f, 0.42f, 0.69f});
    auto [dx, dw, db] = be.layer_norm_backward_dev(*g, *h, *sd, nullptr, 1, 3);
    auto dxv = be.copy_to_host(*dx);
    EXPECT(std::fabs(dxv[0] + dxv[1] + dxv[2]) < 1e-5f);  // orthogonal to 1
    auto dbv = be.copy_to_host(*db);
    EXPECT(dbv[1] == 0.42f);
    // RMS normalisation of [3, 4]: rms = sqrt(12.5) (nn.rs:255-283)
    auto r = be.alloc_from_host({3.f, 4.f});
    auto [ry, rrs] = be.rms_norm_dev(*r, nullptr, 1, 2, 0.0f);
    auto ryv = be.copy_to_host(*ry);
    const float rms = std::sqrt(12.5f);
    EXPECT(std::fabs(ryv[0] - 3.f / rms) < 1e-6f && std::fabs(ryv[1] - 4.f / rms) < 1e-6f);
    auto rg = be.alloc_from_host({1.f, 1.f});
    auto [rdx, rdw] = be.rms_norm_backward_dev(*rg, *r, *rrs, nullptr, 1, 2);
    auto rdxv = be.copy_to_host(*rdx);
    EXPECT(std::fabs(rdxv[0] * 3.f + rdxv[1] * 4.f) < 1e-5f);  // the gradient is orthogonal to x
  }
  {
    auto x = be.alloc_from_host({1, 2, 3, 0, 0, 0});
    auto y = be.copy_to_host(*be.softmax_dev(*x, 2, 3));
    EXPECT(std::fabs(y[0] + y[1] + y[2] - 1.f) < 1e-5f && std::fabs(y[3] - 1.f / 3) < 1e-6f);
    auto a = be.alloc_from_host({1, 2, 3, 4, 5, 6});
    auto s0 = be.copy_to_host(*be.sum_dim_dev(*a, {2, 3}, 0));
    EXPECT(s0[0] == 5 && s0[1] == 7 && s0[2] == 9);
    auto b = be.alloc_from_host({1.f, NAN, 9.f});
    auto am = be.copy_i64_to_host(*be.max_dim_dev(*b, {3}, 0).second);
    EXPECT(am[0] == 1);
    auto t = be.alloc_from_host({2.f, 2.f, 1.f});
    EXPECT(be.copy_i64_to_host(*be.max_dim_dev(*t, {3}, 0).second)[0] == 0);
  }
  {
    auto p = be.alloc_from_host({1.f}), m = be.fill_dev(0.f, 1), v = be.fill_dev(0.f, 1), g = be.alloc_from_host({0.5f});
    be.adamw_step_dev(*p, *m, *v, *g, fb::AdamWStep{0.1f, 0.9f, 0.999f, 1.f - 0.9f, 1.f - 0.999f, 1e-8f, 0.f});
    EXPECT(std::fabs(be.copy_to_host(*p)[0] - 0.9f) < 1e-4f);
    auto r = be.copy_to_host(*be.unary_dev(fb::UnaryKind{FB_UN_RELU}, *be.alloc_from_host({-1.f, -0.f, 2.f, NAN})));
    EXPECT(r[0] == 0.f && r[1] == 0.f && !std::signbit(r[1]) && r[2] == 2.f && std::isnan(r[3]));
    auto bc = be.copy_to_host(*be.binary_bc_dev(fb::BinaryKind{FB_BIN_ADD}, *be.alloc_from_host({1, 2, 3, 4, 5, 6}), {2, 3},
                                                *be.alloc_from_host({10, 20, 30}), {3}, {2, 3}));
    EXPECT(bc[0] == 11 && bc[5] == 36);
  }
  std::printf("host_backend_test ok, %llu kernel launches\n", (unsigned long long)fb_launch_count());
  return 0;
}
