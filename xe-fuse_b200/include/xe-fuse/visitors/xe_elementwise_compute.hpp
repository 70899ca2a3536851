// Unary activation nodes of the builder API.  On B200 a node is only a tag: the math runs inside
// the fused kernel's epilogue (xf_unary of include/xefuse_b200.h); the functors below also work on
// the host so harness code can call them.
// Mirrors the node and functor names of the reference's visitors/xe_elementwise_compute.hpp:18-89.
#pragma once

#include <cmath>

#include "xefuse/frontend.hpp"

namespace xe_fuse {

struct GeLUFn     { static constexpr int code = XF_UNARY_GELU;      float operator()(float x) const { return x * 0.5f * (1.0f + std::erf(x * 0.7071067811865475f)); } };
struct GeLUTanhFn { static constexpr int code = XF_UNARY_GELU_TANH; float operator()(float x) const { return x * 0.5f * (1.0f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x))); } };
struct SiLUFn     { static constexpr int code = XF_UNARY_SILU;      float operator()(float x) const { return x / (1.0f + std::exp(-x)); } };
struct ReLUFn     { static constexpr int code = XF_UNARY_RELU;      float operator()(float x) const { return x > 0.0f ? x : 0.0f; } };
struct SigmoidFn  { static constexpr int code = XF_UNARY_SIGMOID;   float operator()(float x) const { return 1.0f / (1.0f + std::exp(-x)); } };
struct ExpFn      { static constexpr int code = XF_UNARY_EXP;       float operator()(float x) const { return std::exp(x); } };

template <class ElementwiseFn>
struct XeElementwiseCompute { struct Arguments {}; };

}  // namespace xe_fuse

namespace xefuse {
template <class Fn, class X>
struct Lower<fus::XeEVT<xe_fuse::XeElementwiseCompute<Fn>, X>> {
  template <class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val v = lower<X>(std::get<0>(t), c);
    return c.ok ? lower_unary(v, Fn::code, c) : Val{};
  }
};
}  // namespace xefuse
