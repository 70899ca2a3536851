// Pair nodes: an operation on adjacent output columns (2k, 2k+1).  In the B200 kernel a thread
// holds both columns of a pair in neighbouring registers, so no lane exchange is involved.
// Mirrors the names of the reference's visitors/xe_pairwise_compute.hpp:20-109.
#pragma once

#include <cmath>

#include "xefuse/frontend.hpp"

namespace xe_fuse {

// Functors keep the reference's call shape (my value, partner value, am-I-the-even-column).
struct PairwiseSwapFn {
  static constexpr int code = XF_PAIR_SWAP;
  float operator()(float, float partner, bool) const { return partner; }
};
struct SwiGLUFn {
  static constexpr int code = XF_PAIR_SWIGLU;
  float operator()(float mine, float partner, bool even) const {
    const float gate = even ? mine : partner, up = even ? partner : mine;
    return gate / (1.0f + std::exp(-gate)) * up;
  }
};
struct GeGLUFn {
  static constexpr int code = XF_PAIR_GEGLU;
  float operator()(float mine, float partner, bool even) const {
    const float gate = even ? mine : partner, up = even ? partner : mine;
    return gate * 0.5f * (1.0f + std::erf(gate * 0.7071067811865475f)) * up;
  }
};
struct RoPEFn {
  float cos_val = 1.f, sin_val = 0.f;
  float operator()(float mine, float partner, bool even) const {
    return even ? mine * cos_val + partner * sin_val : -partner * sin_val + mine * cos_val;
  }
};

template <class PairwiseFn_>
struct XePairwiseCompute {
  using PairwiseFn = PairwiseFn_;
  struct Arguments {};
};

}  // namespace xe_fuse

namespace xefuse {
template <class Fn, class X>
struct Lower<fus::XeEVT<xe_fuse::XePairwiseCompute<Fn>, X>> {
  template <class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val v = lower<X>(std::get<0>(t), c);
    return c.ok ? lower_pair(v, Fn::code, c) : Val{};
  }
};
}  // namespace xefuse
