// RoPE nodes: rotate each column pair by (cos, sin) = cos_sin[m, 2k], cos_sin[m, 2k+1].
//   XeRoPECompute          children {cos_sin}; rotates the raw accumulator
//   XeRoPEComputeTwoChild  children {value, cos_sin}
//   XeRoPEScaledCompute    children {per-row scale, cos_sin}; rotates acc * scale[m]
// Mirrors the names of the reference's visitors/xe_rope_compute.hpp:19-219.
#pragma once

#include "xefuse/frontend.hpp"

namespace xe_fuse {
struct XeRoPECompute { struct Arguments {}; };
struct XeRoPEComputeTwoChild { struct Arguments {}; };
struct XeRoPEScaledCompute { struct Arguments {}; };
}  // namespace xe_fuse

namespace xefuse {

template <class CS>
struct Lower<fus::XeEVT<xe_fuse::XeRoPECompute, CS>> {
  template <class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val acc = Lower<fus::XeAccFetch>::apply(0, c);
    Val cs = lower<CS>(std::get<0>(t), c);
    return c.ok ? lower_rope(acc, cs, c) : Val{};
  }
};

template <class X, class CS>
struct Lower<fus::XeEVT<xe_fuse::XeRoPEComputeTwoChild, X, CS>> {
  template <class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val v = lower<X>(std::get<0>(t), c);
    Val cs = lower<CS>(std::get<1>(t), c);
    return c.ok ? lower_rope(v, cs, c) : Val{};
  }
};

template <class SC, class CS>
struct Lower<fus::XeEVT<xe_fuse::XeRoPEScaledCompute, SC, CS>> {
  template <class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val acc = Lower<fus::XeAccFetch>::apply(0, c);
    Val sc = lower<SC>(std::get<0>(t), c);
    Val cs = lower<CS>(std::get<1>(t), c);
    if (!c.ok) return Val{};
    Val v = lower_mul(acc, sc, c);
    return c.ok ? lower_rope(v, cs, c) : Val{};
  }
};

}  // namespace xefuse
