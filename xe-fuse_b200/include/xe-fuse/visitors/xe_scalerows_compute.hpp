// "Merged" nodes: acc * R[m], optionally followed by SwiGLU / GeGLU, as one node with a single
// per-row-scale child.  The reference merges them to save registers on Xe; here they lower to the
// same flat program (and the same kernel) as the composed trees.
// Mirrors the names of the reference's visitors/xe_scalerows_compute.hpp:20-142.
#pragma once

#include "xefuse/frontend.hpp"

namespace xe_fuse {
struct XeScaleRowsCompute { struct Arguments {}; };
struct XeScaleRowsSwiGLUCompute { struct Arguments {}; };
struct XeScaleRowsGeGLUCompute { struct Arguments {}; };
}  // namespace xe_fuse

namespace xefuse {

template <int PairOp>
struct LowerScaledRows {
  template <class SC, class Args>
  static Val apply(Args const& t, Ctx& c) {
    Val acc = Lower<fus::XeAccFetch>::apply(0, c);
    Val sc = lower<SC>(std::get<0>(t), c);
    if (!c.ok) return Val{};
    Val v = lower_mul(acc, sc, c);
    if (!c.ok || PairOp == XF_PAIR_NONE) return v;
    return lower_pair(v, PairOp, c);
  }
};

template <class SC>
struct Lower<fus::XeEVT<xe_fuse::XeScaleRowsCompute, SC>> {
  template <class Args> static Val apply(Args const& t, Ctx& c) { return LowerScaledRows<XF_PAIR_NONE>::template apply<SC>(t, c); }
};
template <class SC>
struct Lower<fus::XeEVT<xe_fuse::XeScaleRowsSwiGLUCompute, SC>> {
  template <class Args> static Val apply(Args const& t, Ctx& c) { return LowerScaledRows<XF_PAIR_SWIGLU>::template apply<SC>(t, c); }
};
template <class SC>
struct Lower<fus::XeEVT<xe_fuse::XeScaleRowsGeGLUCompute, SC>> {
  template <class Args> static Val apply(Args const& t, Ctx& c) { return LowerScaledRows<XF_PAIR_GEGLU>::template apply<SC>(t, c); }
};

}  // namespace xefuse
