// K8 -- GEMM + SwiGLU on the raw accumulator (no row scale).
// Same public members and make_evt_args signature as the reference's kernels/gemm_swiglu.hpp:39-94.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementAcc_ = float,
          typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmSwiGLU
    : builder::MakeGemm<builder::SwiGLU<builder::Acc>, ElementA_, ElementB_, ElementD_, ElementAcc_,
                        ElementCompute_, TileShape_> {
  using Accum = builder::Acc;
  using SwiGLUVisitor = XePairwiseCompute<SwiGLUFn>;
  using EVT = builder::SwiGLU<Accum>;
  static typename EVT::Arguments make_evt_args() {
    return {typename Accum::Arguments{}, typename SwiGLUVisitor::Arguments{}};
  }
};

}  // namespace xe_fuse
