// K2 -- GEMM + RMSNorm row scale + SwiGLU on interleaved gate/up columns:
//   D[m,2k] = D[m,2k+1] = silu(acc[m,2k] * R[m]) * (acc[m,2k+1] * R[m]).
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_rmsnorm_swiglu.hpp:43-127.  For a compact [M,N/2] output set
// Extensions::compact_pair_output on the Gemm object.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementScale_ = float,
          typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>,
          typename PairFn_ = SwiGLUFn>
struct GemmRmsNormSwiGLU
    : builder::MakeGemm<builder::Pairwise<PairFn_, builder::ScaleRows<builder::Acc, TileShape_, ElementScale_, ElementCompute_>>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_> {
  using ElementScale = ElementScale_;
  using Accum = builder::Acc;
  using ScaleBroadcast = builder::ColBroadcast<0, TileShape_, ElementScale_, ElementCompute_>;
  using MulCompute = builder::MulOp<ElementCompute_, ElementCompute_>;
  using EVTRmsScale = builder::ScaleRows<Accum, TileShape_, ElementScale_, ElementCompute_>;
  using SwiGLUVisitor = XePairwiseCompute<PairFn_>;
  using EVT = builder::Pairwise<PairFn_, EVTRmsScale>;

  static typename EVT::Arguments make_evt_args(ElementScale const* scale_ptr, int M) {
    typename ScaleBroadcast::Arguments scale;
    scale.ptr_col = scale_ptr;
    scale.null_default = ElementScale(1);
    scale.dCol = {cute::Int<1>{}, cute::Int<0>{}, static_cast<int64_t>(M)};
    typename EVTRmsScale::Arguments inner{typename Accum::Arguments{}, scale, typename MulCompute::Arguments{}};
    return {inner, typename SwiGLUVisitor::Arguments{}};
  }
};

}  // namespace xe_fuse
