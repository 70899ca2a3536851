// K1 -- GEMM + RMSNorm row scale:  D[m,n] = acc[m,n] * R[m].
// Same public members and make_evt_args signature as the reference's kernels/gemm_rmsnorm.hpp:29-104.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementScale_ = float,
          typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmRmsNorm
    : builder::MakeGemm<builder::Mul<builder::Acc, builder::ColBroadcast<0, TileShape_, ElementScale_, ElementCompute_>,
                                     ElementD_, ElementCompute_>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_> {
  using ElementScale = ElementScale_;
  using Accum = builder::Acc;
  using ScaleBroadcast = builder::ColBroadcast<0, TileShape_, ElementScale_, ElementCompute_>;
  using MulCompute = builder::MulOp<ElementD_, ElementCompute_>;
  using EVT = builder::Mul<Accum, ScaleBroadcast, ElementD_, ElementCompute_>;

  // scale_ptr: R[m], one fp32 per row and batch (batch stride M)
  static typename EVT::Arguments make_evt_args(ElementScale const* scale_ptr, int M) {
    typename ScaleBroadcast::Arguments scale;
    scale.ptr_col = scale_ptr;
    scale.null_default = ElementScale(1);
    scale.dCol = {cute::Int<1>{}, cute::Int<0>{}, static_cast<int64_t>(M)};
    return {typename Accum::Arguments{}, scale, typename MulCompute::Arguments{}};
  }
};

}  // namespace xe_fuse
