// K4 -- GEMM + RMSNorm row scale + RoPE:  rotate (acc * R[m]) by cos_sin[m, .].
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_rmsnorm_rope.hpp:43-146.  For a per-head table [M, head_dim] set
// Extensions::cos_sin_period on the Gemm object.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementScale_ = float,
          typename ElementCosSin_ = float, typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmRmsNormRoPE
    : builder::MakeGemm<builder::RoPEComposed<builder::ScaleRows<builder::Acc, TileShape_, ElementScale_, ElementCompute_>, ElementCosSin_>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_> {
  using ElementScale = ElementScale_;
  using ElementCosSin = ElementCosSin_;
  using StrideCosSin = builder::PackedMN;
  using Accum = builder::Acc;
  using ScaleBroadcast = builder::ColBroadcast<0, TileShape_, ElementScale_, ElementCompute_>;
  using MulCompute = builder::MulOp<ElementCompute_, ElementCompute_>;
  using RmsScale = builder::ScaleRows<Accum, TileShape_, ElementScale_, ElementCompute_>;
  using CosSinLoad = builder::AuxLoad<ElementCosSin_>;
  using RoPENode = XeRoPEComputeTwoChild;
  using EVT = builder::RoPEComposed<RmsScale, ElementCosSin_>;

  static typename EVT::Arguments make_evt_args(ElementScale const* scale_ptr, int M,
                                               ElementCosSin const* cos_sin_ptr, StrideCosSin stride_cos_sin) {
    typename ScaleBroadcast::Arguments scale;
    scale.ptr_col = scale_ptr;
    scale.null_default = ElementScale(1);
    scale.dCol = {cute::Int<1>{}, cute::Int<0>{}, static_cast<int64_t>(M)};
    typename RmsScale::Arguments rms{typename Accum::Arguments{}, scale, typename MulCompute::Arguments{}};
    typename CosSinLoad::Arguments cs;
    cs.ptr_aux = cos_sin_ptr;
    cs.null_default = ElementCosSin(0);
    cs.dAux = stride_cos_sin;
    return {rms, cs, typename RoPENode::Arguments{}};
  }
};

}  // namespace xe_fuse
