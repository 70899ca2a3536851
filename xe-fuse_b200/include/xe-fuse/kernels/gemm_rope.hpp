// K3 -- GEMM + RoPE on the raw accumulator; cos_sin is an [M,N] fp32 tensor (cos at even columns,
// sin at odd ones).  Same public members and make_evt_args signature as the reference's
// kernels/gemm_rope.hpp:41-110.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementCosSin_ = float,
          typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmRoPE
    : builder::MakeGemm<builder::RoPE<ElementCosSin_>, ElementA_, ElementB_, ElementD_, ElementAcc_,
                        ElementCompute_, TileShape_> {
  using ElementCosSin = ElementCosSin_;
  using StrideCosSin = builder::PackedMN;
  using CosSinLoad = builder::AuxLoad<ElementCosSin_>;
  using RoPENode = XeRoPECompute;
  using EVT = builder::RoPE<ElementCosSin_>;

  static typename EVT::Arguments make_evt_args(ElementCosSin const* cos_sin_ptr, StrideCosSin stride_cos_sin) {
    typename CosSinLoad::Arguments cs;
    cs.ptr_aux = cos_sin_ptr;
    cs.null_default = ElementCosSin(0);
    cs.dAux = stride_cos_sin;
    return {cs, typename RoPENode::Arguments{}};
  }
};

}  // namespace xe_fuse
