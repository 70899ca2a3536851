// K4 for W8A8 -- dequantise the int32 accumulator, then RoPE; scale_token[m] carries both the
// activation quantisation range and the RMSNorm factor.
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_dequant_rope.hpp:48-177.
#pragma once
#include "xe-fuse/kernels/gemm_dequant_w8a8.hpp"

namespace xe_fuse {

template <typename ElementA_ = int8_t, typename ElementB_ = int8_t, typename ElementD_ = cutlass::bfloat16_t,
          typename ElementScale_ = float, typename ElementCosSin_ = float, typename ElementAcc_ = int32_t,
          typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDequantRoPE
    : builder::MakeGemm<builder::DequantRoPE<TileShape_, ElementScale_, ElementCosSin_, ElementCompute_>, ElementA_,
                        ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_,
                        cutlass::layout::RowMajor, cutlass::layout::RowMajor, 32, 8> {
  using ElementScale = ElementScale_;
  using ElementCosSin = ElementCosSin_;
  using StrideCosSin = builder::PackedMN;
  using Parts = detail::DequantArgs<TileShape_, ElementScale_, ElementCompute_>;
  using DequantTree = typename Parts::DequantTree;
  using CosSinLoad = builder::AuxLoad<ElementCosSin_>;
  using RoPENode = XeRoPEComputeTwoChild;
  using EVT = builder::DequantRoPE<TileShape_, ElementScale_, ElementCosSin_, ElementCompute_>;

  static typename EVT::Arguments make_evt_args(ElementScale const* scale_token_ptr, int M,
                                               ElementScale const* scale_channel_ptr, int N,
                                               ElementCosSin const* cos_sin_ptr, StrideCosSin stride_cos_sin) {
    typename CosSinLoad::Arguments cs;
    cs.ptr_aux = cos_sin_ptr;
    cs.null_default = ElementCosSin(0);
    cs.dAux = stride_cos_sin;
    return {Parts::make(scale_token_ptr, M, scale_channel_ptr, N), cs, typename RoPENode::Arguments{}};
  }
};

}  // namespace xe_fuse
