// K2 for W8A8 -- dequantise the int32 accumulator, then SwiGLU (or GeGLU) on interleaved columns.
// Same public members and make_evt_args signatures as the reference's
// kernels/gemm_dequant_swiglu.hpp:51-268.
#pragma once
#include "xe-fuse/kernels/gemm_dequant_w8a8.hpp"

namespace xe_fuse {

namespace detail {
template <class PairFn, typename ElementA_, typename ElementB_, typename ElementD_, typename ElementScale_,
          typename ElementAcc_, typename ElementCompute_, typename TileShape_>
struct GemmDequantGated
    : builder::MakeGemm<builder::Pairwise<PairFn, builder::DequantW8A8<TileShape_, ElementScale_, ElementCompute_>>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_,
                        cutlass::layout::RowMajor, cutlass::layout::RowMajor, 32, 8> {
  using ElementScale = ElementScale_;
  using Parts = DequantArgs<TileShape_, ElementScale_, ElementCompute_>;
  using DequantTree = typename Parts::DequantTree;
  using EVT = builder::Pairwise<PairFn, DequantTree>;
  static typename EVT::Arguments make_evt_args(ElementScale const* scale_token_ptr, int M,
                                               ElementScale const* scale_channel_ptr, int N) {
    return {Parts::make(scale_token_ptr, M, scale_channel_ptr, N), typename XePairwiseCompute<PairFn>::Arguments{}};
  }
};
}  // namespace detail

template <typename ElementA_ = int8_t, typename ElementB_ = int8_t, typename ElementD_ = cutlass::bfloat16_t,
          typename ElementScale_ = float, typename ElementAcc_ = int32_t, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDequantSwiGLU : detail::GemmDequantGated<SwiGLUFn, ElementA_, ElementB_, ElementD_, ElementScale_,
                                                    ElementAcc_, ElementCompute_, TileShape_> {
  using SwiGLUVisitor = XePairwiseCompute<SwiGLUFn>;
};

template <typename ElementA_ = int8_t, typename ElementB_ = int8_t, typename ElementD_ = cutlass::bfloat16_t,
          typename ElementScale_ = float, typename ElementAcc_ = int32_t, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDequantGeGLU : detail::GemmDequantGated<GeGLUFn, ElementA_, ElementB_, ElementD_, ElementScale_,
                                                   ElementAcc_, ElementCompute_, TileShape_> {
  using GeGLUVisitor = XePairwiseCompute<GeGLUFn>;
};

}  // namespace xe_fuse
