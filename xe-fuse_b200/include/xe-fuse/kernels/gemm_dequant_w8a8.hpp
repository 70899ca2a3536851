// W8A8 dequantisation kernels: int8 x int8 -> int32 accumulator, then
//   D = bf16( float(acc) * scale_token[m] * scale_channel[n] ).
// Same public members and make_evt_args signatures as the reference's
// kernels/gemm_dequant_w8a8.hpp:42-221.  The QuaRot variant (Hadamard output node) is declared so
// that code naming it compiles; can_implement() refuses it.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

namespace detail {
// {acc, scale_token} -> inner product node arguments, shared by the W8A8 bundles.
template <class TileShape, class ElementScale, class ElementCompute>
struct DequantArgs {
  using Accum = builder::Acc;
  using TokenScaleBroadcast = builder::ColBroadcast<0, TileShape, ElementScale, ElementCompute>;
  using ChannelScaleBroadcast = builder::RowBroadcast<1, TileShape, ElementScale, ElementCompute>;
  using MulCompute = builder::MulOp<ElementCompute, ElementCompute>;
  using InnerDequant = builder::Mul<Accum, TokenScaleBroadcast, ElementCompute, ElementCompute>;
  using DequantTree = builder::Mul<InnerDequant, ChannelScaleBroadcast, ElementCompute, ElementCompute>;

  static typename DequantTree::Arguments make(ElementScale const* scale_token_ptr, int M,
                                              ElementScale const* scale_channel_ptr, int N) {
    typename TokenScaleBroadcast::Arguments tok;
    tok.ptr_col = scale_token_ptr;
    tok.null_default = ElementScale(1);
    tok.dCol = {cute::Int<1>{}, cute::Int<0>{}, static_cast<int64_t>(M)};
    typename InnerDequant::Arguments inner{typename Accum::Arguments{}, tok, typename MulCompute::Arguments{}};
    typename ChannelScaleBroadcast::Arguments ch;
    ch.ptr_row = scale_channel_ptr;
    ch.null_default = ElementScale(1);
    ch.dRow = {cute::Int<0>{}, cute::Int<1>{}, static_cast<int64_t>(N)};
    return {inner, ch, typename MulCompute::Arguments{}};
  }
};
}  // namespace detail

template <typename ElementA_ = int8_t, typename ElementB_ = int8_t, typename ElementD_ = cutlass::bfloat16_t,
          typename ElementScale_ = float, typename ElementAcc_ = int32_t, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDequantW8A8
    : builder::MakeGemm<builder::DequantW8A8<TileShape_, ElementScale_, ElementCompute_>, ElementA_, ElementB_,
                        ElementD_, ElementAcc_, ElementCompute_, TileShape_, cutlass::layout::RowMajor,
                        cutlass::layout::RowMajor, 32, 8> {
  using ElementScale = ElementScale_;
  using Parts = detail::DequantArgs<TileShape_, ElementScale_, ElementCompute_>;
  using Accum = typename Parts::Accum;
  using TokenScaleBroadcast = typename Parts::TokenScaleBroadcast;
  using ChannelScaleBroadcast = typename Parts::ChannelScaleBroadcast;
  using MulCompute = typename Parts::MulCompute;
  using InnerDequant = typename Parts::InnerDequant;
  using EVT = typename Parts::DequantTree;

  static typename EVT::Arguments make_evt_args(ElementScale const* scale_token_ptr, int M,
                                               ElementScale const* scale_channel_ptr, int N) {
    return Parts::make(scale_token_ptr, M, scale_channel_ptr, N);
  }
};

template <int GroupSize_ = 16, typename ElementA_ = int8_t, typename ElementB_ = int8_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementScale_ = float,
          typename ElementAcc_ = int32_t, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDequantW8A8QuaRot
    : builder::MakeGemm<builder::HadamardOutput<builder::DequantW8A8<TileShape_, ElementScale_, ElementCompute_>, GroupSize_>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_,
                        cutlass::layout::RowMajor, cutlass::layout::RowMajor, 32, 8> {
  static constexpr int GroupSize = GroupSize_;
  using ElementScale = ElementScale_;
  using PlainKernel = GemmDequantW8A8<ElementA_, ElementB_, ElementD_, ElementScale_, ElementAcc_, ElementCompute_, TileShape_>;
  using DequantEVT = typename PlainKernel::EVT;
  using HadamardOp = XeHadamardCompute<GroupSize_>;
  using EVT = builder::HadamardOutput<DequantEVT, GroupSize_>;
  static typename EVT::Arguments make_evt_args(ElementScale const* scale_token_ptr, int M,
                                               ElementScale const* scale_channel_ptr, int N) {
    return {PlainKernel::make_evt_args(scale_token_ptr, M, scale_channel_ptr, N), typename HadamardOp::Arguments{}};
  }
};

}  // namespace xe_fuse
