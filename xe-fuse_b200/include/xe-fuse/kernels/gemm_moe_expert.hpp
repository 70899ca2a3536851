// Batched expert FFN (mixture-of-experts): K2 with L = number of experts as the batch dimension.
// No special kernel is involved; the batch coordinate is part of every launch.
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_moe_expert.hpp:35-142.
#pragma once
#include "xe-fuse/kernels/gemm_rmsnorm_swiglu.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementScale_ = float,
          typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>,
          typename Activation_ = SwiGLUFn>
struct MoEExpertBatched : GemmRmsNormSwiGLU<ElementA_, ElementB_, ElementD_, ElementScale_, ElementAcc_,
                                            ElementCompute_, TileShape_, Activation_> {
  using Base = GemmRmsNormSwiGLU<ElementA_, ElementB_, ElementD_, ElementScale_, ElementAcc_,
                                 ElementCompute_, TileShape_, Activation_>;
  using ScaleVec = typename Base::ScaleBroadcast;
  using AccFetch = typename Base::Accum;
  using PairwiseVisitor = XePairwiseCompute<Activation_>;
  // scale_ptr holds L * M_exp values: one RMS factor per token of every expert
  static typename Base::EVT::Arguments make_evt_args(ElementScale_ const* scale_ptr, int M_exp) {
    return Base::make_evt_args(scale_ptr, M_exp);
  }
};

template <typename EA = cutlass::bfloat16_t, typename EB = cutlass::bfloat16_t, typename ED = cutlass::bfloat16_t,
          typename ES = float, typename EAcc = float, typename EC = float,
          typename TS = cute::Shape<cute::_256, cute::_256, cute::_32>>
using MoEExpertSwiGLU = MoEExpertBatched<EA, EB, ED, ES, EAcc, EC, TS, SwiGLUFn>;

template <typename EA = cutlass::bfloat16_t, typename EB = cutlass::bfloat16_t, typename ED = cutlass::bfloat16_t,
          typename ES = float, typename EAcc = float, typename EC = float,
          typename TS = cute::Shape<cute::_256, cute::_256, cute::_32>>
using MoEExpertGeGLU = MoEExpertBatched<EA, EB, ED, ES, EAcc, EC, TS, GeGLUFn>;

}  // namespace xe_fuse
