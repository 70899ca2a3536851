// K0a -- GEMM + residual add + per-column gamma:  D[m,n] = gamma[n] * (acc[m,n] + residual[m,n]).
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_residual_gamma.hpp:41-139.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementResidual_ = cutlass::bfloat16_t,
          typename ElementGamma_ = float, typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmResidualGamma
    : builder::MakeGemm<builder::Mul<builder::RowBroadcast<0, TileShape_, ElementGamma_, ElementCompute_>,
                                     builder::AddResidual<ElementResidual_, ElementCompute_>, ElementD_, ElementCompute_>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_> {
  using ElementResidual = ElementResidual_;
  using ElementGamma = ElementGamma_;
  using StrideResidual = builder::PackedMN;
  using Accum = builder::Acc;
  using ResidualLoad = builder::AuxLoad<ElementResidual_>;
  using AddCompute = builder::AddOp<ElementCompute_, ElementCompute_>;
  using EVTAdd = builder::AddResidual<ElementResidual_, ElementCompute_>;
  using GammaBroadcast = builder::RowBroadcast<0, TileShape_, ElementGamma_, ElementCompute_>;
  using MulCompute = builder::MulOp<ElementD_, ElementCompute_>;
  using EVT = builder::Mul<GammaBroadcast, EVTAdd, ElementD_, ElementCompute_>;

  static typename EVT::Arguments make_evt_args(ElementResidual const* residual_ptr, StrideResidual stride_residual,
                                               ElementGamma const* gamma_ptr, int N) {
    typename ResidualLoad::Arguments res;
    res.ptr_aux = residual_ptr;
    res.null_default = ElementResidual(0);
    res.dAux = stride_residual;
    typename EVTAdd::Arguments add{typename Accum::Arguments{}, res, typename AddCompute::Arguments{}};
    typename GammaBroadcast::Arguments gamma;
    gamma.ptr_row = gamma_ptr;
    gamma.null_default = ElementGamma(1);
    gamma.dRow = {cute::Int<0>{}, cute::Int<1>{}, static_cast<int64_t>(N)};
    return {gamma, add, typename MulCompute::Arguments{}};
  }
};

}  // namespace xe_fuse
