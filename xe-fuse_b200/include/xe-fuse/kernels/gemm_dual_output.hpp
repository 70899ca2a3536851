// K0 -- GEMM + residual add with two outputs: the raw sum acc + residual goes to an aux bf16
// buffer (the next RMSNorm's input) and D = gamma[n] * (acc + residual).
// Same public members and make_evt_args signature as the reference's
// kernels/gemm_dual_output.hpp:30-133.
#pragma once
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementResidual_ = cutlass::bfloat16_t,
          typename ElementGamma_ = float, typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmDualOutput
    : builder::MakeGemm<builder::DualOutput<builder::AddResidual<ElementResidual_, ElementCompute_>,
                                            builder::Mul<builder::Acc, builder::RowBroadcast<0, TileShape_, ElementGamma_, ElementCompute_>, ElementD_, ElementCompute_>,
                                            ElementD_>,
                        ElementA_, ElementB_, ElementD_, ElementAcc_, ElementCompute_, TileShape_> {
  using ElementResidual = ElementResidual_;
  using ElementGamma = ElementGamma_;
  using StrideAux = builder::PackedMN;
  using InputTree = builder::AddResidual<ElementResidual_, ElementCompute_>;
  using GammaBroadcast = builder::RowBroadcast<0, TileShape_, ElementGamma_, ElementCompute_>;
  using OutputTree = builder::Mul<builder::Acc, GammaBroadcast, ElementD_, ElementCompute_>;
  using AuxOutTree = builder::EVT<builder::AuxStore<ElementD_, StrideAux>, builder::Acc>;
  using EVT = builder::DualOutput<InputTree, OutputTree, ElementD_>;

  static typename EVT::Arguments make_evt_args(ElementResidual const* residual_ptr, StrideAux stride_residual,
                                               ElementGamma const* gamma_ptr, int N,
                                               ElementD_* aux_ptr, StrideAux stride_aux) {
    typename builder::AuxLoad<ElementResidual_>::Arguments res;
    res.ptr_aux = residual_ptr;
    res.null_default = ElementResidual(0);
    res.dAux = stride_residual;
    typename InputTree::Arguments input{typename builder::Acc::Arguments{}, res,
                                        typename builder::AddOp<ElementCompute_, ElementCompute_>::Arguments{}};
    typename builder::AuxStore<ElementD_, StrideAux>::Arguments store;
    store.ptr_aux = aux_ptr;
    store.null_default = ElementD_(0);
    store.dAux = stride_aux;
    typename AuxOutTree::Arguments aux{typename builder::Acc::Arguments{}, store};
    typename GammaBroadcast::Arguments gamma;
    gamma.ptr_row = gamma_ptr;
    gamma.null_default = ElementGamma(1);
    gamma.dRow = {cute::Int<0>{}, cute::Int<1>{}, static_cast<int64_t>(N)};
    typename OutputTree::Arguments output{typename builder::Acc::Arguments{}, gamma,
                                          typename builder::MulOp<ElementD_, ElementCompute_>::Arguments{}};
    return {input, aux, output};
  }
};

}  // namespace xe_fuse
