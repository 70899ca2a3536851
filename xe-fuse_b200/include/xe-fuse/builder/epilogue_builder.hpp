// xe_fuse::builder -- readable aliases for composing a GEMM epilogue and MakeGemm, which bundles
// an epilogue tree with element types into a ready-to-run Gemm type.
//
// Same alias names, template parameters and Arguments nesting as the reference's
// include/xe-fuse/builder/epilogue_builder.hpp:51-384, so code written against it compiles
// unchanged; the types are this project's and lower to the sm_100a kernels (xefuse/frontend.hpp).
//
//   namespace b = xe_fuse::builder;
//   using EVT  = b::SwiGLU<b::ScaleRows<b::Acc, TileShape, float>>;      // silu(g*R[m]) * (u*R[m])
//   using Gemm = b::MakeGemm<EVT, bf16, bf16, bf16, float, float, TileShape>::Gemm;
#pragma once

#include "xefuse/frontend.hpp"
#include "xe-fuse/visitors/xe_elementwise_compute.hpp"
#include "xe-fuse/visitors/xe_hadamard_compute.hpp"
#include "xe-fuse/visitors/xe_pairwise_compute.hpp"
#include "xe-fuse/visitors/xe_rope_compute.hpp"
#include "xe-fuse/visitors/xe_scalerows_compute.hpp"

namespace xe_fuse::builder {

namespace fusion = cutlass::epilogue::fusion;
using PackedMN = cute::Stride<int64_t, cute::Int<1>, int64_t>;   // full [M,N] tensor, N contiguous

// ---- sources ------------------------------------------------------------------------------
using Acc = fusion::XeAccFetch;                                    // the accumulator

template <typename Element, typename Stride = PackedMN, int VecWidth = 128 / cutlass::sizeof_bits_v<Element>>
using AuxLoad = fusion::XeAuxLoad<Element, Stride, void, VecWidth, true, true>;      // t[m,n]

// v[m]: one value per output row, the same for every column.  Idx is accepted and ignored.
template <int Idx, typename TileShape, typename Element, typename ElementCompute = float,
          int VecWidth = 128 / cutlass::sizeof_bits_v<Element>>
using ColBroadcast = fusion::XeColBroadcast<0, TileShape, Element, ElementCompute,
                                            cute::Stride<cute::Int<1>, cute::Int<0>, int64_t>, VecWidth>;

// v[n]: one value per output column, the same for every row.
template <int Idx, typename TileShape, typename Element, typename ElementCompute = float,
          int VecWidth = 128 / cutlass::sizeof_bits_v<Element>>
using RowBroadcast = fusion::XeRowBroadcast<0, TileShape, Element, ElementCompute,
                                            cute::Stride<cute::Int<0>, cute::Int<1>, int64_t>, VecWidth>;

// ---- binary ops ---------------------------------------------------------------------------
template <typename ElementOut = float, typename ElementCompute = float>
using MulOp = fusion::XeCompute<cutlass::multiplies, ElementOut, ElementCompute,
                                cutlass::FloatRoundStyle::round_to_nearest>;
template <typename ElementOut = float, typename ElementCompute = float>
using AddOp = fusion::XeCompute<cutlass::plus, ElementOut, ElementCompute,
                                cutlass::FloatRoundStyle::round_to_nearest>;

template <typename Op, typename... Children>
using EVT = fusion::XeEVT<Op, Children...>;

template <typename A, typename B, typename ElementOut = float, typename ElementCompute = float>
using Mul = EVT<MulOp<ElementOut, ElementCompute>, A, B>;
template <typename A, typename B, typename ElementOut = float, typename ElementCompute = float>
using Add = EVT<AddOp<ElementOut, ElementCompute>, A, B>;

// ---- compound aliases ---------------------------------------------------------------------
template <typename Input, typename TileShape, typename ElementScale = float, typename ElementCompute = float>
using ScaleRows = Mul<Input, ColBroadcast<0, TileShape, ElementScale, ElementCompute>,
                      ElementCompute, ElementCompute>;                 // in * R[m]

template <typename Input, typename TileShape, typename ElementScale = float, typename ElementCompute = float>
using ScaleCols = Mul<RowBroadcast<0, TileShape, ElementScale, ElementCompute>, Input,
                      ElementCompute, ElementCompute>;                 // gamma[n] * in

template <typename ElementResidual = cutlass::bfloat16_t, typename ElementCompute = float>
using AddResidual = Add<Acc, AuxLoad<ElementResidual>, ElementCompute, ElementCompute>;   // acc + res[m,n]

template <typename TileShape, typename ElementBias = float, typename ElementCompute = float>
using BiasAdd = Add<Acc, RowBroadcast<0, TileShape, ElementBias, ElementCompute>,
                    ElementCompute, ElementCompute>;                   // acc + b[n]

// ---- pair ops -----------------------------------------------------------------------------
template <typename PairwiseFn, typename Input>
using Pairwise = EVT<XePairwiseCompute<PairwiseFn>, Input>;
template <typename Input> using SwiGLU = Pairwise<SwiGLUFn, Input>;
template <typename Input> using GeGLU = Pairwise<GeGLUFn, Input>;

// ---- RoPE ---------------------------------------------------------------------------------
template <typename ElementCosSin = float>
using RoPE = EVT<XeRoPECompute, AuxLoad<ElementCosSin>>;
template <typename Input, typename ElementCosSin = float>
using RoPEComposed = EVT<XeRoPEComputeTwoChild, Input, AuxLoad<ElementCosSin>>;
template <typename TileShape, typename ElementScale = float, typename ElementCosSin = float>
using RoPEScaled = EVT<XeRoPEScaledCompute, ColBroadcast<0, TileShape, ElementScale>, AuxLoad<ElementCosSin>>;

// ---- merged nodes -------------------------------------------------------------------------
template <typename TileShape, typename ElementScale = float>
using ScaleRowsMerged = EVT<XeScaleRowsCompute, ColBroadcast<0, TileShape, ElementScale>>;
template <typename TileShape, typename ElementScale = float>
using SwiGLUScaled = EVT<XeScaleRowsSwiGLUCompute, ColBroadcast<0, TileShape, ElementScale>>;
template <typename TileShape, typename ElementScale = float>
using GeGLUScaled = EVT<XeScaleRowsGeGLUCompute, ColBroadcast<0, TileShape, ElementScale>>;

// ---- unary activations --------------------------------------------------------------------
template <typename Input> using GeLU = EVT<XeElementwiseCompute<GeLUFn>, Input>;
template <typename Input> using GeLUTanh = EVT<XeElementwiseCompute<GeLUTanhFn>, Input>;
template <typename Input> using SiLU = EVT<XeElementwiseCompute<SiLUFn>, Input>;
template <typename Input> using ReLU = EVT<XeElementwiseCompute<ReLUFn>, Input>;
template <typename Input> using Sigmoid = EVT<XeElementwiseCompute<SigmoidFn>, Input>;

// ---- W8A8 dequantisation ------------------------------------------------------------------
// int32 acc * scale_token[m] * scale_channel[n] (+ bias[n]); the product order is (acc*st)*sc.
template <typename TileShape, typename ElementScale = float, typename ElementCompute = float>
using DequantW8A8 = Mul<Mul<Acc, ColBroadcast<0, TileShape, ElementScale, ElementCompute>,
                            ElementCompute, ElementCompute>,
                        RowBroadcast<1, TileShape, ElementScale, ElementCompute>,
                        ElementCompute, ElementCompute>;

template <typename TileShape, typename ElementScale = float, typename ElementBias = float,
          typename ElementCompute = float>
using DequantW8A8Biased = Add<DequantW8A8<TileShape, ElementScale, ElementCompute>,
                              RowBroadcast<2, TileShape, ElementBias, ElementCompute>,
                              ElementCompute, ElementCompute>;

template <typename TileShape, typename ElementScale = float, typename ElementCosSin = float,
          typename ElementCompute = float>
using DequantRoPE = RoPEComposed<DequantW8A8<TileShape, ElementScale, ElementCompute>, ElementCosSin>;
template <typename TileShape, typename ElementScale = float, typename ElementCompute = float>
using DequantSwiGLU = SwiGLU<DequantW8A8<TileShape, ElementScale, ElementCompute>>;
template <typename TileShape, typename ElementScale = float, typename ElementCompute = float>
using DequantGeGLU = GeGLU<DequantW8A8<TileShape, ElementScale, ElementCompute>>;

template <typename InnerEVT, int GroupSize = 16>
using HadamardOutput = EVT<XeHadamardCompute<GroupSize>, InnerEVT>;   // refused at can_implement()

// ---- second output ------------------------------------------------------------------------
template <typename Element, typename Stride = PackedMN, int VecWidth = 128 / cutlass::sizeof_bits_v<Element>>
using AuxStore = fusion::XeAuxStore<Element, Stride, void, VecWidth, true, false>;

// Evaluate InputTree once; store it to an aux buffer; OutputTree (written over `Acc`) makes D.
template <typename InputTree, typename OutputTree, typename AuxElement = cutlass::bfloat16_t,
          typename AuxStride = PackedMN>
using DualOutput = fusion::Sm90SplitTreeVisitor<InputTree, OutputTree, EVT<AuxStore<AuxElement, AuxStride>, Acc>>;

// ---- MakeGemm -----------------------------------------------------------------------------
template <typename EVT_, typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementAcc_ = float,
          typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>,
          typename LayoutA_ = cutlass::layout::RowMajor, typename LayoutB_ = cutlass::layout::RowMajor,
          int AlignmentAB_ = 8, int AlignmentCD_ = 8>
struct MakeGemm {
  using EVT = EVT_;
  using ElementA = ElementA_;
  using ElementB = ElementB_;
  using ElementD = ElementD_;
  using ElementAcc = ElementAcc_;
  using ElementCompute = ElementCompute_;
  using TileShape = TileShape_;
  using LayoutA = LayoutA_;
  using LayoutB = LayoutB_;
  using StrideC = PackedMN;
  using StrideD = PackedMN;
  static constexpr int AlignmentAB = AlignmentAB_;
  static constexpr int AlignmentCD = AlignmentCD_;

  using ClusterShape = cute::Shape<cute::_1, cute::_1, cute::_1>;
  using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape,
      cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementCompute,
      ElementD, StrideC, AlignmentCD_, ElementD, StrideD, AlignmentCD_,
      cutlass::epilogue::collective::EpilogueScheduleAuto, EVT>::CollectiveOp;
  using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, ElementA, LayoutA, AlignmentAB_,
      ElementB, LayoutB, AlignmentAB_, ElementAcc, TileShape, ClusterShape,
      cutlass::gemm::collective::StageCountAuto, cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
  using GemmKernel = cutlass::gemm::kernel::GemmUniversal<cute::Shape<int, int, int, int>,
                                                          CollectiveMainloop, CollectiveEpilogue>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;
};

}  // namespace xe_fuse::builder
