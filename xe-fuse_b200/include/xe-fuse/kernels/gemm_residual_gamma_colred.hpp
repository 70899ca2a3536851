// K0a_CR -- K0a with the sum of squares for the next RMSNorm folded into the GEMM epilogue:
//   D[m,n]  = gamma[n] * (acc[m,n] + residual[m,n])
//   sum_sq  = partial sums over N of D[m,n]^2 (the fp32 value before rounding), no atomics
// followed by launch_reduce_partials_rsqrt(), which reads the partials instead of the M x N output
// and writes rstd[M].  Same public members, make_evt_args signature and call sequence as the
// reference's kernels/gemm_residual_gamma_colred.hpp:33-226; the residual arrives as the kernel's
// source tensor C (ptr_C / stride_C), as there.
//
// What differs is invisible to a caller that sizes the buffer with get_partials_size(): the
// partials are kept per 32 output columns, [L][ceil(N/32)][M] floats, rather than per CTA tile.
#pragma once
#include "sycl_common.hpp"
#include "xe-fuse/builder/epilogue_builder.hpp"

namespace xe_fuse {

template <typename ElementA_ = cutlass::bfloat16_t, typename ElementB_ = cutlass::bfloat16_t,
          typename ElementD_ = cutlass::bfloat16_t, typename ElementResidual_ = cutlass::bfloat16_t,
          typename ElementGamma_ = float, typename ElementAcc_ = float, typename ElementCompute_ = float,
          typename TileShape_ = cute::Shape<cute::_256, cute::_256, cute::_32>>
struct GemmResidualGammaColRed {
  using ElementA = ElementA_;
  using ElementB = ElementB_;
  using ElementD = ElementD_;
  using ElementResidual = ElementResidual_;
  using ElementGamma = ElementGamma_;
  using ElementAcc = ElementAcc_;
  using ElementCompute = ElementCompute_;
  using TileShape = TileShape_;

  static constexpr int CTA_M = cute::size<0>(TileShape{});
  static constexpr int CTA_N = cute::size<1>(TileShape{});

  // Elements of the partial-sum buffer.  Every slot is overwritten once per GEMM: no pre-zeroing.
  static size_t get_partials_size(int M, int N, int L) { return xf_row_sumsq_count(M, N, L); }

  using LayoutA = cutlass::layout::RowMajor;
  using LayoutB = cutlass::layout::RowMajor;
  using StrideC = cute::Stride<int64_t, cute::Int<1>, int64_t>;
  using StrideD = cute::Stride<int64_t, cute::Int<1>, int64_t>;
  using StrideResidual = cute::Stride<int64_t, cute::Int<1>, int64_t>;

  using SrcFetch = cutlass::epilogue::fusion::Sm90SrcFetch<ElementResidual>;

  // gamma[n] * (acc + C)
  using AddTree = builder::EVT<builder::AddOp<ElementCompute, ElementCompute>, builder::Acc, SrcFetch>;
  using GammaBroadcast = builder::RowBroadcast<0, TileShape, ElementGamma, ElementCompute>;
  using InputTree = builder::EVT<builder::MulOp<ElementCompute, ElementCompute>, GammaBroadcast, AddTree>;

  // pass-through to the D store
  using IdentityOp = cutlass::epilogue::fusion::XeCompute<cutlass::epilogue::thread::Identity, ElementD,
                                                          ElementCompute, cutlass::FloatRoundStyle::round_to_nearest>;
  using OutputTree = builder::EVT<IdentityOp, builder::Acc>;

  // sum over N of the squared value, written as partials
  using SquaredInput = builder::Mul<builder::Acc, builder::Acc, ElementCompute, ElementCompute>;
  using ColRed = cutlass::epilogue::fusion::XeColReduction<
      cutlass::plus, cutlass::plus, cutlass::plus, 0, TileShape, ElementCompute, ElementCompute,
      cutlass::FloatRoundStyle::round_to_nearest, cute::Stride<cute::Int<1>, cute::Int<0>, int64_t>,
      128 / cutlass::sizeof_bits_v<ElementCompute>, true, false>;
  using ColRedTree = builder::EVT<ColRed, SquaredInput>;

  using EVT = cutlass::epilogue::fusion::Sm90SplitTreeVisitor<InputTree, OutputTree, ColRedTree>;

  using ClusterShape = cute::Shape<cute::_1, cute::_1, cute::_1>;
  using CollectiveEpilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
      cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape,
      cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementCompute, ElementResidual, StrideC, 8,
      ElementD, StrideD, 8, cutlass::epilogue::collective::EpilogueScheduleAuto, EVT>::CollectiveOp;
  using CollectiveMainloop = typename cutlass::gemm::collective::CollectiveBuilder<
      cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, ElementA, LayoutA, 8, ElementB, LayoutB, 8, ElementAcc,
      TileShape, ClusterShape, cutlass::gemm::collective::StageCountAuto,
      cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
  using GemmKernel =
      cutlass::gemm::kernel::GemmUniversal<cute::Shape<int, int, int, int>, CollectiveMainloop, CollectiveEpilogue>;
  using Gemm = cutlass::gemm::device::GemmUniversalAdapter<GemmKernel>;

  static typename EVT::Arguments make_evt_args(ElementGamma const* gamma_ptr, int N, ElementCompute* sum_sq_ptr,
                                               int M, int L = 1) {
    (void)L;
    typename AddTree::Arguments add{typename builder::Acc::Arguments{}, typename SrcFetch::Arguments{},
                                    typename builder::AddOp<ElementCompute, ElementCompute>::Arguments{}};
    typename GammaBroadcast::Arguments gamma;
    gamma.ptr_row = gamma_ptr;
    gamma.null_default = ElementGamma(1);
    gamma.dRow = {cute::Int<0>{}, cute::Int<1>{}, static_cast<int64_t>(N)};
    typename InputTree::Arguments input{gamma, add,
                                        typename builder::MulOp<ElementCompute, ElementCompute>::Arguments{}};

    typename OutputTree::Arguments output{typename builder::Acc::Arguments{}, typename IdentityOp::Arguments{}};

    typename SquaredInput::Arguments squared{typename builder::Acc::Arguments{}, typename builder::Acc::Arguments{},
                                             typename builder::MulOp<ElementCompute, ElementCompute>::Arguments{}};
    typename ColRed::Arguments red;
    red.ptr_col = sum_sq_ptr;
    red.reduction_identity = ElementCompute(0);
    red.dCol = {cute::Int<1>{}, cute::Int<0>{}, static_cast<int64_t>(M) * ((N + 31) / 32)};
    typename ColRedTree::Arguments col_red{squared, red};

    // split-tree order: input tree, auxiliary trees, output tree
    return typename EVT::Arguments{input, col_red, output};
  }
};

// partials (the sum_sq buffer of a K0a_CR launch) -> rstd[M * L].  The CTA tile extents are
// accepted for source compatibility; the partial layout does not depend on them.
template <int CTA_M_, int CTA_N_, typename ElementOutput = float>
void launch_reduce_partials_rsqrt(sycl::queue&, float const* partials_ptr, ElementOutput* rstd_ptr, int M, int N,
                                  int L, float eps = 1e-6f) {
  static_assert(std::is_same<ElementOutput, float>::value, "fp32 factors out");
  if (xf_reduce_partials_rsqrt(partials_ptr, rstd_ptr, M, N, L, eps, nullptr) != XF_SUCCESS)
    std::fprintf(stderr, "launch_reduce_partials_rsqrt: %s\n", xf_last_error_string());
}

}  // namespace xe_fuse
