// Host-only check of the front end's lowering: prints, for each epilogue tree the presets use, the
// flat program it lowers to (one line per tree) and the status can_implement() returns.  No GPU.
#include <cstdio>
#include <string>

#include "cutlass/util/packed_stride.hpp"
#include "xe-fuse/builder/epilogue_builder.hpp"
#include "xe-fuse/kernels/gemm_dequant_rope.hpp"
#include "xe-fuse/kernels/gemm_dequant_swiglu.hpp"
#include "xe-fuse/kernels/gemm_dequant_w8a8.hpp"
#include "xe-fuse/kernels/gemm_dual_output.hpp"
#include "xe-fuse/kernels/gemm_residual_gamma.hpp"
#include "xe-fuse/kernels/gemm_residual_gamma_colred.hpp"
#include "xe-fuse/kernels/gemm_rmsnorm.hpp"
#include "xe-fuse/kernels/gemm_rmsnorm_rope.hpp"
#include "xe-fuse/kernels/gemm_rmsnorm_swiglu.hpp"
#include "xe-fuse/kernels/gemm_rope.hpp"
#include "xe-fuse/kernels/gemm_swiglu.hpp"

using namespace cute;
namespace b = xe_fuse::builder;
using bf16 = cutlass::bfloat16_t;
using TS = Shape<_256, _256, _32>;

static const int M = 256, N = 512, K = 128, L = 1;
static float* const kRow = reinterpret_cast<float*>(0x1000);
static float* const kCol = reinterpret_cast<float*>(0x2000);
static float* const kBias = reinterpret_cast<float*>(0x3000);
static float* const kCs = reinterpret_cast<float*>(0x4000);
static bf16* const kRes = reinterpret_cast<bf16*>(0x5000);
static bf16* const kAux = reinterpret_cast<bf16*>(0x6000);

template <class Kt, class EvtArgs>
static void show(const char* name, EvtArgs const& ea, xefuse::Extensions ext = {}, const void* ptr_c = nullptr) {
  using Op = typename Kt::Gemm;
  using Kernel = typename Op::GemmKernel;
  auto sA = cutlass::make_cute_packed_stride(typename Kernel::StrideA{}, make_shape(M, K, L));
  auto sB = cutlass::make_cute_packed_stride(typename Kernel::StrideB{}, make_shape(N, K, L));
  auto sD = cutlass::make_cute_packed_stride(b::PackedMN{}, make_shape(M, N, L));
  typename Kernel::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm, {M, N, K, L},
                                  {reinterpret_cast<typename Kernel::ElementA*>(0x10000), sA,
                                   reinterpret_cast<typename Kernel::ElementB*>(0x20000), sB},
                                  {ea, static_cast<typename Kernel::ElementC const*>(ptr_c), sD,
                                   reinterpret_cast<typename Kernel::ElementD*>(0x30000), sD}, {}};
  xf_gemm_desc d;
  cutlass::Status ls = Op::lower(args, ext, d);
  cutlass::Status cs = Op::can_implement(args, ext);
  auto at = [](const void* p) { return (unsigned)(reinterpret_cast<uintptr_t>(p)); };
  std::printf("%s lower=%d can=%d ab=%d d=%d lda=%lld ldb=%lld ldd=%lld tile=%d,%d,%d res=%d@%x aux=%d@%x "
              "row=%d@%x/%g col=%d@%x bias=%d@%x unary=%d pair=%d cs=%x period=%d layout=%d sumsq=%x\n",
              name, int(ls), int(cs), d.dtype_ab, d.dtype_d, (long long)d.lda, (long long)d.ldb, (long long)d.ldd,
              d.tile_m, d.tile_n, d.tile_k, d.epi.residual.enabled, at(d.epi.residual.ptr), d.epi.aux_store.enabled,
              at(d.epi.aux_store.ptr), d.epi.row_scale.enabled, at(d.epi.row_scale.ptr), d.epi.row_scale.null_default,
              d.epi.col_scale.enabled, at(d.epi.col_scale.ptr), d.epi.bias.enabled, at(d.epi.bias.ptr), d.epi.unary,
              d.epi.pair, at(d.epi.cos_sin.ptr), d.epi.cos_sin_period, d.epi.out_layout, at(d.epi.row_sumsq));
}

template <class EVT, class EA = bf16, class EAcc = float>
using Mk = b::MakeGemm<EVT, EA, EA, bf16, EAcc, float, TS>;

int main() {
  auto sMN = cutlass::make_cute_packed_stride(b::PackedMN{}, make_shape(M, N, L));
  typename b::ColBroadcast<0, TS, float>::Arguments row;
  row.ptr_col = kRow; row.null_default = 1.f; row.dCol = {Int<1>{}, Int<0>{}, int64_t(M)};
  typename b::RowBroadcast<0, TS, float>::Arguments col;
  col.ptr_row = kCol; col.null_default = 1.f; col.dRow = {Int<0>{}, Int<1>{}, int64_t(N)};
  typename b::RowBroadcast<0, TS, float>::Arguments bias;
  bias.ptr_row = kBias; bias.null_default = 0.f; bias.dRow = {Int<0>{}, Int<1>{}, int64_t(N)};
  typename b::AuxLoad<float>::Arguments cs;
  cs.ptr_aux = kCs; cs.dAux = sMN;
  b::Acc::Arguments acc;
  b::MulOp<>::Arguments mul;
  b::AddOp<>::Arguments add;

  show<xe_fuse::GemmRmsNorm<>>("k1", xe_fuse::GemmRmsNorm<>::make_evt_args(kRow, M));
  show<xe_fuse::GemmRmsNormSwiGLU<>>("k2", xe_fuse::GemmRmsNormSwiGLU<>::make_evt_args(kRow, M));
  {
    xefuse::Extensions e; e.compact_pair_output = true;
    show<xe_fuse::GemmRmsNormSwiGLU<>>("k2_compact", xe_fuse::GemmRmsNormSwiGLU<>::make_evt_args(kRow, M), e);
  }
  show<xe_fuse::GemmSwiGLU<>>("k8", xe_fuse::GemmSwiGLU<>::make_evt_args());
  show<xe_fuse::GemmRoPE<>>("k3", xe_fuse::GemmRoPE<>::make_evt_args(kCs, sMN));
  show<xe_fuse::GemmRmsNormRoPE<>>("k4", xe_fuse::GemmRmsNormRoPE<>::make_evt_args(kRow, M, kCs, sMN));
  {
    using EVT = b::RoPEScaled<TS, float, float>;
    typename EVT::Arguments ea{row, cs, xe_fuse::XeRoPEScaledCompute::Arguments{}};
    xefuse::Extensions e; e.cos_sin_period = 128;
    show<Mk<EVT>>("k4v2_table", ea, e);
  }
  show<xe_fuse::GemmResidualGamma<>>("k0a", xe_fuse::GemmResidualGamma<>::make_evt_args(kRes, sMN, kCol, N));
  {
    // K0a with the sum of squares folded in: the residual is the kernel's source tensor C
    using CR = xe_fuse::GemmResidualGammaColRed<>;
    float* const kSumSq = reinterpret_cast<float*>(0x7000);
    show<CR>("k0a_cr", CR::make_evt_args(kCol, N, kSumSq, M), {}, kRes);
    show<CR>("k0a_cr_null", CR::make_evt_args(kCol, N, nullptr, M), {}, kRes);    // reduction disabled
    show<CR>("bad_cr_no_source", CR::make_evt_args(kCol, N, kSumSq, M));           // SrcFetch without C
    show<xe_fuse::GemmRmsNorm<>>("bad_unused_source", xe_fuse::GemmRmsNorm<>::make_evt_args(kRow, M), {}, kRes);
  }
  show<xe_fuse::GemmDualOutput<>>("k0_dual", xe_fuse::GemmDualOutput<>::make_evt_args(kRes, sMN, kCol, N, kAux, sMN));
  show<xe_fuse::GemmDequantW8A8<>>("w8a8", xe_fuse::GemmDequantW8A8<>::make_evt_args(kRow, M, kCol, N));
  {
    using EVT = b::DequantW8A8Biased<TS, float, float, float>;
    typename b::RowBroadcast<2, TS, float>::Arguments b2;
    b2.ptr_row = kBias; b2.null_default = 0.f; b2.dRow = {Int<0>{}, Int<1>{}, int64_t(N)};
    typename EVT::Arguments ea{xe_fuse::GemmDequantW8A8<>::make_evt_args(kRow, M, kCol, N), b2, add};
    show<b::MakeGemm<EVT, int8_t, int8_t, bf16, int32_t, float, TS, cutlass::layout::RowMajor,
                     cutlass::layout::RowMajor, 32, 8>>("w8a8_biased", ea);
  }
  show<xe_fuse::GemmDequantRoPE<>>("w8a8_rope", xe_fuse::GemmDequantRoPE<>::make_evt_args(kRow, M, kCol, N, kCs, sMN));
  show<xe_fuse::GemmDequantSwiGLU<>>("w8a8_swiglu", xe_fuse::GemmDequantSwiGLU<>::make_evt_args(kRow, M, kCol, N));
  show<xe_fuse::GemmDequantGeGLU<>>("w8a8_geglu", xe_fuse::GemmDequantGeGLU<>::make_evt_args(kRow, M, kCol, N));
  {
    using EVT = b::GeLU<b::BiasAdd<TS, float>>;
    typename b::BiasAdd<TS, float>::Arguments inner{acc, bias, add};
    typename EVT::Arguments ea{inner, xe_fuse::XeElementwiseCompute<xe_fuse::GeLUFn>::Arguments{}};
    show<Mk<EVT>>("bias_gelu", ea);
  }
  {
    using EVT = b::SiLU<b::ScaleRows<b::Acc, TS, float>>;
    typename b::ScaleRows<b::Acc, TS, float>::Arguments inner{acc, row, mul};
    typename EVT::Arguments ea{inner, xe_fuse::XeElementwiseCompute<xe_fuse::SiLUFn>::Arguments{}};
    show<Mk<EVT>>("scale_silu", ea);
  }
  {  // null pointer in a broadcast => its null_default is used
    using EVT = b::ScaleRows<b::Acc, TS, float>;
    auto r0 = row; r0.ptr_col = nullptr; r0.null_default = 0.5f;
    typename EVT::Arguments ea{acc, r0, mul};
    show<Mk<EVT>>("null_row", ea);
  }
  {  // identity epilogue through the default fusion of the collective builder
    using Epi = cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, TS, Shape<_1, _1, _1>,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, bf16, b::PackedMN, 8, bf16, b::PackedMN, 8,
        cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
    using Main = cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Xe20, cutlass::arch::OpClassTensorOp, bf16, cutlass::layout::RowMajor, 8, bf16,
        cutlass::layout::RowMajor, 8, float, TS, Shape<_1, _1, _1>, cutlass::gemm::collective::StageCountAuto,
        cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
    struct Bare {
      using Gemm = cutlass::gemm::device::GemmUniversalAdapter<
          cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Main, Epi>>;
    };
    show<Bare>("bare", typename Epi::FusionCallbacks::Arguments{1.0f, 0.0f});
    show<Bare>("bare_alpha2", typename Epi::FusionCallbacks::Arguments{2.0f, 0.0f});
    show<Bare>("bad_beta", typename Epi::FusionCallbacks::Arguments{1.0f, 1.0f});
  }
  // ---- trees outside the flat program are refused
  {
    using EVT = b::ScaleCols<b::GeLU<b::Acc>, TS, float>;   // gamma[n] after the activation
    typename b::GeLU<b::Acc>::Arguments inner{acc, xe_fuse::XeElementwiseCompute<xe_fuse::GeLUFn>::Arguments{}};
    typename EVT::Arguments ea{col, inner, mul};
    show<Mk<EVT>>("bad_scale_after_unary", ea);
  }
  {
    using EVT = b::Add<b::ScaleRows<b::Acc, TS, float>, b::AuxLoad<bf16>>;   // residual after the row scale
    typename b::AuxLoad<bf16>::Arguments res;
    res.ptr_aux = kRes; res.dAux = sMN;
    typename b::ScaleRows<b::Acc, TS, float>::Arguments inner{acc, row, mul};
    typename EVT::Arguments ea{inner, res, add};
    show<Mk<EVT>>("bad_residual_after_scale", ea);
  }
  {
    using EVT = b::HadamardOutput<b::DequantW8A8<TS, float, float>, 16>;
    typename EVT::Arguments ea{xe_fuse::GemmDequantW8A8<>::make_evt_args(kRow, M, kCol, N),
                               xe_fuse::XeHadamardCompute<16>::Arguments{}};
    show<b::MakeGemm<EVT, int8_t, int8_t, bf16, int32_t, float, TS>>("bad_hadamard", ea);
  }
  {
    using EVT = b::Mul<b::Acc, b::Acc>;   // the accumulator twice
    typename EVT::Arguments ea{acc, acc, mul};
    show<Mk<EVT>>("bad_acc_twice", ea);
  }
  return 0;
}
