// cutlass::reference::device::GemmComplex: the naive device GEMM harness mains use to rebuild the
// expected accumulator.  D = alpha * A * B + beta * C per batch, A [M,K] and B [K,N] row-major,
// accumulation in ElementAcc precision.  Runs the library's reference kernel (one thread per
// output element, sequential k): slow and simple on purpose.
#pragma once
#include "xefuse/frontend.hpp"

namespace cutlass::reference::device {

template <class EA, class LA, class EB, class LB, class EC, class LC, class ED, class LD, class Scalar>
void GemmComplex(gemm::GemmCoord problem, Scalar alpha, TensorRef<EA, LA> A, ComplexTransform,
                 TensorRef<EB, LB> B, ComplexTransform, Scalar beta, TensorRef<EC, LC> C,
                 TensorRef<ED, LD> D, Scalar /*initial_accum*/, int batch_count = 1,
                 int64_t batch_stride_A = 0, int64_t batch_stride_B = 0, int64_t batch_stride_C = 0,
                 int64_t batch_stride_D = 0) {
  static_assert(std::is_same<LA, layout::RowMajor>::value && std::is_same<LB, layout::RowMajor>::value &&
                std::is_same<LD, layout::RowMajor>::value, "row-major operands only");
  using AE = std::remove_const_t<EA>;
  using BE = std::remove_const_t<EB>;
  xf_status s = xf_harness_ref_gemm(
      xefuse::DType<AE>::value, A.data(), A.stride(0), batch_stride_A, xefuse::DType<BE>::value, B.data(),
      B.stride(0), batch_stride_B, xefuse::DType<std::remove_const_t<EC>>::value, C.data(), C.stride(0),
      batch_stride_C, xefuse::DType<ED>::value, D.data(), D.stride(0), batch_stride_D, problem.m(),
      problem.n(), problem.k(), batch_count, float(alpha), float(beta), nullptr);
  if (s != XF_SUCCESS) std::fprintf(stderr, "GemmComplex: %s\n", xf_last_error_string());
}

}  // namespace cutlass::reference::device
