// Row-reduction producers of the per-row vectors the fused epilogues consume:
//   launch_compute_rstd               R[m] = 1 / sqrt(mean_n x[m,n]^2 + eps)
//   launch_compute_rstd_and_quantize  RMS-normalise a row and quantise it to int8 with a per-token
//                                     absmax scale that absorbs the RMS factor
// Same names and argument order as the reference's kernels/compute_rstd.hpp:12-125; the queue
// argument is the default CUDA stream.
#pragma once
#include <type_traits>

#include "sycl_common.hpp"
#include "xefuse/frontend.hpp"

namespace xe_fuse {

template <typename ElementInput, typename ElementOutput = float>
void launch_compute_rstd(sycl::queue&, ElementInput const* input_ptr, ElementOutput* rstd_ptr, int M, int N,
                         int L, float eps = 1e-6f) {
  static_assert(std::is_same<ElementInput, cutlass::bfloat16_t>::value && std::is_same<ElementOutput, float>::value,
                "bf16 rows in, fp32 factors out");
  if (xf_compute_rstd(input_ptr, rstd_ptr, M, N, L, eps, nullptr) != XF_SUCCESS)
    std::fprintf(stderr, "launch_compute_rstd: %s\n", xf_last_error_string());
}

template <typename ElementInput>
void launch_compute_rstd_and_quantize(sycl::queue&, ElementInput const* input_ptr, int8_t* quant_out_ptr,
                                      float* scale_token_ptr, int M, int N, int L, float eps = 1e-6f) {
  static_assert(std::is_same<ElementInput, cutlass::bfloat16_t>::value, "bf16 rows in");
  if (xf_compute_rstd_and_quantize(input_ptr, quant_out_ptr, scale_token_ptr, M, N, L, eps, nullptr) != XF_SUCCESS)
    std::fprintf(stderr, "launch_compute_rstd_and_quantize: %s\n", xf_last_error_string());
}

}  // namespace xe_fuse
