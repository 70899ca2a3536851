// xe_fuse::standalone -- the unfused elementwise passes (bf16 [L][M][N], in place) that the fused
// epilogues are benchmarked against.  Same function names and argument order as the reference's
// standalone/ops.hpp:32-354; each call enqueues one vectorised HBM-bound kernel of the library on
// the default stream.
#pragma once
#include "sycl_common.hpp"
#include "xefuse/frontend.hpp"

namespace xe_fuse::standalone {

using bf16 = cutlass::bfloat16_t;

inline void check_(xf_status s, const char* what) {
  if (s != XF_SUCCESS) std::fprintf(stderr, "standalone::%s: %s\n", what, xf_last_error_string());
}

inline void scale_rows(sycl::queue&, bf16* data, float const* scale, int M, int N, int L) {
  check_(xf_sa_scale_rows(data, scale, M, N, L, nullptr), "scale_rows");
}
inline void scale_cols(sycl::queue&, bf16* data, float const* gamma, int M, int N, int L) {
  check_(xf_sa_scale_cols(data, gamma, M, N, L, nullptr), "scale_cols");
}
inline void add_residual(sycl::queue&, bf16* data, bf16 const* residual, int M, int N, int L) {
  check_(xf_sa_add_residual(data, residual, M, N, L, nullptr), "add_residual");
}
inline void residual_gamma(sycl::queue&, bf16* data, bf16 const* residual, float const* gamma, int M, int N, int L) {
  check_(xf_sa_residual_gamma(data, residual, gamma, M, N, L, nullptr), "residual_gamma");
}
inline void swiglu(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_swiglu(data, M, N, L, nullptr), "swiglu");
}
inline void geglu(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_geglu(data, M, N, L, nullptr), "geglu");
}
// data <- rope(tmp): tmp is a read-only copy of the values to rotate
inline void rope(sycl::queue&, bf16* data, bf16 const* tmp, float const* cos_sin, int M, int N, int L) {
  check_(xf_sa_rope(data, tmp, cos_sin, M, N, L, nullptr), "rope");
}
inline void rope_scaled(sycl::queue&, bf16* data, bf16 const* tmp, float const* scale, float const* cos_sin,
                        int M, int N, int L) {
  check_(xf_sa_rope_scaled(data, tmp, scale, cos_sin, M, N, L, nullptr), "rope_scaled");
}
inline void gelu(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_unary(data, XF_UNARY_GELU, M, N, L, nullptr), "gelu");
}
inline void gelu_tanh(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_unary(data, XF_UNARY_GELU_TANH, M, N, L, nullptr), "gelu_tanh");
}
inline void silu(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_unary(data, XF_UNARY_SILU, M, N, L, nullptr), "silu");
}
inline void relu(sycl::queue&, bf16* data, int M, int N, int L) {
  check_(xf_sa_unary(data, XF_UNARY_RELU, M, N, L, nullptr), "relu");
}
inline void bias_add(sycl::queue&, bf16* data, float const* bias, int M, int N, int L) {
  check_(xf_sa_bias_add(data, bias, M, N, L, nullptr), "bias_add");
}
inline void compute_rstd(sycl::queue&, float* rstd, bf16 const* input, int M, int N, int L, float eps = 1e-6f) {
  check_(xf_compute_rstd(input, rstd, M, N, L, eps, nullptr), "compute_rstd");
}
inline void dequant_w8a8(sycl::queue&, bf16* out, int32_t const* acc, float const* scale_token,
                         float const* scale_channel, int M, int N, int L) {
  check_(xf_sa_dequant_w8a8(out, acc, scale_token, scale_channel, M, N, L, nullptr), "dequant_w8a8");
}

}  // namespace xe_fuse::standalone
