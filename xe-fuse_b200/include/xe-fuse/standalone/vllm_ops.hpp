// xe_fuse::vllm_equiv -- the engine-style stand-alone passes the reference's generated pipelines
// time as their "bare GEMM + fused stand-alone kernels" arm.  Same function names, argument order
// and defaults as the reference's standalone/vllm_ops.hpp:33-346; each call enqueues one HBM-bound
// kernel of the library (xf_ve_*) on the default stream.
#pragma once
#include <cstdint>

#include "sycl_common.hpp"
#include "xefuse/frontend.hpp"

namespace xe_fuse::vllm_equiv {

using bf16 = cutlass::bfloat16_t;

inline void check_(xf_status s, const char* what) {
  if (s != XF_SUCCESS) std::fprintf(stderr, "vllm_equiv::%s: %s\n", what, xf_last_error_string());
}

// out[m,n] = input[m,n] * rsqrt(mean(input[m,:]^2) + eps) * weight[n]; out may be input
inline void rms_norm(sycl::queue&, bf16* out, bf16 const* input, bf16 const* weight, int M, int N,
                     float eps = 1e-6f) {
  check_(xf_ve_rms_norm(out, input, weight, M, N, eps, nullptr), "rms_norm");
}

// residual += input; input = RMSNorm(residual) * weight (both in place)
inline void fused_add_rms_norm(sycl::queue&, bf16* input, bf16* residual, bf16 const* weight, int M, int N,
                               float eps = 1e-6f) {
  check_(xf_ve_fused_add_rms_norm(input, residual, weight, M, N, eps, nullptr), "fused_add_rms_norm");
}

// out[m,i] = silu(input[m,i]) * input[m,d+i]; input [M,2d], out [M,d]
inline void silu_and_mul(sycl::queue&, bf16* out, bf16 const* input, int d, int M) {
  check_(xf_ve_act_and_mul(out, input, d, M, 0, nullptr), "silu_and_mul");
}

// out[m,i] = gelu(input[m,i]) * input[m,d+i]
inline void gelu_and_mul(sycl::queue&, bf16* out, bf16 const* input, int d, int M) {
  check_(xf_ve_act_and_mul(out, input, d, M, 1, nullptr), "gelu_and_mul");
}

// NeoX-style rotary embedding in place; key may be nullptr
inline void rotary_embedding(sycl::queue&, bf16* query, bf16* key, float const* cos_sin_cache, int head_size,
                             int num_heads, int num_kv_heads, int rot_dim, int M) {
  check_(xf_ve_rotary_embedding(query, key, cos_sin_cache, head_size, num_heads, num_kv_heads, rot_dim, M,
                                nullptr),
         "rotary_embedding");
}

// int32 accumulator [L,M,2d] -> bf16 [L,M,2d], dequantise + SwiGLU over the halves (result in both)
inline void dequant_and_silu_mul(sycl::queue&, bf16* out, int32_t const* acc, float const* scale_token,
                                 float const* scale_channel, int d, int M, int L = 1) {
  check_(xf_ve_dequant_act_mul(out, acc, scale_token, scale_channel, d, M, L, 0, nullptr),
         "dequant_and_silu_mul");
}

inline void dequant_and_gelu_mul(sycl::queue&, bf16* out, int32_t const* acc, float const* scale_token,
                                 float const* scale_channel, int d, int M, int L = 1) {
  check_(xf_ve_dequant_act_mul(out, acc, scale_token, scale_channel, d, M, L, 1, nullptr),
         "dequant_and_gelu_mul");
}

// int32 accumulator [L,M,N] -> bf16, dequantise + interleaved-pair rotation, cos_sin [L,M,N] fp32
inline void dequant_and_rotary_embedding(sycl::queue&, bf16* out, int32_t const* acc, float const* scale_token,
                                         float const* scale_channel, float const* cos_sin_cache, int M, int N,
                                         int L = 1) {
  check_(xf_ve_dequant_rotary(out, acc, scale_token, scale_channel, cos_sin_cache, M, N, L, nullptr),
         "dequant_and_rotary_embedding");
}

}  // namespace xe_fuse::vllm_equiv
