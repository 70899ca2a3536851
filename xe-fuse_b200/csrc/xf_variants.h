// The tile variants of the fused GEMM kernel, in the order every table indexed by variant uses, and
// the epilogue classes each variant is compiled for.
//
//   X(KIND, BN, CTAS, KS, KC, NAME)
//   KIND 0 = bf16 x bf16 -> fp32, 1 = int8 x int8 -> int32; BN = tile columns; CTAS = CTAs per MMA;
//   KS = 128-byte K slabs per pipeline stage; KC = K groups per cluster (cluster split-K)
//   name = <dtype>_<tile rows>x<columns>_cta<CTAs per MMA>_k<K elements per stage>[_kc<K groups per cluster>]
#pragma once

#define XF_FOR_EACH_VARIANT(X)                    \
  X(0, 256, 2, 1, 1, "bf16_256x256_cta2_k64")     \
  X(0, 256, 2, 2, 1, "bf16_256x256_cta2_k128")    \
  X(0, 256, 1, 1, 1, "bf16_128x256_cta1_k64")     \
  X(0, 128, 2, 1, 1, "bf16_256x128_cta2_k64")     \
  X(0, 128, 2, 2, 1, "bf16_256x128_cta2_k128")    \
  X(0, 128, 1, 1, 1, "bf16_128x128_cta1_k64")     \
  X(0, 128, 1, 2, 1, "bf16_128x128_cta1_k128")    \
  X(0, 256, 2, 2, 2, "bf16_256x256_cta2_k128_kc2") \
  X(1, 256, 2, 1, 1, "s8_256x256_cta2_k128")      \
  X(1, 256, 2, 2, 1, "s8_256x256_cta2_k256")      \
  X(1, 256, 1, 1, 1, "s8_128x256_cta1_k128")      \
  X(1, 128, 1, 1, 1, "s8_128x128_cta1_k128")      \
  X(1, 128, 1, 2, 1, "s8_128x128_cta1_k256")      \
  X(1, 256, 2, 2, 2, "s8_256x256_cta2_k256_kc2")

namespace xf {

struct GemmParams;
typedef void (*KernelFn)(const GemmParams);

// Epilogue classes: which feature mask (EF_* of the kernel header) a kernel instance is compiled
// with.  One table of kernels per class, defined in xf_gemm_class_<name>.cu, indexed by variant.
enum : int { EC_SCALE = 0, EC_MAT = 1, EC_GLU = 2, EC_ROPE = 3, EC_ALL = 4, EC_COUNT = 5 };
extern const KernelFn g_kernels_scale[];   // row / column scales and bias only (k1, w8a8 dequant)
extern const KernelFn g_kernels_mat[];     // + residual and auxiliary output (k0a, dual output)
extern const KernelFn g_kernels_glu[];     // + SwiGLU / GeGLU (k2)
extern const KernelFn g_kernels_rope[];    // + RoPE (k3, k4, k4v2)
extern const KernelFn g_kernels_all[];     // every step of the flat program

}  // namespace xf
