// Kernel instances of the fused GEMM for one epilogue class (feature mask 0): every tile variant.
#include "xf_gemm_kernel.cuh"
#include "xf_variants.h"

namespace xf {

#define XF_INSTANCE(KIND, BN, CTAS, KS, KC, NAME) gemm_evt_kernel<KIND, BN, CTAS, KS, KC, 0>,
const KernelFn g_kernels_scale[] = {XF_FOR_EACH_VARIANT(XF_INSTANCE)};
#undef XF_INSTANCE

}  // namespace xf
