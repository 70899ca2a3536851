// Kernel instances of the fused GEMM for one epilogue class (feature mask EF_MAT): every tile variant.
#include "xf_gemm_kernel.cuh"
#include "xf_variants.h"

namespace xf {

#define XF_INSTANCE(KIND, BN, CTAS, KS, KC, NAME) gemm_evt_kernel<KIND, BN, CTAS, KS, KC, EF_MAT>,
const KernelFn g_kernels_mat[] = {XF_FOR_EACH_VARIANT(XF_INSTANCE)};
#undef XF_INSTANCE

}  // namespace xf
