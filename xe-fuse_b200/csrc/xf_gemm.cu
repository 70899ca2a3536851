// Host side of the fused GEMM: argument checks, kernel/tile selection, TMA tensor-map encoding,
// cluster launch.  Exposes the xf_gemm_* entry points declared in include/xefuse_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/xefuse_b200.h"
#include "xf_gemm_kernel.cuh"
#include "xf_host_util.h"
#include "xf_variants.h"

namespace xf {

// ---------------------------------------------------------------------------- error text
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

// ---------------------------------------------------------------------------- driver entry
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static bool encode_3d(CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t d0,
                      uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                      uint32_t b0, uint32_t b1, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (CUresult %d) dims={%llu,%llu,%llu} strides={%llu,%llu} box={%u,%u}",
              (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
              (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes, b0, b1);
    return false;
  }
  return true;
}

// ---------------------------------------------------------------------------- kernel table
// A variant fixes the tile; each is compiled once per epilogue class (xf_variants.h), and a plan
// launches the instance of the smallest class that covers its descriptor.
struct Variant {
  int kind, bn, ctas, ks, kc, stages, smem;
  const char* name;
};

#define XF_VARIANT(KIND, BN, CTAS, KS, KC, NAME)                                      \
  {KIND, BN, CTAS, KS, KC, TileCfg<KIND, BN, CTAS, KS, KC>::STAGES,                    \
   TileCfg<KIND, BN, CTAS, KS, KC>::SMEM_BYTES, NAME},

static const Variant g_variants[] = {XF_FOR_EACH_VARIANT(XF_VARIANT)};
#undef XF_VARIANT
static const KernelFn* const g_class_tables[EC_COUNT] = {g_kernels_scale, g_kernels_mat, g_kernels_glu,
                                                         g_kernels_rope, g_kernels_all};
static KernelFn kernel_of(const Variant& v, int epi_class) {
  return g_class_tables[epi_class][&v - g_variants];
}
static const int g_num_variants = sizeof(g_variants) / sizeof(g_variants[0]);

}  // namespace xf

struct xf_plan {
  xf::GemmParams params;
  const xf::Variant* variant;
  xf::KernelFn fn;         // the variant's instance for this plan's epilogue class
  int grid;
  int device;
  int no_pdl;   // 1: launch without programmatic stream serialization
  size_t workspace_used;   // bytes of the workspace the plan's kernel touches
  size_t clear_bytes;      // leading bytes (status word, split counters) that must be zero before a launch
  char name[64];
};

namespace xf {

static int elem_size(int dt) {
  switch (dt) {
    case XF_DT_BF16: return 2;
    case XF_DT_S8: return 1;
    default: return 4;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static xf_status check_vec(const xf_vec& v, const char* what) {
  if (!v.enabled) return XF_SUCCESS;
  if (v.dtype != XF_DT_F32 && v.dtype != XF_DT_BF16) {
    set_error("%s: vector dtype must be f32 or bf16", what);
    return XF_ERR_INVALID_DATA_TYPE;
  }
  return XF_SUCCESS;
}

static xf_status check_mat(const xf_mat& m, const char* what, int N, bool allow_bf16) {
  if (!m.enabled) return XF_SUCCESS;
  if (m.ptr == nullptr) {
    set_error("%s: null pointer", what);
    return XF_ERR_INVALID_PROBLEM;
  }
  if (!(m.dtype == XF_DT_F32 || (allow_bf16 && m.dtype == XF_DT_BF16))) {
    set_error("%s: unsupported dtype %d", what, m.dtype);
    return XF_ERR_INVALID_DATA_TYPE;
  }
  if (m.ld < N) {
    set_error("%s: row pitch %lld smaller than the %d columns read", what, (long long)m.ld, N);
    return XF_ERR_INVALID_LAYOUT;
  }
  return XF_SUCCESS;
}

static xf_status validate(const xf_gemm_desc* d) {
  if (!d) {
    set_error("null descriptor");
    return XF_ERR_INVALID_PROBLEM;
  }
  if (d->dtype_ab != XF_DT_BF16 && d->dtype_ab != XF_DT_S8) {
    set_error("A/B dtype must be bf16 or int8 (got %d)", d->dtype_ab);
    return XF_ERR_INVALID_DATA_TYPE;
  }
  if (d->flags & XF_FLAG_DIAG_MASK) {
    const char* allow = getenv("XEFUSE_ALLOW_DIAG");
    if (!allow || allow[0] != '1') {
      set_error("the XF_FLAG_DIAG_* flags make D garbage; they are honoured only with XEFUSE_ALLOW_DIAG=1 "
                "in the environment");
      return XF_ERR_NOT_SUPPORTED;
    }
  }
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->L <= 0) {
    set_error("problem extents must be positive (M=%d N=%d K=%d L=%d)", d->M, d->N, d->K, d->L);
    return XF_ERR_INVALID_PROBLEM;
  }
  if (!d->A || !d->B || !d->D) {
    set_error("A, B and D must be non-null");
    return XF_ERR_INVALID_PROBLEM;
  }
  const int es = elem_size(d->dtype_ab);
  if ((d->a_k_slab == 0 && d->lda < d->K) || d->ldb < d->N) {
    set_error("leading dimensions too small (lda=%lld K=%d, ldb=%lld N=%d)", (long long)d->lda, d->K,
              (long long)d->ldb, d->N);
    return XF_ERR_INVALID_LAYOUT;
  }
  if (!aligned16(d->A) || !aligned16(d->B) || (d->lda * es) % 16 != 0 || (d->ldb * es) % 16 != 0 ||
      (d->batch_a * es) % 16 != 0 || (d->batch_b * es) % 16 != 0) {
    set_error("A/B base pointers, row pitches and batch strides must be multiples of 16 bytes "
              "(lda=%lld ldb=%lld, %d-byte elements)", (long long)d->lda, (long long)d->ldb, es);
    return XF_ERR_MISALIGNED_OPERAND;
  }
  if (d->a_k_slab != 0) {
    if (d->a_k_slab < 0 || d->a_k_slab % 256 != 0 || d->K % d->a_k_slab != 0 || d->L != 1 ||
        d->lda < d->a_k_slab || (d->a_k_slab_stride * es) % 16 != 0) {
      set_error("A in K slabs needs L == 1, a slab width that is a multiple of 256 and divides K, "
                "lda >= slab width and a 16-byte aligned slab stride (slab=%d K=%d L=%d)",
                d->a_k_slab, d->K, d->L);
      return XF_ERR_INVALID_LAYOUT;
    }
  }
  if (d->num_d_peer < 0 || d->num_d_peer > 7) {
    set_error("num_d_peer must be 0..7 (got %d)", d->num_d_peer);
    return XF_ERR_INVALID_PROBLEM;
  }
  for (int c = 0; c < d->num_d_peer; ++c) {
    if (!d->D_peer[c] || d->dtype_d != XF_DT_BF16) {
      set_error("peer outputs must be non-null and bf16");
      return XF_ERR_INVALID_PROBLEM;
    }
    if (!aligned16(d->D_peer[c]) != !aligned16(d->D)) {
      set_error("peer outputs must have the alignment of D");
      return XF_ERR_MISALIGNED_OPERAND;
    }
  }
  const xf_epilogue_desc& e = d->epi;
  const bool any_epi = e.residual.enabled || e.aux_store.enabled || e.row_scale.enabled ||
                       e.col_scale.enabled || e.bias.enabled || e.unary != XF_UNARY_NONE ||
                       e.pair != XF_PAIR_NONE;
  if (d->dtype_d == XF_DT_S32) {
    if (d->dtype_ab != XF_DT_S8 || any_epi) {
      set_error("int32 output is the raw int8 accumulator: needs int8 inputs and an empty epilogue");
      return XF_ERR_NOT_SUPPORTED;
    }
  } else if (d->dtype_d != XF_DT_BF16 && d->dtype_d != XF_DT_F32) {
    set_error("D dtype must be bf16, f32 or s32 (got %d)", d->dtype_d);
    return XF_ERR_INVALID_DATA_TYPE;
  }
  if (e.unary < XF_UNARY_NONE || e.unary > XF_UNARY_EXP || e.pair < XF_PAIR_NONE ||
      e.pair > XF_PAIR_SWAP) {
    set_error("unknown unary (%d) or pair (%d) op", e.unary, e.pair);
    return XF_ERR_NOT_SUPPORTED;
  }
  if (e.pair != XF_PAIR_NONE && (d->N & 1)) {
    set_error("pair ops need an even N (N=%d)", d->N);
    return XF_ERR_INVALID_PROBLEM;
  }
  const bool compact = e.out_layout == XF_OUT_COMPACT;
  if (compact) {
    if (e.pair != XF_PAIR_SWIGLU && e.pair != XF_PAIR_GEGLU) {
      set_error("the compact [M,N/2] layout needs a SwiGLU/GeGLU pair op");
      return XF_ERR_NOT_SUPPORTED;
    }
    if (d->dtype_d != XF_DT_BF16) {
      set_error("the compact layout writes bf16 only");
      return XF_ERR_NOT_SUPPORTED;
    }
  } else if (e.out_layout != XF_OUT_FULL) {
    set_error("unknown output layout %d", e.out_layout);
    return XF_ERR_NOT_SUPPORTED;
  }
  const int n_out = compact ? d->N / 2 : d->N;
  if (d->ldd < n_out) {
    set_error("ldd=%lld smaller than the %d output columns", (long long)d->ldd, n_out);
    return XF_ERR_INVALID_LAYOUT;
  }
  if (e.row_sumsq) {
    if (e.pair != XF_PAIR_NONE || compact) {
      set_error("row_sumsq needs an epilogue without a pair op and the full output layout");
      return XF_ERR_NOT_SUPPORTED;
    }
    if (d->dtype_d == XF_DT_S32) {
      set_error("row_sumsq needs a floating-point epilogue (dtype_d bf16 or f32)");
      return XF_ERR_NOT_SUPPORTED;
    }
  }
  xf_status s;
  if ((s = check_vec(e.row_scale, "row_scale")) != XF_SUCCESS) return s;
  if ((s = check_vec(e.col_scale, "col_scale")) != XF_SUCCESS) return s;
  if ((s = check_vec(e.bias, "bias")) != XF_SUCCESS) return s;
  if ((s = check_mat(e.residual, "residual", d->N, true)) != XF_SUCCESS) return s;
  if (e.aux_store.enabled) {
    if (!e.aux_store.ptr || e.aux_store.dtype != XF_DT_BF16 || e.aux_store.ld < d->N) {
      set_error("aux_store must be a non-null bf16 [M,N] tensor");
      return XF_ERR_NOT_SUPPORTED;
    }
  }
  if (e.pair == XF_PAIR_ROPE) {
    if (e.cos_sin_period < 0 || (e.cos_sin_period % 32) != 0) {
      set_error("cos_sin_period must be 0 or a multiple of 32 (got %d)", e.cos_sin_period);
      return XF_ERR_NOT_SUPPORTED;
    }
    xf_mat cs = e.cos_sin;
    cs.enabled = 1;
    const int width = e.cos_sin_period > 0 ? e.cos_sin_period : d->N;
    if ((s = check_mat(cs, "cos_sin", width, false)) != XF_SUCCESS) return s;
  }
  return XF_SUCCESS;
}

static VecArg to_vec(const xf_vec& v) {
  VecArg a;
  a.ptr = v.ptr;
  a.batch_stride = v.batch_stride;
  a.null_default = v.null_default;
  a.dtype = v.dtype;
  a.enabled = v.enabled ? 1 : 0;
  a.pad_ = 0;
  return a;
}
static MatArg to_mat(const xf_mat& m) {
  MatArg a;
  a.ptr = m.ptr;
  a.ld = m.ld;
  a.batch_stride = m.batch_stride;
  a.dtype = m.dtype;
  a.enabled = m.enabled ? 1 : 0;
  return a;
}

static int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Measured throughput of each variant on a large bf16 problem (4096 x 28672 x 4096 on B200),
// relative to the paired 256x256 tile with 128-element K stages.  Narrow tiles and short stages
// pay the per-stage barrier hand-off more often and re-read operands from L2 more.
static double variant_eff(const Variant& v) {
  if (v.bn == 256) return v.ctas == 2 ? (v.ks == 2 ? 1.00 : 0.91) : 0.84;
  return v.ctas == 2 ? (v.ks == 2 ? 0.67 : 0.48) : (v.ks == 2 ? 0.72 : 0.55);
}

// Time one scheduling unit spends on one tile, in microseconds: a fixed part (pipeline fill, the
// exposed end of the epilogue) plus the K loop, fitted to 256x256 tiles at K = 4096 and 14336 bf16
// (26 and 85 us at the clocks the part sustains under load).
static double tile_time_us(const Variant& v, int K, int es) {
  return (2.0 + 0.0029 * K * es) * (v.bn / 256.0) / variant_eff(v);
}

// Cluster split-K (variants with kc > 1): the kc CTA pairs of a cluster each run 1/kc of one tile's
// K range and swap partial accumulators through distributed shared memory, about a microsecond.
// One tile per cluster, so the problem must fit the clusters the device can hold at once, and
// every pair needs a few K blocks to fill its pipeline.
static const double kClusterExchangeUs = 1.0;
static const int kMinKbPerGroup = 4;
static bool cluster_split_fits(const Variant& v, const xf_gemm_desc* d, int tiles, int max_clusters) {
  const int es = d->dtype_ab == XF_DT_BF16 ? 2 : 1;
  const int num_kb = (d->K + (128 / es) * v.ks - 1) / ((128 / es) * v.ks);
  if (num_kb < kMinKbPerGroup * v.kc) return false;
  if (d->flags & XF_FLAG_FORCE_CLUSTER_SPLIT) return true;   // more tiles than clusters only queue
  return tiles <= max_clusters;
}

// Split-K of the remainder wave.  With T tiles on U scheduling units, the last wave holds
// T % U tiles and leaves the other units idle; cutting each of those tiles into S K slices fills
// S times as many units for 1/S of the time, at the price of passing the partial accumulators
// through L2 (publish, wait for the other slices, sum).  A unit runs its slice before its whole
// tiles, so when there are whole waves part of that exchange hides behind the next tile's main
// loop (measured: about 7 us remain for a 256-column tile); in a problem of less than one wave
// nothing hides it (about 10 us).  Returns S, or 0 for whole tiles.
static const int kMaxSplit = 8;
static const int kMinKbPerSlice = 4;
static double split_overhead_us(const Variant& v, bool whole_waves) {
  if (whole_waves) return v.bn == 256 ? 7.0 : 5.0;
  return v.bn == 256 ? 10.0 : 7.0;
}
static int split_factor(const Variant& v, const xf_gemm_desc* d, int tiles, int units) {
  if (d->flags & XF_FLAG_NO_SPLIT) return 0;
  if (units <= 0) return 0;
  const int rem = tiles % units;
  if (rem == 0) return 0;
  const int es = d->dtype_ab == XF_DT_BF16 ? 2 : 1;
  const int num_kb = ceil_div(d->K, (128 / es) * v.ks);
  int s = units / rem;
  if (s > num_kb / kMinKbPerSlice) s = num_kb / kMinKbPerSlice;
  if (s > kMaxSplit) s = kMaxSplit;
  // Each slice finishes whole 32-output-column units of the tile (unit u goes to slice u mod S); with
  // more slices than units (a compact 256-column tile has 4) the extra slices only contribute their
  // partial sums.
  if (s < 2) return 0;
  const double t = tile_time_us(v, d->K, es);
  return t * (1.0 - 1.0 / s) > split_overhead_us(v, tiles >= units) ? s : 0;
}

// Picks the CTA tile.  The caller's TileShape (an Intel Xe work-group tile) is only a hint; the
// native tiles are {128,256} rows x {128,256} columns.  The estimate is whole waves x tile time
// plus the remainder wave, whole or split.
static const Variant* select_variant(const xf_gemm_desc* d, int sm_count, int max_quads) {
  const int kind = d->dtype_ab == XF_DT_BF16 ? 0 : 1;
  const int es = kind == 0 ? 2 : 1;
  const Variant* best = nullptr;
  double best_cost = 0;
  for (int i = 0; i < g_num_variants; ++i) {
    const Variant& v = g_variants[i];
    if (v.kind != kind) continue;
    if (v.kc > 1) {
      if (d->flags & (XF_FLAG_NO_CLUSTER_SPLIT | XF_FLAG_FORCE_1CTA | XF_FLAG_FORCE_BN128 | XF_FLAG_FORCE_KS1))
        continue;
      const int tiles = ceil_div(d->M, 128 * v.ctas) * ceil_div(d->N, v.bn) * d->L;
      if (!cluster_split_fits(v, d, tiles, max_quads)) continue;
      if (d->flags & XF_FLAG_FORCE_CLUSTER_SPLIT) return &v;
      const double cost = tile_time_us(v, (d->K + v.kc - 1) / v.kc, es) + kClusterExchangeUs;
      if (!best || cost < best_cost * 0.999) {
        best = &v;
        best_cost = cost;
      }
      continue;
    }
    if ((d->flags & XF_FLAG_FORCE_1CTA) && v.ctas != 1) continue;
    if ((d->flags & XF_FLAG_FORCE_2CTA) && v.ctas != 2) continue;
    if ((d->flags & XF_FLAG_FORCE_BN128) && v.bn != 128) continue;
    if ((d->flags & XF_FLAG_FORCE_BN256) && v.bn != 256) continue;
    if ((d->flags & XF_FLAG_FORCE_KS1) && v.ks != 1) continue;
    if ((d->flags & XF_FLAG_FORCE_KS2) && v.ks != 2) continue;
    const int tiles = ceil_div(d->M, 128 * v.ctas) * ceil_div(d->N, v.bn) * d->L;
    const int units = sm_count / v.ctas;
    const int split = split_factor(v, d, tiles, units);
    const double t = tile_time_us(v, d->K, es);
    double cost = (tiles / units) * t;
    if (tiles % units) cost += split ? t / split + split_overhead_us(v, tiles >= units) : t;
    if (!best || cost < best_cost * 0.999) {
      best = &v;
      best_cost = cost;
    }
  }
  return best;
}

// What the schedule of one problem looks like on the current device: the tile variant, how many
// scheduling units (CTAs or CTA pairs) run at once, and the split of the remainder wave with the
// workspace it needs.  Workspace layout: [0,16) status word, [256, ...) split counters, then the
// partial accumulators (256-byte aligned).
struct Geometry {
  const Variant* v;
  int dev, sm_count, units;   // units: CTAs / CTA pairs / clusters that run at once
  int total_tiles, num_kb;
  int split_s, split_tiles;
  size_t counters_off, partials_off, workspace_bytes;
};

// Clusters of variant v the current device can hold at once (0 if the query fails).
static int active_clusters_of(const Variant& v, int sm_count) {
  const int cl = v.ctas * v.kc;
  const void* fn = reinterpret_cast<const void*>(kernel_of(v, EC_ALL));   // every class has this footprint
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, v.smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count - (sm_count % cl), 1, 1);
  cfg.blockDim = dim3(384, 1, 1);
  cfg.dynamicSmemBytes = v.smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = cl; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int nclusters = 0;
  if (cudaOccupancyMaxActiveClusters(&nclusters, fn, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return nclusters;
}

// Co-resident clusters of the cluster split-K variant (kc K groups) of one input type on device
// `dev`; looked up once per device and kind.
static int max_active_clusters(int kind, int kc, int dev, int sm_count) {
  static std::mutex mu;
  static int cache[64][2];   // 0 = not looked up yet, -1 = none
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && cache[dev][kind] != 0) return cache[dev][kind] < 0 ? 0 : cache[dev][kind];
  int n = 0;
  for (int i = 0; i < g_num_variants; ++i)
    if (g_variants[i].kind == kind && g_variants[i].kc == kc) n = active_clusters_of(g_variants[i], sm_count);
  if (dev >= 0 && dev < 64) cache[dev][kind] = n > 0 ? n : -1;
  return n;
}

static xf_status plan_geometry(const xf_gemm_desc* d, Geometry* g) {
  memset(g, 0, sizeof(*g));
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error("no CUDA device: %s", cudaGetErrorString(cudaGetLastError()));
    return XF_ERR_ARCH_MISMATCH;
  }
  int major = 0, sm_count = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (major != 10) {
    set_error("this library holds sm_100a code only; device %d has compute capability %d.x", dev, major);
    return XF_ERR_ARCH_MISMATCH;
  }
  const Variant* v = select_variant(d, sm_count, max_active_clusters(d->dtype_ab == XF_DT_BF16 ? 0 : 1, 2, dev, sm_count));
  if (!v) {
    set_error("no kernel variant matches the requested flags");
    return XF_ERR_NOT_SUPPORTED;
  }
  g->v = v; g->dev = dev; g->sm_count = sm_count;
  {
    // every class instance of the variant may use the variant's shared memory: set once per device
    static std::mutex mu;
    static bool done[64][sizeof(g_variants) / sizeof(g_variants[0])];
    std::lock_guard<std::mutex> lock(mu);
    const int vi = static_cast<int>(v - g_variants);
    if (dev < 0 || dev >= 64 || !done[dev][vi]) {
      for (int c = 0; c < EC_COUNT; ++c) {
        cudaError_t ce = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel_of(*v, c)),
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, v->smem);
        if (ce != cudaSuccess) {
          set_error("cudaFuncSetAttribute(smem=%d) failed: %s", v->smem, cudaGetErrorString(ce));
          return XF_ERR_INTERNAL;
        }
      }
      if (dev >= 0 && dev < 64) done[dev][vi] = true;
    }
  }
  const int es = elem_size(d->dtype_ab);
  g->num_kb = ceil_div(d->K, (128 / es) * v->ks);
  g->total_tiles = ceil_div(d->M, 128 * v->ctas) * ceil_div(d->N, v->bn) * d->L;
  int units = sm_count / (v->ctas * v->kc);
  if (v->ctas * v->kc > 1) {
    // clusters that can be co-resident (GPC boundaries may leave SMs outside any cluster)
    const int n = active_clusters_of(*v, sm_count);
    if (n > 0) units = n;
  }
  g->units = units;
  g->split_s = v->kc > 1 ? 0 : split_factor(*v, d, g->total_tiles, units);
  g->split_tiles = g->split_s ? g->total_tiles % units : 0;
  g->counters_off = 256;
  const size_t counters = static_cast<size_t>(g->split_tiles) * v->ctas * 8 * sizeof(int);
  g->partials_off = g->counters_off + ((counters + 255) & ~static_cast<size_t>(255));
  const size_t partials = static_cast<size_t>(g->split_tiles) * g->split_s * v->ctas * 128 * v->bn * 4;
  g->workspace_bytes = g->split_s ? g->partials_off + partials : 16;
  return XF_SUCCESS;
}

// Zeroes `bytes` of device memory and returns only once that has happened.  A plain cudaMemset of
// device memory is queued on the legacy default stream and may still be pending when the caller
// launches on a non-blocking stream of its own; here the clear runs on a private non-blocking
// stream per device and is waited for.
static cudaError_t clear_now(void* ptr, size_t bytes, int dev) {
  static std::mutex mu;
  static cudaStream_t streams[64];
  cudaStream_t st = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!streams[dev]) {
      cudaError_t e = cudaStreamCreateWithFlags(&streams[dev], cudaStreamNonBlocking);
      if (e != cudaSuccess) return e;
    }
    st = streams[dev];
  }
  cudaError_t e = cudaMemsetAsync(ptr, 0, bytes, st);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(st);
}

static xf_status build_plan(const xf_gemm_desc* d, void* workspace, xf_plan* plan,
                            bool clear_status_now = true, bool strict_workspace = false) {
  Geometry g;
  xf_status gs = plan_geometry(d, &g);
  if (gs != XF_SUCCESS) return gs;
  if (strict_workspace && g.workspace_bytes > d->workspace_bytes) {
    set_error("this problem's schedule cuts the tiles of its last wave into %d K slices and needs %zu bytes "
              "of workspace; only %llu are available here.  Set XF_FLAG_NO_SPLIT to run whole tiles (16 "
              "bytes), or allocate a workspace and use xf_gemm_plan_create / xf_gemm_run",
              g.split_s, g.workspace_bytes, (unsigned long long)d->workspace_bytes);
    return XF_ERR_NOT_SUPPORTED;
  }
  if (g.split_s && (!workspace || d->workspace_bytes < g.workspace_bytes || !aligned16(workspace))) {
    // the caller did not promise room for the partial accumulators: whole tiles only.  The tile
    // variant may differ from the one a split would have chosen, so select again.
    xf_gemm_desc whole = *d;
    whole.flags |= XF_FLAG_NO_SPLIT;
    gs = plan_geometry(&whole, &g);
    if (gs != XF_SUCCESS) return gs;
  }
  const int dev = g.dev;
  const Variant* v = g.v;
  plan->variant = v;
  plan->no_pdl = (d->flags & XF_FLAG_NO_PDL) ? 1 : 0;
  plan->device = dev;
  GemmParams& p = plan->params;
  memset(&p, 0, sizeof(p));
  const int es = elem_size(d->dtype_ab);
  const int kslab = 128 / es;            // K elements per 128-byte slab (A box width)
  const int kblk = kslab * v->ks;        // K elements per pipeline stage (B box height)
  const int grp_cols = 128 / es;
  p.M = d->M; p.N = d->N; p.K = d->K; p.L = d->L;
  p.tiles_m = ceil_div(d->M, 128 * v->ctas);
  p.tiles_n = ceil_div(d->N, v->bn);
  p.num_kb = ceil_div(d->K, kblk);
  // Rasterisation: tiles run M-fastest inside groups of group_m row tiles, so the units that run
  // together share B panels and a group's A panels are read again by every following wave of the
  // group.  The group is as tall as the A panels that fit a share of L2 (fewer passes over B).
  {
    int l2 = 0;
    cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev);
    const double panel = static_cast<double>(128 * v->ctas) * d->K * es;   // bytes of one row tile's A panel
    int gm = static_cast<int>(0.40 * l2 / (panel > 1 ? panel : 1));
    if (gm < 8) gm = 8;   // shorter groups only add passes over B (measured on 8192 x 8192 x 28672 int8)
    if (gm > p.tiles_m) gm = p.tiles_m;
    if (const char* eg = getenv("XEFUSE_GROUP_M")) {   // tuning override
      const int v2 = atoi(eg);
      if (v2 > 0) gm = v2;
    }
    p.group_m = gm;
    p.l2_hint_a = p.l2_hint_b = 0;
    if (const char* eh = getenv("XEFUSE_L2_HINTS")) {  // tuning override: "<a><b>", 0 none 1 last 2 first
      if (eh[0] >= '0' && eh[0] <= '2') p.l2_hint_a = eh[0] - '0';
      if (eh[0] && eh[1] >= '0' && eh[1] <= '2') p.l2_hint_b = eh[1] - '0';
    }
  }
  p.a_batched = (d->L > 1 && d->batch_a != 0) ? 1 : 0;
  p.b_batched = (d->L > 1 && d->batch_b != 0) ? 1 : 0;
  p.D = d->D; p.ldd = d->ldd; p.batch_d = d->batch_d;
  p.d_dtype = d->dtype_d;
  p.status = reinterpret_cast<int*>(workspace);
  // about two seconds of SM clocks; a millisecond for callers that would rather fail fast
  p.wait_budget = (d->flags & XF_FLAG_SHORT_WAITS) ? 2000000LL : 4000000000LL;
  const xf_epilogue_desc& e = d->epi;
  p.epi.residual = to_mat(e.residual);
  p.epi.aux_store = to_mat(e.aux_store);
  p.epi.row_scale = to_vec(e.row_scale);
  p.epi.col_scale = to_vec(e.col_scale);
  p.epi.bias = to_vec(e.bias);
  p.epi.cos_sin = to_mat(e.cos_sin);
  p.epi.cos_sin.enabled = (e.pair == XF_PAIR_ROPE);
  p.epi.cos_sin_period = e.cos_sin_period;
  p.epi.unary = e.unary;
  p.epi.pair = e.pair;
  p.epi.compact = (e.out_layout == XF_OUT_COMPACT) ? 1 : 0;
  p.epi.row_sumsq = e.row_sumsq;

  const int n_out = p.epi.compact ? d->N / 2 : d->N;
  const bool tma_store_ok = d->dtype_d == XF_DT_BF16 && aligned16(d->D) && (d->ldd * 2) % 16 == 0 &&
                            (d->batch_d * 2) % 16 == 0 && !(d->flags & XF_FLAG_DIRECT_STORE);
  p.direct_store = tma_store_ok ? 0 : 1;
  p.diag = ((d->flags & XF_FLAG_DIAG_NO_LOAD) ? 1 : 0) | ((d->flags & XF_FLAG_DIAG_NO_MMA) ? 2 : 0) |
           ((d->flags & XF_FLAG_DIAG_NO_EPILOGUE) ? 4 : 0) | ((d->flags & XF_FLAG_DIAG_NO_STORE) ? 8 : 0) |
           ((d->flags & XF_FLAG_NO_TAIL_HELP) ? 16 : 0) | ((d->flags & XF_FLAG_NO_ACC_PREFETCH) ? 32 : 0) |
           ((d->flags & XF_FLAG_DIAG_NO_ACC_READ) ? 64 : 0);
  // The kernel instance: the smallest epilogue class that holds every step this descriptor uses.
  {
    int need = 0;
    if (e.residual.enabled || e.aux_store.enabled) need |= EF_MAT;
    if (e.unary != XF_UNARY_NONE) need |= EF_UNARY;
    if (e.pair == XF_PAIR_SWIGLU || e.pair == XF_PAIR_GEGLU) need |= EF_GLU;
    if (e.pair == XF_PAIR_ROPE) need |= EF_ROPE;
    if ((e.pair != XF_PAIR_NONE && !(need & (EF_GLU | EF_ROPE))) || d->dtype_d != XF_DT_BF16 || p.direct_store ||
        e.row_sumsq != nullptr)
      need |= EF_MISC;
    const int cls = need == 0 ? EC_SCALE : need == EF_MAT ? EC_MAT : need == EF_GLU ? EC_GLU
                    : need == EF_ROPE ? EC_ROPE : EC_ALL;
    plan->fn = kernel_of(*v, (d->flags & XF_FLAG_GENERIC_EPILOGUE) ? EC_ALL : cls);
  }

  const CUtensorMapDataType dt =
      d->dtype_ab == XF_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint64_t la = p.a_batched ? d->L : 1, lb = p.b_batched ? d->L : 1;
  const uint64_t sa2 = p.a_batched ? (uint64_t)d->batch_a * es : (uint64_t)d->lda * es * d->M;
  const uint64_t sb2 = p.b_batched ? (uint64_t)d->batch_b * es : (uint64_t)d->ldb * es * d->K;
  p.a_k_slab = d->a_k_slab;
  if (d->a_k_slab > 0) {
    if (!encode_3d(&p.tm_a, dt, d->A, d->a_k_slab, d->M, d->K / d->a_k_slab, (uint64_t)d->lda * es,
                   (uint64_t)d->a_k_slab_stride * es, kslab, 128, CU_TENSOR_MAP_SWIZZLE_128B))
      return XF_ERR_INTERNAL;
  } else if (!encode_3d(&p.tm_a, dt, d->A, d->K, d->M, la, (uint64_t)d->lda * es, sa2, kslab, 128,
                        CU_TENSOR_MAP_SWIZZLE_128B))
    return XF_ERR_INTERNAL;
  if (!encode_3d(&p.tm_b, dt, d->B, d->N, d->K, lb, (uint64_t)d->ldb * es, sb2, grp_cols, kblk,
                 CU_TENSOR_MAP_SWIZZLE_128B))
    return XF_ERR_INTERNAL;
  if (!p.direct_store) {
    const uint64_t sd2 = d->L > 1 ? (uint64_t)d->batch_d * 2 : (uint64_t)d->ldd * 2 * d->M;
    if (!encode_3d(&p.tm_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d->D, n_out, d->M, d->L,
                   (uint64_t)d->ldd * 2, sd2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B))
      return XF_ERR_INTERNAL;
  }
  // Epilogue operand of each CTA's last tile through TMA (see GemmParams::tm_opnd): the cos_sin
  // table when the epilogue rotates pairs, else the residual; only where TMA can address it.
  p.tail_opnd = 0;
  if (v->kc == 1 && d->dtype_d != XF_DT_S32 && !(d->flags & XF_FLAG_NO_TAIL_STAGING)) {
    const bool multi = d->L > 1;
    if (e.pair == XF_PAIR_ROPE) {
      const int P = e.cos_sin_period;
      const xf_mat& m = e.cos_sin;
      if (P > 0 && P <= 128 && v->bn % P == 0 && m.dtype == XF_DT_F32 && aligned16(m.ptr) &&
          (m.ld * 4) % 16 == 0 && (!multi || (m.batch_stride > 0 && (m.batch_stride * 4) % 16 == 0))) {
        const uint64_t s2 = multi ? (uint64_t)m.batch_stride * 4 : (uint64_t)m.ld * 4 * d->M;
        if (encode_3d(&p.tm_opnd, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, m.ptr, P, d->M, d->L, (uint64_t)m.ld * 4, s2,
                      32, 128, CU_TENSOR_MAP_SWIZZLE_128B)) {
          p.tail_opnd = 2;
          p.tail_opnd_boxes = P / 32;
        }
      }
    } else if (e.residual.enabled) {
      const xf_mat& m = e.residual;
      if (m.dtype == XF_DT_BF16 && aligned16(m.ptr) && (m.ld * 2) % 16 == 0 &&
          (!multi || (m.batch_stride > 0 && (m.batch_stride * 2) % 16 == 0))) {
        const uint64_t s2 = multi ? (uint64_t)m.batch_stride * 2 : (uint64_t)m.ld * 2 * d->M;
        if (encode_3d(&p.tm_opnd, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, m.ptr, d->N, d->M, d->L, (uint64_t)m.ld * 2,
                      s2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B)) {
          p.tail_opnd = 1;
          p.tail_opnd_boxes = v->bn / 64;
        }
      }
    }
  }
  // Residual slices through TMA (GemmParams::tm_res): needs what the bf16 TMA store of D needs.
  p.res_tma = 0;
  if (e.residual.enabled && e.pair != XF_PAIR_ROPE && !p.direct_store && !p.epi.compact &&
      !(d->flags & XF_FLAG_NO_RESIDUAL_TMA)) {
    const xf_mat& m = e.residual;
    const bool multi = d->L > 1;
    if (m.dtype == XF_DT_BF16 && aligned16(m.ptr) && (m.ld * 2) % 16 == 0 &&
        (!multi || (m.batch_stride > 0 && (m.batch_stride * 2) % 16 == 0))) {
      const uint64_t s2 = multi ? (uint64_t)m.batch_stride * 2 : (uint64_t)m.ld * 2 * d->M;
      if (encode_3d(&p.tm_res, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, m.ptr, d->N, d->M, d->L, (uint64_t)m.ld * 2, s2,
                    32, 32, CU_TENSOR_MAP_SWIZZLE_64B))
        p.res_tma = 1;
    }
  }
  p.aux_tma = 0;
  if (e.aux_store.enabled && !p.direct_store && !p.epi.compact && !(d->flags & XF_FLAG_NO_RESIDUAL_TMA)) {
    const xf_mat& m = e.aux_store;
    const bool multi = d->L > 1;
    if (m.dtype == XF_DT_BF16 && aligned16(m.ptr) && (m.ld * 2) % 16 == 0 &&
        (!multi || (m.batch_stride > 0 && (m.batch_stride * 2) % 16 == 0))) {
      const uint64_t s2 = multi ? (uint64_t)m.batch_stride * 2 : (uint64_t)m.ld * 2 * d->M;
      if (encode_3d(&p.tm_aux, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, m.ptr, d->N, d->M, d->L, (uint64_t)m.ld * 2, s2,
                    32, 32, CU_TENSOR_MAP_SWIZZLE_64B))
        p.aux_tma = 1;
    }
  }
  p.num_d_peer = d->num_d_peer;
  for (int c = 0; c < d->num_d_peer; ++c) {
    p.D_peer[c] = d->D_peer[c];
    if (!p.direct_store) {
      const uint64_t sd2 = d->L > 1 ? (uint64_t)d->batch_d * 2 : (uint64_t)d->ldd * 2 * d->M;
      if (!encode_3d(&p.tm_d_peer[c], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d->D_peer[c], n_out, d->M, d->L,
                     (uint64_t)d->ldd * 2, sd2, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B))
        return XF_ERR_INTERNAL;
    }
  }

  const int total_tiles = g.total_tiles;
  p.split_s = g.split_s;
  p.split_first = total_tiles - g.split_tiles;
  p.total_items = p.split_first + g.split_tiles * (g.split_s ? g.split_s : 1);
  if (g.split_s) {
    p.split_counters = reinterpret_cast<int*>(static_cast<char*>(workspace) + g.counters_off);
    p.split_partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + g.partials_off);
  }
  // cluster split-K runs one tile per cluster (clusters beyond the co-resident ones queue)
  const int nunits = (v->kc > 1 || p.total_items < g.units) ? p.total_items : g.units;
  plan->grid = nunits * v->ctas * v->kc;
  cudaError_t ce;
  plan->workspace_used = g.split_s ? g.workspace_bytes : 16;
  plan->clear_bytes = g.split_s ? g.partials_off : 16;
  if (g.split_s)
    snprintf(plan->name, sizeof(plan->name), "%s_s%d_ksplit%d", v->name, v->stages, g.split_s);
  else
    snprintf(plan->name, sizeof(plan->name), "%s_s%d", v->name, v->stages);
  if (p.status && clear_status_now) {
    // the status word, and the split counters: each launch leaves them at zero again
    ce = clear_now(p.status, g.split_s ? g.partials_off : 16, dev);
    if (ce != cudaSuccess) {
      set_error("clearing the workspace status word failed: %s", cudaGetErrorString(ce));
      return XF_ERR_INTERNAL;
    }
  }
  return XF_SUCCESS;
}

}  // namespace xf

extern "C" {

xf_status xf_gemm_can_implement(const xf_gemm_desc* desc) { return xf::validate(desc); }

xf_status xf_gemm_workspace_size(const xf_gemm_desc* desc, size_t* bytes) {
  if (!bytes) {
    xf::set_error("null output pointer");
    return XF_ERR_INVALID_PROBLEM;
  }
  *bytes = 16;
  if (!desc || xf::validate(desc) != XF_SUCCESS) return XF_SUCCESS;  // can_implement reports why
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    return XF_SUCCESS;  // no GPU here: a plan cannot be created either
  }
  xf::Geometry g;
  xf_status s = xf::plan_geometry(desc, &g);
  if (s != XF_SUCCESS) return s;
  *bytes = g.workspace_bytes;
  return XF_SUCCESS;
}

static xf_status static_workspace_address(void** out, int* dev_out);

xf_status xf_gemm_plan_create(const xf_gemm_desc* desc, void* workspace, xf_plan** out) {
  if (!out) {
    xf::set_error("null plan output pointer");
    return XF_ERR_INVALID_PROBLEM;
  }
  *out = nullptr;
  xf_status s = xf::validate(desc);
  if (s != XF_SUCCESS) return s;
  xf_plan* plan = static_cast<xf_plan*>(calloc(1, sizeof(xf_plan) + 64));
  if (!plan) {
    xf::set_error("out of host memory");
    return XF_ERR_MEMORY_ALLOCATION;
  }
  s = xf::build_plan(desc, workspace, plan);
  if (s != XF_SUCCESS) {
    free(plan);
    return s;
  }
  // The first plan on a device also looks up the static scratch array of the allocation-free entry,
  // so that the module holding it is resident before that entry is ever called (the kernels live
  // in modules of their own and are loaded when first launched).
  void* unused = nullptr;
  static_workspace_address(&unused, nullptr);
  *out = plan;
  return XF_SUCCESS;
}

xf_status xf_gemm_run(xf_plan* plan, void* stream) {
  if (!plan) {
    xf::set_error("null plan");
    return XF_ERR_INVALID_PROBLEM;
  }
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess || cur != plan->device) {
    xf::set_error("plan %s was created on device %d but device %d is current", plan->name, plan->device, cur);
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan->grid, 1, 1);
  cfg.blockDim = dim3(384, 1, 1);
  cfg.dynamicSmemBytes = plan->variant->smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = plan->variant->ctas * plan->variant->kc;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel's set-up may overlap the tail of the previous
  // kernel of the stream (the kernel waits for that kernel's completion before any global access)
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = plan->no_pdl ? 1 : 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, plan->fn, plan->params);
  if (e != cudaSuccess) {
    xf::set_error("launch of %s failed: %s", plan->name, cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

// ---------------------------------------------------------------------------------------------
// xf_gemm_run_static_workspace: the fused GEMM for callers that may not allocate.
//
// The kernel's scratch -- the status word a bounded wait writes when it gives up and, when the
// tiles of the last wave are cut into K slices, the slice counters and partial accumulators --
// normally lives in a workspace the caller allocates.  Here it lives in the file-scope device array
// below, which every GPU that loads this library holds until the process exits.  Nothing in this
// entry point allocates: the plan is built on the stack, the array's device address comes from
// cudaGetSymbolAddress (host code must not pass the array's name to a kernel: on the host that
// name is only a stand-in, not a device address), and the words that must start at zero are
// cleared with a memset ordered on the caller's stream.  All calls on one device share the array,
// so two calls whose kernels overlap on the GPU race on it.
static __device__ __align__(256) unsigned char g_static_workspace[XF_STATIC_WORKSPACE_BYTES];

static const int kMaxDevices = 64;
static void* g_static_ws_addr[kMaxDevices];
static bool g_static_ws_ready[kMaxDevices];
static std::mutex g_static_ws_mutex;

// Device address of g_static_workspace on the CURRENT device; looked up once per device.
static xf_status static_workspace_address(void** out, int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    xf::set_error("no CUDA device: %s", cudaGetErrorString(e));
    return XF_ERR_ARCH_MISMATCH;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    xf::set_error("device ordinal %d beyond the %d devices the static workspace table covers", dev,
                  kMaxDevices);
    return XF_ERR_NOT_SUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_static_ws_mutex);
  if (!g_static_ws_ready[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_workspace);
    if (e != cudaSuccess || p == nullptr) {
      xf::set_error("cudaGetSymbolAddress(static workspace) failed on device %d: %s", dev,
                    cudaGetErrorString(e));
      return XF_ERR_INTERNAL;
    }
    g_static_ws_addr[dev] = p;
    g_static_ws_ready[dev] = true;
  }
  *out = g_static_ws_addr[dev];
  if (dev_out) *dev_out = dev;
  return XF_SUCCESS;
}

xf_status xf_gemm_run_static_workspace(const xf_gemm_desc* caller_desc, void* stream) {
  xf_status s = xf::validate(caller_desc);
  if (s != XF_SUCCESS) return s;
  void* ws = nullptr;
  s = static_workspace_address(&ws, nullptr);
  if (s != XF_SUCCESS) return s;
  // The array is the whole workspace this call may use.  A schedule that needs more (a split of
  // the last wave whose partial accumulators do not fit) is refused by build_plan, not quietly
  // replaced: the caller decides between XF_FLAG_NO_SPLIT and a workspace of its own.
  xf_gemm_desc local = *caller_desc;
  local.workspace_bytes = XF_STATIC_WORKSPACE_BYTES;
  xf_plan plan;  // on the stack: no host allocation either
  memset(&plan, 0, sizeof(plan));
  s = xf::build_plan(&local, ws, &plan, /*clear_status_now=*/false, /*strict_workspace=*/true);
  if (s != XF_SUCCESS) return s;
  // The array keeps whatever the previous call left: the status word and the slice counters must
  // start at zero (the partial accumulators are written before they are read).
  cudaError_t e = cudaMemsetAsync(ws, 0, plan.clear_bytes, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    xf::set_error("clearing the static workspace failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return xf_gemm_run(&plan, stream);
}

xf_status xf_gemm_static_workspace_status(int32_t* device_code) {
  if (!device_code) {
    xf::set_error("null argument");
    return XF_ERR_INVALID_PROBLEM;
  }
  *device_code = 0;
  void* ws = nullptr;
  int dev = 0;
  xf_status s = static_workspace_address(&ws, &dev);
  if (s != XF_SUCCESS) return s;
  cudaError_t e = cudaMemcpy(device_code, ws, sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    xf::set_error("reading the static workspace's status word failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  if (*device_code != 0) {
    // reported once; the next xf_gemm_run_static_workspace clears the counters it uses anyway
    e = cudaMemset(ws, 0, 16);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    xf::set_error("a kernel launched by xf_gemm_run_static_workspace gave up in a bounded wait (device code %d)",
                  *device_code);
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

xf_status xf_gemm_plan_device_status(xf_plan* plan, int32_t* device_code) {
  if (!plan || !device_code) {
    xf::set_error("null argument");
    return XF_ERR_INVALID_PROBLEM;
  }
  *device_code = 0;
  if (!plan->params.status) return XF_SUCCESS;
  cudaError_t e = cudaMemcpy(device_code, plan->params.status, sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    xf::set_error("reading the status word failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  if (*device_code != 0) {
    // reported once: clear the word, and the split counters a launch that gave up may have left
    // part-way, so the plan can run again
    xf::clear_now(plan->params.status, plan->clear_bytes, plan->device);
    xf::set_error("kernel %s gave up in a bounded wait (device code %d)", plan->name, *device_code);
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

const char* xf_gemm_plan_kernel_name(const xf_plan* plan) { return plan ? plan->name : ""; }

xf_status xf_gemm_cluster_capacity(int32_t dtype_ab, int32_t* pairs, int32_t* quads) {
  if (!pairs || !quads || (dtype_ab != XF_DT_BF16 && dtype_ab != XF_DT_S8)) {
    xf::set_error("cluster_capacity: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  int dev = 0, sm_count = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    xf::set_error("no CUDA device");
    return XF_ERR_ARCH_MISMATCH;
  }
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  const int kind = dtype_ab == XF_DT_BF16 ? 0 : 1;
  *pairs = sm_count / 2;
  for (int i = 0; i < xf::g_num_variants; ++i) {
    const xf::Variant& v = xf::g_variants[i];
    if (v.kind == kind && v.bn == 256 && v.ctas == 2 && v.ks == 2 && v.kc == 1) {
      const int n = xf::active_clusters_of(v, sm_count);
      if (n > 0) *pairs = n;
    }
  }
  *quads = xf::max_active_clusters(kind, 2, dev, sm_count);
  return XF_SUCCESS;
}

xf_status xf_plan_destroy(xf_plan* plan) {
  free(plan);
  return XF_SUCCESS;
}

const char* xf_last_error_string(void) { return xf::last_error(); }

const char* xf_status_string(xf_status s) {
  switch (s) {
    case XF_SUCCESS: return "Success";
    case XF_ERR_MISALIGNED_OPERAND: return "Error Misaligned Operand";
    case XF_ERR_INVALID_DATA_TYPE: return "Error Invalid Data Type";
    case XF_ERR_INVALID_LAYOUT: return "Error Invalid Layout";
    case XF_ERR_INVALID_PROBLEM: return "Error Invalid Problem";
    case XF_ERR_NOT_SUPPORTED: return "Error Not Supported";
    case XF_ERR_WORKSPACE_NULL: return "Error Workspace Null";
    case XF_ERR_INTERNAL: return "Error Internal";
    case XF_ERR_ARCH_MISMATCH: return "Error Architecture Mismatch";
    case XF_ERR_INSUFFICIENT_DRIVER: return "Error Insufficient Driver";
    case XF_ERR_MEMORY_ALLOCATION: return "Error Memory Allocation failed";
    default: return "Invalid status";
  }
}

int32_t xf_version(void) { return 100; }
int32_t xf_compiled_arch(void) { return 100; }

}  // extern "C"
