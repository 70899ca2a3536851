/*
 * xefuse_b200 — C ABI of the B200 (sm_100a) fused GEMM + epilogue library.
 *
 * This is the boundary the header-only C++ front end (xe_fuse::builder::MakeGemm<...>::Gemm,
 * xe_fuse::Gemm* named kernels, xe_fuse::standalone::*) calls into.  Everything is plain C:
 * POD structs, raw device pointers, sizes, a cudaStream_t passed as void*.  No C++ or torch
 * types cross it, nothing throws across it, every entry returns an xf_status.
 *
 * Reference interfaces each entry replaces (paths inside IntelLabs/Xe-Fuse):
 *   xf_gemm_can_implement   <- GemmUniversalAdapter::can_implement(args)
 *                              (include/xe-fuse/builder/epilogue_builder.hpp:378-381, tests/test_k1.cpp:99)
 *   xf_gemm_workspace_size  <- GemmUniversalAdapter::get_workspace_size(args)   (tests/test_k1.cpp:96)
 *   xf_gemm_plan_create     <- GemmUniversalAdapter::initialize(args, workspace) (tests/test_k1.cpp:100)
 *   xf_gemm_run             <- GemmUniversalAdapter::run()                       (tests/test_k1.cpp:101)
 *   xf_epilogue_desc        <- the EVT::Arguments tree of the builder aliases
 *                              (include/xe-fuse/builder/epilogue_builder.hpp:58-280)
 *   xf_sa_*                 <- xe_fuse::standalone::* (include/xe-fuse/standalone/ops.hpp:32-354)
 *   xf_compute_rstd*        <- xe_fuse::launch_compute_rstd / launch_compute_rstd_and_quantize
 *                              (include/xe-fuse/kernels/compute_rstd.hpp:12-125)
 *
 * Memory layout (all row-major, the reference's convention, tests/test_k1.cpp:54-64):
 *   A [L][M][K]  (K contiguous)       bf16 or int8
 *   B [L][K][N]  (N contiguous)       bf16 or int8   -- note: N-contiguous weights
 *   D [L][M][Nout] (Nout contiguous)  bf16 (or fp32 / int32 "raw accumulator" output)
 * Leading dimensions are in elements.  A batch stride of 0 shares one matrix across L.
 */
#ifndef XEFUSE_B200_H_
#define XEFUSE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define XF_API
#else
#define XF_API __attribute__((visibility("default")))
#endif

/* Status codes.  Values mirror cutlass::Status so the front end can cast 1:1. */
typedef enum xf_status {
  XF_SUCCESS = 0,
  XF_ERR_MISALIGNED_OPERAND = 1,
  XF_ERR_INVALID_DATA_TYPE = 2,
  XF_ERR_INVALID_LAYOUT = 3,
  XF_ERR_INVALID_PROBLEM = 4,
  XF_ERR_NOT_SUPPORTED = 5,
  XF_ERR_WORKSPACE_NULL = 6,
  XF_ERR_INTERNAL = 7,
  XF_ERR_ARCH_MISMATCH = 8,
  XF_ERR_INSUFFICIENT_DRIVER = 9,
  XF_ERR_MEMORY_ALLOCATION = 10,
  XF_INVALID = 11
} xf_status;

typedef enum xf_dtype {
  XF_DT_BF16 = 0,
  XF_DT_S8 = 1,
  XF_DT_F32 = 2,
  XF_DT_S32 = 3
} xf_dtype;

/* Unary activation applied after the affine steps
 * (functors of include/xe-fuse/visitors/xe_elementwise_compute.hpp:53-89). */
typedef enum xf_unary {
  XF_UNARY_NONE = 0,
  XF_UNARY_GELU = 1,      /* x*0.5*(1+erf(x/sqrt2)) */
  XF_UNARY_GELU_TANH = 2, /* tanh approximation       */
  XF_UNARY_SILU = 3,      /* x/(1+exp(-x))            */
  XF_UNARY_RELU = 4,
  XF_UNARY_SIGMOID = 5,
  XF_UNARY_EXP = 6
} xf_unary;

/* Operation on adjacent column pairs (2k, 2k+1)
 * (include/xe-fuse/visitors/xe_pairwise_compute.hpp:71-89, xe_rope_compute.hpp:51-59). */
typedef enum xf_pair {
  XF_PAIR_NONE = 0,
  XF_PAIR_SWIGLU = 1, /* silu(x[2k]) * x[2k+1] */
  XF_PAIR_GEGLU = 2,  /* gelu(x[2k]) * x[2k+1] */
  XF_PAIR_ROPE = 3,   /* e' = e*c + o*s ; o' = -e*s + o*c */
  XF_PAIR_SWAP = 4    /* each column takes its partner's value */
} xf_pair;

/* Where the pair result goes. */
typedef enum xf_out_layout {
  XF_OUT_FULL = 0,    /* D is [M,N]; pair ops that yield one value per pair write it to both columns
                         (what the reference's K2 does, tests/test_k2.cpp:4-5) */
  XF_OUT_COMPACT = 1  /* D is [M,N/2]; one value per pair (SwiGLU/GeGLU only) */
} xf_out_layout;

/* A broadcast vector operand: v[m] (per output row) or v[n] (per output column). */
typedef struct xf_vec {
  const void* ptr;        /* device pointer; NULL => null_default is used for every element */
  int32_t dtype;          /* XF_DT_F32 or XF_DT_BF16 */
  int32_t enabled;        /* 0 => step skipped */
  int64_t batch_stride;   /* elements between batches (dCol/dRow's third mode) */
  float null_default;
  int32_t pad_;
} xf_vec;

/* A full [M,N] operand (AuxLoad / AuxStore). */
typedef struct xf_mat {
  const void* ptr;        /* device pointer */
  int32_t dtype;          /* XF_DT_BF16 or XF_DT_F32 */
  int32_t enabled;
  int64_t ld;             /* elements between rows */
  int64_t batch_stride;   /* elements between batches */
} xf_mat;

/*
 * Flat epilogue program.  Every supported visitor tree lowers to this fixed order, each step
 * optional; v starts as float(acc):
 *   1. v += residual[m,n]            (AddResidual)
 *   2. aux_store[m,n] = v            (DualOutput's AuxStore; second output)
 *   3. v *= row_scale[m]             (ScaleRows / per-token scale)
 *   4. v *= col_scale[n]             (ScaleCols / per-channel scale)
 *   5. v += bias[n]                  (BiasAdd)
 *   6. v = unary(v)
 *   7. pair op on columns (2k,2k+1); RoPE takes c,s = cos_sin[m, 2k], cos_sin[m, 2k+1]
 *   8. D = round-to-nearest-even(v)
 */
typedef struct xf_epilogue_desc {
  xf_mat residual;
  xf_mat aux_store;       /* ptr is written; dtype bf16 */
  xf_vec row_scale;
  xf_vec col_scale;
  xf_vec bias;
  int32_t unary;          /* xf_unary */
  int32_t pair;           /* xf_pair */
  xf_mat cos_sin;         /* fp32; ld = row pitch in elements */
  int32_t cos_sin_period; /* 0: table spans all N columns (reference form).  P>0: column n reads
                             cos_sin[m, n % P] (one head_dim-wide table shared by all heads);
                             P must be a multiple of 32 */
  int32_t out_layout;     /* xf_out_layout */
  /* Optional side output for a following RMSNorm: per row, the sums of squares of the final fp32
   * values v (before the rounding to bf16) over each group of 32 consecutive columns, laid out
   * [L][ceil(N/32)][M] floats (xf_row_sumsq_count gives the element count).  Every slot is written
   * exactly once per launch, without atomics: no zeroing needed, results are deterministic.
   * xf_reduce_partials_rsqrt turns them into rstd[m].  Needs pair == none and the full layout.
   * The reference's counterpart is the per-tile ColReduction of K0a_CR
   * (kernels/gemm_residual_gamma_colred.hpp:89-115). */
  float* row_sumsq;
} xf_epilogue_desc;

typedef struct xf_gemm_desc {
  int32_t dtype_ab;       /* XF_DT_BF16 (fp32 accumulate) or XF_DT_S8 (int32 accumulate) */
  int32_t dtype_d;        /* XF_DT_BF16; XF_DT_F32 / XF_DT_S32 give the raw accumulator after the
                             epilogue steps that are enabled (none => exact accumulator) */
  int32_t M, N, K, L;
  const void* A; int64_t lda; int64_t batch_a;
  const void* B; int64_t ldb; int64_t batch_b;
  void* D;       int64_t ldd; int64_t batch_d;
  int32_t tile_m, tile_n, tile_k; /* the caller's TileShape: a hint, mapped to a native CTA tile */
  int32_t flags;          /* XF_FLAG_* */
  xf_epilogue_desc epi;
  /* A stored as K slabs (the all-gathered output of a column-sharded producer stage): element
   * A[m,k] lives at A + (k / a_k_slab) * a_k_slab_stride + m * lda + (k % a_k_slab).  0 = A is one
   * [M,K] matrix.  a_k_slab must be a multiple of 256 elements and divide K; needs L == 1. */
  int32_t a_k_slab;
  int32_t num_d_peer;     /* 0..7 further destinations of the output */
  int64_t a_k_slab_stride;
  /* Further copies of D, with D's ldd/batch_d: every output tile is also stored to each of them
   * from the epilogue.  With pointers into the other GPUs' gathered buffers (peer-mapped memory)
   * this is the all-gather of column shards, overlapped with the GEMM instead of following it. */
  void* D_peer[7];
  /* Size of the workspace that will be handed to xf_gemm_plan_create.  The plan cuts the tiles of
   * the last wave into K slices only if this covers what xf_gemm_workspace_size reports for the
   * same descriptor; with less (0 included) it runs whole tiles and uses the first 16 bytes only,
   * so a caller that never sets it stays correct.  xf_gemm_workspace_size ignores the field. */
  uint64_t workspace_bytes;
} xf_gemm_desc;

/* flags */
#define XF_FLAG_DIRECT_STORE 1   /* write D with plain global stores instead of TMA stores */
#define XF_FLAG_FORCE_1CTA   2   /* never pair CTAs (cta_group::1 only) */
#define XF_FLAG_FORCE_2CTA   4   /* always pair CTAs (cta_group::2) when the shape allows */
#define XF_FLAG_FORCE_BN128  8   /* use the 128-column CTA tile */
#define XF_FLAG_FORCE_BN256  16  /* use the 256-column CTA tile */
#define XF_FLAG_FORCE_KS1    32  /* one 128-byte K slab per pipeline stage */
#define XF_FLAG_FORCE_KS2    64  /* two 128-byte K slabs per pipeline stage */
#define XF_FLAG_NO_SPLIT     128 /* never cut the tiles of the last, partly filled wave into K slices */
#define XF_FLAG_SHORT_WAITS 8192 /* bounded waits inside the kernel give up after about a millisecond
                                    instead of about two seconds (fail fast; also how the give-up
                                    path is tested) */
#define XF_FLAG_NO_TAIL_HELP 32768 /* the producer / MMA / allocator warps do not join the epilogue of a
                                    CTA's last tile (by default they do, as a third worker per TMEM
                                    quadrant: that epilogue has no main loop left to hide behind) */
#define XF_FLAG_NO_PDL      4096 /* launch without programmatic stream serialization: by default the
                                    kernel's set-up may overlap the tail of the previous kernel of the
                                    stream; its global reads and writes always wait for that kernel */
#define XF_FLAG_NO_CLUSTER_SPLIT 65536 /* never use the cluster split-K variants (small problems: the CTA
                                    pairs of one cluster share a tile's K range and swap partial
                                    accumulators through distributed shared memory) */
#define XF_FLAG_NO_TAIL_STAGING 262144 /* a CTA's last tile reads its residual / cos_sin operand with plain
                                    loads like every other tile (by default TMA stages that one tile's
                                    operand in an idle pipeline stage while the main loop drains) */
#define XF_FLAG_NO_ACC_PREFETCH 524288 /* the epilogue reads each 32-column accumulator slice out of tensor
                                    memory when it needs it (by default a warp requests its next slice
                                    while it works on the current one, where it has registers to spare) */
#define XF_FLAG_NO_RESIDUAL_TMA 2097152 /* the epilogue reads the residual with per-thread 16-byte loads and
                                    writes the auxiliary output with per-thread stores (by default TMA
                                    brings each 32 x 32 residual block into the staging buffer its result
                                    is then stored from, and the auxiliary block leaves the same way) */
#define XF_FLAG_GENERIC_EPILOGUE 4194304 /* launch the kernel instance that carries every epilogue step (by
                                    default a plan launches the instance compiled for the smallest class
                                    of steps that covers its descriptor; same results, shorter tail) */
#define XF_FLAG_FORCE_CLUSTER_SPLIT 131072 /* use a cluster split-K variant whenever K is long enough, also
                                    for problems with more tiles than co-resident clusters */

/* Timing diagnostics, not for production: each flag removes one part of the kernel and leaves D
 * GARBAGE.  They are refused (XF_ERR_NOT_SUPPORTED) unless the environment holds
 * XEFUSE_ALLOW_DIAG=1 when the problem is checked. */
#define XF_FLAG_DIAG_NO_LOAD  256    /* skip the TMA operand loads */
#define XF_FLAG_DIAG_NO_MMA   512    /* skip the tensor-core MMAs */
#define XF_FLAG_DIAG_NO_EPILOGUE 1024 /* drain TMEM, compute and store nothing */
#define XF_FLAG_DIAG_NO_STORE 2048   /* run the epilogue math, store nothing */
#define XF_FLAG_DIAG_NO_ACC_READ 1048576 /* the epilogue works on zeros instead of reading tensor memory */
#define XF_FLAG_DIAG_MASK (256 | 512 | 1024 | 2048 | 1048576)

typedef struct xf_plan xf_plan;

/* Checks a problem without touching the GPU.  Returns XF_SUCCESS or the reason it is refused. */
XF_API xf_status xf_gemm_can_implement(const xf_gemm_desc* desc);
/* Bytes of caller-owned device workspace xf_gemm_plan_create needs on the CURRENT device: a
 * 16-byte status word, plus, when the tiles of the last wave are cut into K slices, counters and
 * fp32/int32 partial accumulators (a few MB).  Query it on the device the plan will run on, with
 * the descriptor (flags included) the plan will be created from. */
XF_API xf_status xf_gemm_workspace_size(const xf_gemm_desc* desc, size_t* bytes);
/* Copies the descriptor, picks a kernel, encodes TMA tensor maps.  workspace may be NULL when
 * xf_gemm_workspace_size reported 0; otherwise it must stay valid for the plan's lifetime. */
XF_API xf_status xf_gemm_plan_create(const xf_gemm_desc* desc, void* workspace, xf_plan** plan);
/* Enqueues one fused launch on `stream` (a cudaStream_t; NULL = default stream).  Re-entrant.  The
 * device the plan was created on must be current (XF_ERR_INVALID_PROBLEM otherwise). */
XF_API xf_status xf_gemm_run(xf_plan* plan, void* stream);
/* How many CTA pairs and how many 4-CTA clusters (cluster split-K, two pairs per tile) of the
 * 256 x 256 kernel the current device can hold at once for the given input type: the scheduling
 * units the planner counts in (74 and about 36 on a 148-SM B200; GPC boundaries decide). */
XF_API xf_status xf_gemm_cluster_capacity(int32_t dtype_ab, int32_t* pairs, int32_t* quads);
/* Reads back the device status word of the plan's last launches.  Synchronise the stream(s) the
 * plan ran on first: the read itself only orders against the legacy default stream.
 * 0 = ok (returns XF_SUCCESS), otherwise the code of the bounded wait that gave up: 1 producer
 * waiting for a free stage, 2 MMA issuer waiting for operands, 3 MMA issuer waiting for a free
 * accumulator, 4 epilogue waiting for the accumulator, 5 a K slice waiting for the other slices'
 * partials, 6 a cluster split-K pair waiting for the other pairs' partials (returns XF_ERR_INTERNAL;
 * the outputs of that launch are not valid).  A non-zero code is
 * reported once: the word and the split counters are cleared so the plan can run again. */
XF_API xf_status xf_gemm_plan_device_status(xf_plan* plan, int32_t* device_code);
/* Name of the kernel variant the plan selected, e.g. "bf16_128x256_cta2_s6". */
XF_API const char* xf_gemm_plan_kernel_name(const xf_plan* plan);
XF_API xf_status xf_plan_destroy(xf_plan* plan);

/*
 * One-call fused GEMM that allocates nothing, for callers that cannot call cudaMalloc: a serving
 * process that handed all of HBM to its own memory pool at start-up (a later cudaMalloc would
 * fail, or stall every stream while the driver synchronises the device), or a plug-in that is
 * only lent buffers by its host and owns no allocator.  It has no counterpart in the reference,
 * whose callers always allocate a workspace (tests/test_k1.cpp:96-97).
 *
 * The caller passes inputs and outputs in `desc` as usual.  The kernel's scratch -- the status
 * word of its bounded waits and, when the tiles of the last wave are cut into K slices, the slice
 * counters and partial accumulators -- lives in a static device array of
 * XF_STATIC_WORKSPACE_BYTES (2 MiB) that each GPU using the library holds until process exit.  A
 * problem whose schedule needs more than that (xf_gemm_workspace_size tells) is refused with
 * XF_ERR_NOT_SUPPORTED and a message naming the size; pass XF_FLAG_NO_SPLIT to run it with whole
 * tiles, which needs 16 bytes.  No cudaMalloc, cudaFree or host allocation happens inside: the
 * plan lives on the stack and is rebuilt on every call (three tensor-map encodes), so prefer a
 * plan when you can allocate.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call outside any stream capture.  All calls on a device
 * share the array and each call clears the words it needs at zero on `stream` before its kernel,
 * so calls whose kernels may overlap on the GPU (different streams, no ordering between them)
 * race on it: order them, or use plans with separate workspaces.
 */
#define XF_STATIC_WORKSPACE_BYTES 2097152
XF_API xf_status xf_gemm_run_static_workspace(const xf_gemm_desc* desc, void* stream);
/* Status word of the static array on the current device, with the contract of
 * xf_gemm_plan_device_status: 0 = the launches since the last query were fine; otherwise the code
 * of the bounded wait that gave up (XF_ERR_INTERNAL; reported once, then cleared).  Synchronise
 * the stream(s) first.  Allocates nothing.  No counterpart in the reference either. */
XF_API xf_status xf_gemm_static_workspace_status(int32_t* device_code);

/* Thread-local text of the last error produced by any entry point on this thread. */
XF_API const char* xf_last_error_string(void);
XF_API const char* xf_status_string(xf_status s);
/* Library version and the SM architecture the kernels were compiled for (100 => sm_100a). */
XF_API int32_t xf_version(void);
XF_API int32_t xf_compiled_arch(void);

/*
 * Stand-alone (unfused) elementwise passes over a bf16 [L][M][N] tensor, in place; these are the
 * baseline the fused kernels are compared with (include/xe-fuse/standalone/ops.hpp).
 */
XF_API xf_status xf_sa_scale_rows(void* D, const float* scale, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_scale_cols(void* D, const float* scale, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_add_residual(void* D, const void* residual, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_residual_gamma(void* D, const void* residual, const float* gamma,
                                      int M, int N, int L, void* stream);
XF_API xf_status xf_sa_swiglu(void* D, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_geglu(void* D, int M, int N, int L, void* stream);
/* out = rope(in); in and out are distinct buffers (ops.hpp:119-144). */
XF_API xf_status xf_sa_rope(void* out, const void* in, const float* cos_sin, int M, int N, int L,
                            void* stream);
/* out = rope(in * scale[m]); in and out are distinct buffers (ops.hpp:146-176). */
XF_API xf_status xf_sa_rope_scaled(void* out, const void* in, const float* scale,
                                   const float* cos_sin, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_unary(void* D, int unary, int M, int N, int L, void* stream);
XF_API xf_status xf_sa_bias_add(void* D, const float* bias, int M, int N, int L, void* stream);
/* out_bf16 = float(acc_i32) * scale_token[m] * scale_channel[n] (ops.hpp:335-354). */
XF_API xf_status xf_sa_dequant_w8a8(void* out, const int32_t* acc, const float* scale_token,
                                    const float* scale_channel, int M, int N, int L, void* stream);
/* rstd[m] = 1/sqrt(mean_n x[m,n]^2 + eps) over bf16 rows (compute_rstd.hpp:12-49). */
XF_API xf_status xf_compute_rstd(const void* x, float* rstd, int M, int N, int L, float eps,
                                 void* stream);
/* RMS-normalise a bf16 row and quantise it to int8 with a per-token absmax scale that absorbs
 * rstd (compute_rstd.hpp:67-125). */
XF_API xf_status xf_compute_rstd_and_quantize(const void* x, int8_t* xq, float* scale_token,
                                              int M, int N, int L, float eps, void* stream);

/* Number of floats xf_epilogue_desc.row_sumsq must hold for an M x N x L problem. */
XF_API size_t xf_row_sumsq_count(int M, int N, int L);
/* rstd[l*M+m] = 1/sqrt(sum of row m's partials / N + eps) from the row_sumsq side output of a fused
 * GEMM (launch_reduce_partials_rsqrt, kernels/gemm_residual_gamma_colred.hpp:199-226). */
XF_API xf_status xf_reduce_partials_rsqrt(const float* partials, float* rstd, int M, int N, int L,
                                          float eps, void* stream);

/*
 * Engine-style stand-alone passes: the comparison arm of the reference's generated pipelines
 * (namespace xe_fuse::vllm_equiv, include/xe-fuse/standalone/vllm_ops.hpp).  bf16 data unless
 * noted, fp32 math, one rounding to bf16.  All asynchronous on `stream`.
 */
/* out[m,:] = input[m,:] * rsqrt(mean(input[m,:]^2) + eps) * weight[:]; weight bf16 [N]; out may be
 * input (vllm_ops.hpp:33-69). */
XF_API xf_status xf_ve_rms_norm(void* out, const void* input, const void* weight, int M, int N,
                                float eps, void* stream);
/* residual += input; input = RMSNorm(residual) * weight, both in place (vllm_ops.hpp:75-114). */
XF_API xf_status xf_ve_fused_add_rms_norm(void* input, void* residual, const void* weight, int M,
                                          int N, float eps, void* stream);
/* out[m,i] = act(input[m,i]) * input[m,d+i]; input [M,2d], out [M,d]; gelu=0 SiLU, 1 erf-GeLU
 * (silu_and_mul / gelu_and_mul, vllm_ops.hpp:119-164). */
XF_API xf_status xf_ve_act_and_mul(void* out, const void* input, int d, int M, int gelu,
                                   void* stream);
/* NeoX rotary embedding in place on query [M,num_heads,head_size] and, if not null, key
 * [M,num_kv_heads,head_size]; cos_sin_cache fp32 [M,rot_dim] = cos half then sin half
 * (vllm_ops.hpp:170-227). */
XF_API xf_status xf_ve_rotary_embedding(void* query, void* key, const float* cos_sin_cache,
                                        int head_size, int num_heads, int num_kv_heads, int rot_dim,
                                        int M, void* stream);
/* int32 accumulator [L,M,2d] -> bf16 [L,M,2d]: W8A8 dequantisation, act(gate)*up over the two
 * halves, the result written to both halves (dequant_and_silu_mul / dequant_and_gelu_mul,
 * vllm_ops.hpp:244-311). */
XF_API xf_status xf_ve_dequant_act_mul(void* out, const int32_t* acc, const float* scale_token,
                                       const float* scale_channel, int d, int M, int L, int gelu,
                                       void* stream);
/* int32 accumulator [L,M,N] -> bf16: W8A8 dequantisation then the interleaved-pair rotation with a
 * full fp32 cos_sin [L,M,N] (dequant_and_rotary_embedding, vllm_ops.hpp:317-346). */
XF_API xf_status xf_ve_dequant_rotary(void* out, const int32_t* acc, const float* scale_token,
                                      const float* scale_channel, const float* cos_sin, int M, int N,
                                      int L, void* stream);

/*
 * Harness utilities behind the front end's cutlass/util shims (not on the fused path): the
 * seeded fill the harness mains call initialize_block, the naive device GEMM they use to rebuild
 * the expected accumulator (cutlass::reference::device::GemmComplex in tests/test_k1.cpp:113-117)
 * and the relative comparison (BlockCompareRelativelyEqual, tests/test_k1.cpp:138-140).
 */
XF_API xf_status xf_harness_fill_uniform(int dtype, void* ptr, long long n, uint64_t seed, int lo,
                                         int hi, void* stream);
XF_API xf_status xf_harness_ref_gemm(int dtype_a, const void* A, int64_t lda, int64_t batch_a,
                                     int dtype_b, const void* B, int64_t ldb, int64_t batch_b,
                                     int dtype_c, const void* C, int64_t ldc, int64_t batch_c,
                                     int dtype_d, void* D, int64_t ldd, int64_t batch_d, int M, int N,
                                     int K, int L, float alpha, float beta, void* stream);
XF_API xf_status xf_harness_compare(int dtype, const void* a, const void* b, long long n,
                                    float epsilon, float nonzero_floor, long long* mismatches,
                                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XEFUSE_B200_H_ */
