/*
 * CPU oracle for the fused GEMM + epilogue path.  TEST INFRASTRUCTURE ONLY: nothing the library
 * ships links, loads or calls this file; only tests/, the smoke check and bench.py's CPU-baseline
 * legs use it, as the checker and as the timed CPU arm.
 *
 * PARITY UNPINNED.  The reference (IntelLabs/Xe-Fuse) has no host implementation, no golden
 * vectors and no fixtures for this path; its tests rebuild the expected result on the device with
 * cutlass::reference::device::GemmComplex (from intel/sycl-tla, fetched at tag `main`, not in the
 * tree) plus a per-preset parallel_for lambda.  This file restates those lambda bodies in plain C
 * (sycl::exp/erf -> expf/erff), each function citing the lines it follows, over an fp32-accumulate
 * GEMM for bf16 inputs and an exact int32 GEMM for int8 inputs.
 *
 * Conventions (tests/test_k1.cpp:54-64): A [M,K] row-major, B [K,N] row-major, D [M,N] row-major.
 * bf16 values travel as uint16_t bit patterns; conversion back to bf16 is round-to-nearest-even
 * (FloatRoundStyle::round_to_nearest, include/xe-fuse/builder/epilogue_builder.hpp:94).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define XO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 helpers */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

XO_API void xo_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_rne(src[i]);
}

XO_API void xo_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

XO_API void xo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

XO_API int xo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ GEMMs */
/* C[m,n] = sum_k float(A[m,k]) * float(B[k,n]), fp32 accumulation in increasing k
 * (what GemmComplex with ElementAcc=float computes, tests/test_k4.cpp:120-124). */
XO_API void xo_gemm_bf16_f32(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K) {
  /* widen B once so the inner loop is a plain fp32 axpy the compiler vectorises */
  float* Bf = (float*)malloc((size_t)K * N * sizeof(float));
  xo_bf16_to_f32(B, Bf, (int64_t)K * N);
  const int JB = 2048;
#pragma omp parallel for schedule(dynamic, 1)
  for (int m0 = 0; m0 < M; m0 += 4) {
    const int mr = (M - m0) < 4 ? (M - m0) : 4;
    for (int j0 = 0; j0 < N; j0 += JB) {
      const int jn = (N - j0) < JB ? (N - j0) : JB;
      float acc[4][2048];
      for (int r = 0; r < mr; ++r)
        for (int j = 0; j < jn; ++j) acc[r][j] = 0.0f;
      for (int k = 0; k < K; ++k) {
        const float* b = Bf + (size_t)k * N + j0;
        float a[4];
        for (int r = 0; r < mr; ++r) a[r] = bf16_to_f32(A[(size_t)(m0 + r) * K + k]);
        if (mr == 4) {
          for (int j = 0; j < jn; ++j) {
            const float bv = b[j];
            acc[0][j] += a[0] * bv;
            acc[1][j] += a[1] * bv;
            acc[2][j] += a[2] * bv;
            acc[3][j] += a[3] * bv;
          }
        } else {
          for (int r = 0; r < mr; ++r)
            for (int j = 0; j < jn; ++j) acc[r][j] += a[r] * b[j];
        }
      }
      for (int r = 0; r < mr; ++r)
        memcpy(C + (size_t)(m0 + r) * N + j0, acc[r], (size_t)jn * sizeof(float));
    }
  }
  free(Bf);
}

/* Exact int32 accumulation of int8 x int8.  (The reference's W8A8 tests accumulate in float over
 * int8-valued floats, tests/test_k4_w8a8.cpp:166-184; the integer sum is the value that float sum
 * approximates and is what a bit-exact check needs.  |acc| <= K*128*128 < 2^31 for K < 131072.) */
XO_API void xo_gemm_s8_s32(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
  const int JB = 2048;
#pragma omp parallel for schedule(dynamic, 1)
  for (int m0 = 0; m0 < M; m0 += 4) {
    const int mr = (M - m0) < 4 ? (M - m0) : 4;
    for (int j0 = 0; j0 < N; j0 += JB) {
      const int jn = (N - j0) < JB ? (N - j0) : JB;
      int32_t acc[4][2048];
      for (int r = 0; r < mr; ++r)
        for (int j = 0; j < jn; ++j) acc[r][j] = 0;
      for (int k = 0; k < K; ++k) {
        const int8_t* b = B + (size_t)k * N + j0;
        int32_t a[4] = {0, 0, 0, 0};
        for (int r = 0; r < mr; ++r) a[r] = A[(size_t)(m0 + r) * K + k];
        for (int j = 0; j < jn; ++j) {
          const int32_t bv = b[j];
          acc[0][j] += a[0] * bv;
          acc[1][j] += a[1] * bv;
          acc[2][j] += a[2] * bv;
          acc[3][j] += a[3] * bv;
        }
      }
      for (int r = 0; r < mr; ++r)
        memcpy(C + (size_t)(m0 + r) * N + j0, acc[r], (size_t)jn * sizeof(int32_t));
    }
  }
}

/* ------------------------------------------------------------------ activations */
/* include/xe-fuse/visitors/xe_elementwise_compute.hpp:53-89 */
static inline float gelu_erf(float x) { return x * 0.5f * (1.0f + erff(x * 0.7071067811865475f)); }
static inline float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  float x3 = x * x * x;
  return x * 0.5f * (1.0f + tanhf(k * (x + 0.044715f * x3)));
}
static inline float silu(float x) { return x / (1.0f + expf(-x)); }
static inline float relu(float x) { return x > 0.0f ? x : 0.0f; }
static inline float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

enum { XO_UN_NONE = 0, XO_UN_GELU, XO_UN_GELU_TANH, XO_UN_SILU, XO_UN_RELU, XO_UN_SIGMOID, XO_UN_EXP };
enum { XO_PAIR_NONE = 0, XO_PAIR_SWIGLU, XO_PAIR_GEGLU, XO_PAIR_ROPE, XO_PAIR_SWAP };

static inline float unary(int op, float x) {
  switch (op) {
    case XO_UN_GELU: return gelu_erf(x);
    case XO_UN_GELU_TANH: return gelu_tanh(x);
    case XO_UN_SILU: return silu(x);
    case XO_UN_RELU: return relu(x);
    case XO_UN_SIGMOID: return sigmoidf(x);
    case XO_UN_EXP: return expf(x);
    default: return x;
  }
}

/* ------------------------------------------------------------------ the flat epilogue program
 * acc      float [M,N] (int32 accumulators are passed converted with (float)acc, the conversion
 *          XeCompute<..., ElementCompute=float> performs)
 * residual bf16 [M,N] or NULL        -> v += residual            (AddResidual, builder:136-138)
 * aux_out  bf16 [M,N] or NULL        <- v                        (DualOutput AuxStore, builder:316-323)
 * row      float [M] or NULL         -> v *= row[m]              (ScaleRows, builder:120-124)
 * col      float [N] or NULL         -> v *= col[n]              (ScaleCols, builder:128-133)
 * bias     float [N] or NULL         -> v += bias[n]             (BiasAdd, builder:229-232)
 * unary, pair                         as the enums above
 * cos_sin  float rows of pitch cs_ld; period P>0 reads column n % P (0: n)
 * compact  1: out is [M,N/2], one value per pair (SwiGLU/GeGLU); 0: out is [M,N]
 * out      bf16 (RNE)
 */
XO_API void xo_epilogue(const float* acc, int M, int N, const uint16_t* residual, int64_t res_ld,
                        uint16_t* aux_out, int64_t aux_ld, const float* row, const float* col,
                        const float* bias, int unary_op, int pair_op, const float* cos_sin,
                        int64_t cs_ld, int cs_period, int compact, uint16_t* out, int64_t out_ld,
                        float* out_f32) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* v = (float*)malloc((size_t)N * sizeof(float));
    for (int n = 0; n < N; ++n) {
      float x = acc[(size_t)m * N + n];
      if (residual) x = x + bf16_to_f32(residual[(size_t)m * res_ld + n]);
      if (aux_out) aux_out[(size_t)m * aux_ld + n] = f32_to_bf16_rne(x);
      if (row) x = x * row[m];
      if (col) x = x * col[n];
      if (bias) x = x + bias[n];
      x = unary(unary_op, x);
      v[n] = x;
    }
    if (pair_op != XO_PAIR_NONE) {
      for (int n = 0; n + 1 < N; n += 2) {
        const float e = v[n], o = v[n + 1];
        if (pair_op == XO_PAIR_SWIGLU) {
          /* xe_pairwise_compute.hpp:71-78: both lanes return silu(gate)*up */
          const float r = silu(e) * o;
          v[n] = r; v[n + 1] = r;
        } else if (pair_op == XO_PAIR_GEGLU) {
          /* xe_pairwise_compute.hpp:82-89 */
          const float r = gelu_erf(e) * o;
          v[n] = r; v[n + 1] = r;
        } else if (pair_op == XO_PAIR_ROPE) {
          /* xe_rope_compute.hpp:51-59; tests/test_k4.cpp:155-166 */
          const int cn = cs_period > 0 ? (n % cs_period) : n;
          const float c = cos_sin[(size_t)m * cs_ld + cn];
          const float s = cos_sin[(size_t)m * cs_ld + cn + 1];
          v[n] = e * c + o * s;
          v[n + 1] = -e * s + o * c;
        } else if (pair_op == XO_PAIR_SWAP) {
          v[n] = o; v[n + 1] = e;
        }
      }
    }
    if (compact) {
      for (int j = 0; j < N / 2; ++j) {
        if (out) out[(size_t)m * out_ld + j] = f32_to_bf16_rne(v[2 * j]);
        if (out_f32) out_f32[(size_t)m * out_ld + j] = v[2 * j];
      }
    } else {
      for (int n = 0; n < N; ++n) {
        if (out) out[(size_t)m * out_ld + n] = f32_to_bf16_rne(v[n]);
        if (out_f32) out_f32[(size_t)m * out_ld + n] = v[n];
      }
    }
    free(v);
  }
}

XO_API void xo_s32_to_f32(const int32_t* src, float* dst, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = (float)src[i];
}

/* ------------------------------------------------------------------ per-preset restatements
 * Written straight from each test's lambda, independently of xo_epilogue, so the tests can check
 * that the flat program above and the preset formulas agree. */

/* k1: tests/test_k1.cpp:119-135  D = acc * scale[m] */
XO_API void xo_preset_k1(const float* acc, const float* scale, int M, int N, uint16_t* out) {
  for (int64_t i = 0; i < (int64_t)M * N; ++i) {
    int m = (int)((i / N) % M);
    out[i] = f32_to_bf16_rne(acc[i] * scale[m]);
  }
}

/* k2: autotune/pipeline_template.cpp.j2:462-477 (fp32 throughout), every column written */
XO_API void xo_preset_k2(const float* acc, const float* scale, int M, int N, int geglu, uint16_t* out) {
  for (int64_t i = 0; i < (int64_t)M * N; ++i) {
    int col = (int)(i % N);
    int row = (int)((i / N) % M);
    int64_t row_base = i - col;
    int even_col = col & ~1, odd_col = even_col + 1;
    float s = scale[row];
    if (odd_col >= N) { out[i] = f32_to_bf16_rne(acc[i] * s); continue; }
    float gate = acc[row_base + even_col] * s;
    float up = acc[row_base + odd_col] * s;
    float a = geglu ? gelu_erf(gate) : gate / (1.0f + expf(-gate));
    out[i] = f32_to_bf16_rne(a * up);
  }
}

/* k3 / k4 / k4v2: tests/test_k3.cpp:137-162, tests/test_k4.cpp:142-173 (scale == NULL => k3) */
XO_API void xo_preset_k4(const float* acc, const float* scale, const float* cos_sin, int M, int N,
                         uint16_t* out) {
  for (int64_t i = 0; i < (int64_t)M * N; ++i) {
    int col = (int)(i % N);
    int row = (int)((i / N) % M);
    int64_t row_base = i - col;
    float s = scale ? scale[row] : 1.0f;
    int even_col = col & ~1, odd_col = even_col + 1;
    if (odd_col >= N) { out[i] = f32_to_bf16_rne(acc[i] * s); continue; }
    float x_even = acc[row_base + even_col] * s;
    float x_odd = acc[row_base + odd_col] * s;
    float cos_val = cos_sin[row_base + even_col];
    float sin_val = cos_sin[row_base + odd_col];
    float o = ((col & 1) == 0) ? (x_even * cos_val + x_odd * sin_val)
                               : (-x_even * sin_val + x_odd * cos_val);
    out[i] = f32_to_bf16_rne(o);
  }
}

/* k0a: tests/test_k0a.cpp:139-150  D = gamma[n] * (acc + residual) */
XO_API void xo_preset_k0a(const float* acc, const uint16_t* residual, const float* gamma, int M,
                          int N, uint16_t* out) {
  for (int64_t i = 0; i < (int64_t)M * N; ++i) {
    int col = (int)(i % N);
    float a = acc[i];
    float r = bf16_to_f32(residual[i]);
    out[i] = f32_to_bf16_rne(gamma[col] * (a + r));
  }
}

/* w8a8 (+bias): include/xe-fuse/standalone/ops.hpp:335-354 and :221-230;
 * autotune/pipeline_w8a8_template.cpp.j2:175-184.  Order (acc*st)*sc, then + bias. */
XO_API void xo_preset_w8a8(const int32_t* acc, const float* scale_token, const float* scale_channel,
                           const float* bias, int M, int N, uint16_t* out) {
  for (int64_t i = 0; i < (int64_t)M * N; ++i) {
    int col = (int)(i % N);
    int m = (int)((i / N) % M);
    float val = (float)acc[i] * scale_token[m] * scale_channel[col];
    if (bias) val = val + bias[col];
    out[i] = f32_to_bf16_rne(val);
  }
}

/* ------------------------------------------------------------------ producers */
/* include/xe-fuse/kernels/compute_rstd.hpp:28-46  R[m] = 1/sqrt(mean(x^2) + eps) */
XO_API void xo_compute_rstd(const uint16_t* x, float* rstd, int M, int N, float eps) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    double ss = 0.0; /* wider than the device's fp32 tree sum; both are within fp32 rounding */
    for (int n = 0; n < N; ++n) {
      float v = bf16_to_f32(x[(size_t)m * N + n]);
      ss += (double)v * v;
    }
    float mean_sq = (float)(ss / (double)N);
    rstd[m] = 1.0f / sqrtf(mean_sq + eps);
  }
}

/* include/xe-fuse/kernels/compute_rstd.hpp:84-121: normalise, absmax/127 + 1e-8, round half away
 * from zero (sycl::round), clamp to [-128,127]. */
XO_API void xo_rstd_and_quantize(const uint16_t* x, const float* rstd, int8_t* xq, float* scale_token,
                                 int M, int N) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const float r = rstd[m];
    float mx = 0.0f;
    for (int n = 0; n < N; ++n) mx = fmaxf(mx, fabsf(bf16_to_f32(x[(size_t)m * N + n]) * r));
    const float sc = mx / 127.0f + 1e-8f;
    for (int n = 0; n < N; ++n) {
      float normed = bf16_to_f32(x[(size_t)m * N + n]) * r;
      float q = roundf(normed / sc);
      q = fminf(fmaxf(q, -128.0f), 127.0f);
      xq[(size_t)m * N + n] = (int8_t)q;
    }
    scale_token[m] = sc;
  }
}

/* autotune/pipeline_w8a8_template.cpp.j2:135-153: per-column absmax/127 + 1e-8, round half away,
 * clamp.  W is [K,N] row-major bf16. */
XO_API void xo_quantize_weight_cols(const uint16_t* W, int8_t* Wq, float* scale_channel, int K, int N) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float mx = 0.0f;
    for (int k = 0; k < K; ++k) mx = fmaxf(mx, fabsf(bf16_to_f32(W[(size_t)k * N + n])));
    const float sc = mx / 127.0f + 1e-8f;
    for (int k = 0; k < K; ++k) {
      float q = roundf(bf16_to_f32(W[(size_t)k * N + n]) / sc);
      q = fminf(fmaxf(q, -128.0f), 127.0f);
      Wq[(size_t)k * N + n] = (int8_t)q;
    }
    scale_channel[n] = sc;
  }
}

/* Per-token absmax symmetric quantisation of an activation row without normalisation
 * (rstd == 1): the input preparation of the W8A8 configuration. */
XO_API void xo_quantize_rows(const uint16_t* x, int8_t* xq, float* scale_token, int M, int N) {
  float* ones = (float*)malloc((size_t)M * sizeof(float));
  for (int m = 0; m < M; ++m) ones[m] = 1.0f;
  xo_rstd_and_quantize(x, ones, xq, scale_token, M, N);
  free(ones);
}

/* RoPE table as the reference's host generator builds it (tests/test_k4.cpp:81-92):
 * cs[m, 2i] = cos(m * theta^(-2i/width)), cs[m, 2i+1] = sin(same); width = N in the reference
 * tests, head_dim for a per-head table. */
XO_API void xo_rope_table(float* cs, int M, int width, float theta) {
  for (int m = 0; m < M; ++m)
    for (int i = 0; i < width / 2; ++i) {
      float freq = 1.0f / powf(theta, 2.0f * i / (float)width);
      float angle = (float)m * freq;
      cs[(size_t)m * width + 2 * i] = cosf(angle);
      cs[(size_t)m * width + 2 * i + 1] = sinf(angle);
    }
}

/* ------------------------------------------------------------------------------------------
 * Engine-style stand-alone passes (include/xe-fuse/standalone/vllm_ops.hpp), the comparison arm
 * of the reference's generated pipelines.  Row sums here run in element order in fp32, as one
 * work-item of the reference would; the device sums the same terms in a tree.
 * ------------------------------------------------------------------------------------------ */

/* vllm_ops.hpp:33-69: out = bf16(x * rsqrt(mean(x^2) + eps) * weight), weight bf16. */
XO_API void xo_ve_rms_norm(uint16_t* out, const uint16_t* in, const uint16_t* weight, int M, int N, float eps) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float var = 0.0f;
    for (int n = 0; n < N; ++n) {
      float x = bf16_to_f32(in[(size_t)m * N + n]);
      var += x * x;
    }
    const float s = 1.0f / sqrtf(var / (float)N + eps);
    for (int n = 0; n < N; ++n) {
      float x = bf16_to_f32(in[(size_t)m * N + n]);
      out[(size_t)m * N + n] = f32_to_bf16_rne(x * s * bf16_to_f32(weight[n]));
    }
  }
}

/* vllm_ops.hpp:75-114: residual = bf16(input + residual) with the variance over the unrounded
 * sums; input = bf16(residual * s * weight) from the rounded residual. */
XO_API void xo_ve_fused_add_rms_norm(uint16_t* input, uint16_t* residual, const uint16_t* weight, int M, int N,
                                     float eps) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float var = 0.0f;
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t)m * N + n;
      float sum = bf16_to_f32(input[i]) + bf16_to_f32(residual[i]);
      var += sum * sum;
      residual[i] = f32_to_bf16_rne(sum);
    }
    const float s = 1.0f / sqrtf(var / (float)N + eps);
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t)m * N + n;
      input[i] = f32_to_bf16_rne(bf16_to_f32(residual[i]) * s * bf16_to_f32(weight[n]));
    }
  }
}

/* vllm_ops.hpp:119-164: out[m,i] = act(in[m,i]) * in[m,d+i]; gelu != 0 selects erf-GeLU. */
XO_API void xo_ve_act_and_mul(uint16_t* out, const uint16_t* in, int d, int M, int gelu) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int i = 0; i < d; ++i) {
      float gate = bf16_to_f32(in[(size_t)m * 2 * d + i]);
      float up = bf16_to_f32(in[(size_t)m * 2 * d + d + i]);
      float a = gelu ? gelu_erf(gate) : silu(gate);
      out[(size_t)m * d + i] = f32_to_bf16_rne(a * up);
    }
}

/* vllm_ops.hpp:170-227: NeoX pairs (h[j], h[rot_dim/2+j]) of every head of one [M,heads,head_size]
 * tensor, cache [M,rot_dim] = cos half | sin half.  Call once for the query and once for the key. */
XO_API void xo_ve_rotary_neox(uint16_t* data, const float* cache, int head_size, int heads, int rot_dim, int M) {
  const int embed = rot_dim / 2;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int h = 0; h < heads; ++h)
      for (int j = 0; j < embed; ++j) {
        uint16_t* base = data + ((size_t)m * heads + h) * head_size;
        float x = bf16_to_f32(base[j]), y = bf16_to_f32(base[embed + j]);
        float c = cache[(size_t)m * rot_dim + j], s = cache[(size_t)m * rot_dim + embed + j];
        base[j] = f32_to_bf16_rne(x * c - y * s);
        base[embed + j] = f32_to_bf16_rne(y * c + x * s);
      }
}

/* vllm_ops.hpp:244-311: rows = L*M; gate/up halves dequantised as (acc*st)*sc, result duplicated. */
XO_API void xo_ve_dequant_act_mul(uint16_t* out, const int32_t* acc, const float* st, const float* sc, int d, int M,
                                  int L, int gelu) {
  const int N = 2 * d;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < M * L; ++r) {
    const int l = r / M;
    for (int i = 0; i < d; ++i) {
      float gate = (float)acc[(size_t)r * N + i] * st[r] * sc[(size_t)l * N + i];
      float up = (float)acc[(size_t)r * N + d + i] * st[r] * sc[(size_t)l * N + d + i];
      uint16_t v = f32_to_bf16_rne((gelu ? gelu_erf(gate) : silu(gate)) * up);
      out[(size_t)r * N + i] = v;
      out[(size_t)r * N + d + i] = v;
    }
  }
}

/* vllm_ops.hpp:317-346: dequantise, then rotate the interleaved pairs with cos_sin [L,M,N]; a last
 * unpaired column is only dequantised. */
XO_API void xo_ve_dequant_rotary(uint16_t* out, const int32_t* acc, const float* st, const float* sc,
                                 const float* cos_sin, int M, int N, int L) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < M * L; ++r) {
    const int l = r / M;
    const size_t base = (size_t)r * N;
    for (int e = 0; e < N; e += 2) {
      float xe = (float)acc[base + e] * st[r] * sc[(size_t)l * N + e];
      if (e + 1 >= N) {
        out[base + e] = f32_to_bf16_rne(xe);
        break;
      }
      float xo = (float)acc[base + e + 1] * st[r] * sc[(size_t)l * N + e + 1];
      float c = cos_sin[base + e], s = cos_sin[base + e + 1];
      out[base + e] = f32_to_bf16_rne(xe * c + xo * s);
      out[base + e + 1] = f32_to_bf16_rne(-xe * s + xo * c);
    }
  }
}
