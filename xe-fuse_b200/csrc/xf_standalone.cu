// Stand-alone (unfused) elementwise passes over bf16 [L][M][N] tensors and the row-reduction
// producers (rstd, activation quantisation).  These are HBM-bound: each thread moves 16-byte
// vectors, grids are sized in whole waves of the SM count, and every kernel reads each input once.
// They exist as the "unfused" arm the fused GEMM epilogues are measured against and as the
// producers of the per-row vectors the fused kernels consume.
//
// Semantics follow include/xe-fuse/standalone/ops.hpp and include/xe-fuse/kernels/compute_rstd.hpp
// of the reference: fp32 math on bf16 data, one round-to-nearest-even back to bf16.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/xefuse_b200.h"
#include "xf_host_util.h"
#include "xf_params.h"

namespace xf {
namespace sa {

enum Op : int {
  OP_SCALE_ROWS, OP_SCALE_COLS, OP_ADD_RESIDUAL, OP_RESIDUAL_GAMMA, OP_SWIGLU, OP_GEGLU, OP_ROPE,
  OP_ROPE_SCALED, OP_UNARY, OP_BIAS_ADD, OP_DEQUANT
};

struct Args {
  void* out;            // bf16 [L*M, N]
  const void* in;       // bf16 source (== out for in-place ops) or int32 accumulator (dequant)
  const void* mat;      // bf16 residual
  const float* rowv;    // per-row vector, indexed by global row (batch*M + m)
  const float* colv;    // per-column vector
  const float* cos_sin; // fp32 [L*M, N]
  long long rows;       // L*M
  int M, N;
  int unary;
  int colv_batched;     // 1: colv index is batch*N + col
};

__device__ __forceinline__ float act(int op, float x) {
  switch (op) {
    case UN_GELU: return x * 0.5f * (1.0f + erff(x * 0.7071067811865475f));
    case UN_GELU_TANH: {
      float x3 = x * x * x;
      return x * 0.5f * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x3)));
    }
    case UN_SILU: return __fdividef(x, 1.0f + __expf(-x));
    case UN_RELU: return x > 0.0f ? x : 0.0f;
    case UN_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-x));
    case UN_EXP: return __expf(x);
    default: return x;
  }
}

template <int VEC>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float (&v)[VEC]) {
  if constexpr (VEC == 8) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      v[2 * t] = __uint_as_float(w[t] << 16);
      v[2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = __bfloat162float(p[i]);
  }
}

template <int VEC>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const float (&v)[VEC]) {
  if constexpr (VEC == 8) {
    uint32_t w[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
      w[t] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = __float2bfloat16_rn(v[i]);
  }
}

template <int VEC>
__device__ __forceinline__ void load_f32(const float* p, float (&v)[VEC]) {
  if constexpr (VEC == 8) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = p[i];
  }
}

// One thread owns VEC consecutive columns of one row; VEC divides N so a vector never straddles
// rows.  Grid-stride loop over all vectors.
template <int OP, int VEC>
__global__ void __launch_bounds__(256) elementwise_kernel(const Args a) {
  const long long vec_per_row = a.N / VEC;
  const long long total = a.rows * vec_per_row;
  for (long long idx = blockIdx.x * 256LL + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * 256LL) {
    const long long row = idx / vec_per_row;
    const int col = static_cast<int>(idx - row * vec_per_row) * VEC;
    const long long off = row * a.N + col;
    float v[VEC];
    if constexpr (OP == OP_DEQUANT) {
      const int* ip = reinterpret_cast<const int*>(a.in) + off;
      if constexpr (VEC == 8) {
        const int4 lo = *reinterpret_cast<const int4*>(ip);
        const int4 hi = *reinterpret_cast<const int4*>(ip + 4);
        v[0] = static_cast<float>(lo.x); v[1] = static_cast<float>(lo.y);
        v[2] = static_cast<float>(lo.z); v[3] = static_cast<float>(lo.w);
        v[4] = static_cast<float>(hi.x); v[5] = static_cast<float>(hi.y);
        v[6] = static_cast<float>(hi.z); v[7] = static_cast<float>(hi.w);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = static_cast<float>(ip[i]);
      }
    } else {
      load_bf16<VEC>(reinterpret_cast<const __nv_bfloat16*>(a.in) + off, v);
    }
    const int batch = static_cast<int>(row / a.M);
    if constexpr (OP == OP_SCALE_ROWS) {
      const float s = a.rowv[row];
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] *= s;
    } else if constexpr (OP == OP_SCALE_COLS) {
      float g[VEC];
      load_f32<VEC>(a.colv + col, g);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] *= g[i];
    } else if constexpr (OP == OP_ADD_RESIDUAL || OP == OP_RESIDUAL_GAMMA) {
      float r[VEC];
      load_bf16<VEC>(reinterpret_cast<const __nv_bfloat16*>(a.mat) + off, r);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] += r[i];
      if constexpr (OP == OP_RESIDUAL_GAMMA) {
        float g[VEC];
        load_f32<VEC>(a.colv + col, g);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] *= g[i];
      }
    } else if constexpr (OP == OP_SWIGLU || OP == OP_GEGLU) {
#pragma unroll
      for (int j = 0; j < VEC / 2; ++j) {
        const float g = v[2 * j], u = v[2 * j + 1];
        const float o = (OP == OP_SWIGLU ? __fdividef(g, 1.0f + __expf(-g))
                                         : g * 0.5f * (1.0f + erff(g * 0.7071067811865475f))) * u;
        v[2 * j] = o;
        v[2 * j + 1] = o;
      }
    } else if constexpr (OP == OP_ROPE || OP == OP_ROPE_SCALED) {
      float cs[VEC];
      load_f32<VEC>(a.cos_sin + off, cs);
      float s = 1.0f;
      if constexpr (OP == OP_ROPE_SCALED) s = a.rowv[row];
#pragma unroll
      for (int j = 0; j < VEC / 2; ++j) {
        const float xe = v[2 * j] * s, xo = v[2 * j + 1] * s;
        v[2 * j] = xe * cs[2 * j] + xo * cs[2 * j + 1];
        v[2 * j + 1] = -xe * cs[2 * j + 1] + xo * cs[2 * j];
      }
    } else if constexpr (OP == OP_UNARY) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = act(a.unary, v[i]);
    } else if constexpr (OP == OP_BIAS_ADD) {
      float b[VEC];
      load_f32<VEC>(a.colv + col, b);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] += b[i];
    } else if constexpr (OP == OP_DEQUANT) {
      const float st = a.rowv[row];
      float sc[VEC];
      load_f32<VEC>(a.colv + static_cast<long long>(batch) * a.N + col, sc);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = v[i] * st * sc[i];
    }
    store_bf16<VEC>(reinterpret_cast<__nv_bfloat16*>(a.out) + off, v);
  }
}

static bool al16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int wave_grid(long long work_items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long blocks = (work_items + 255) / 256;
  long long cap = static_cast<long long>(sms) * 16;  // 16 resident 256-thread blocks fill an SM's 64 warps twice over
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

template <int OP>
static xf_status launch(const Args& a, bool pairwise, cudaStream_t st) {
  if (a.rows <= 0 || a.N <= 0 || a.M <= 0) {
    set_error("standalone op: extents must be positive");
    return XF_ERR_INVALID_PROBLEM;
  }
  if (!a.out || !a.in) {
    set_error("standalone op: null tensor pointer");
    return XF_ERR_INVALID_PROBLEM;
  }
  const bool v8 = (a.N % 8 == 0) && al16(a.out) && al16(a.in) && al16(a.mat) && al16(a.colv) &&
                  al16(a.cos_sin);
  if (v8) {
    const long long total = a.rows * (a.N / 8);
    elementwise_kernel<OP, 8><<<wave_grid(total), 256, 0, st>>>(a);
  } else if (a.N % 2 == 0) {
    const long long total = a.rows * (a.N / 2);
    elementwise_kernel<OP, 2><<<wave_grid(total), 256, 0, st>>>(a);
  } else {
    if (pairwise) {
      set_error("standalone pair op needs an even N (N=%d)", a.N);
      return XF_ERR_INVALID_PROBLEM;
    }
    const long long total = a.rows * a.N;
    elementwise_kernel<OP, 1><<<wave_grid(total), 256, 0, st>>>(a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("standalone kernel launch failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

// ------------------------------------------------------------------------ row reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* red) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < nw) ? red[l] : (IS_MAX ? 0.0f : 0.0f);
  r = IS_MAX ? warp_max(r) : warp_sum(r);
  return r;
}

// One 256-thread block per row; QUANT additionally writes the int8 row and its scale.
template <bool QUANT>
__global__ void __launch_bounds__(256) rstd_kernel(const __nv_bfloat16* __restrict__ x,
                                                   float* __restrict__ rstd_or_scale,
                                                   int8_t* __restrict__ xq, long long rows, int N,
                                                   float eps) {
  __shared__ float red[8];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * N;
    const bool vec = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
    float ss = 0.0f;
    if (vec) {
      for (int c = threadIdx.x * 8; c < N; c += 256 * 8) {
        float v[8];
        load_bf16<8>(xr + c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
      }
    } else {
      for (int c = threadIdx.x; c < N; c += 256) {
        float v = __bfloat162float(xr[c]);
        ss += v * v;
      }
    }
    ss = block_reduce<false>(ss, red);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
    if constexpr (!QUANT) {
      if (threadIdx.x == 0) rstd_or_scale[row] = rstd;
    } else {
      float mx = 0.0f;
      for (int c = threadIdx.x; c < N; c += 256)
        mx = fmaxf(mx, fabsf(__bfloat162float(xr[c]) * rstd));
      mx = block_reduce<true>(mx, red);
      const float scale = mx / 127.0f + 1e-8f;
      int8_t* qr = xq + row * N;
      for (int c = threadIdx.x; c < N; c += 256) {
        float q = roundf(__bfloat162float(xr[c]) * rstd / scale);  // half away from zero
        q = fminf(fmaxf(q, -128.0f), 127.0f);
        qr[c] = static_cast<int8_t>(q);
      }
      if (threadIdx.x == 0) rstd_or_scale[row] = scale;
    }
  }
}

// RMS-normalise + absmax-quantise with ONE pass over HBM: the row is staged in shared memory as it
// is read (16-byte loads), the two reductions and the quantisation then run from shared memory and
// the int8 row is written with 16-byte stores.  Needs N % 16 == 0 and a row that fits shared memory.
__global__ void __launch_bounds__(1024) rstd_quant_smem_kernel(const __nv_bfloat16* __restrict__ x,
                                                              float* __restrict__ scale_out,
                                                              int8_t* __restrict__ xq, long long rows,
                                                              int N, float eps) {
  extern __shared__ __align__(16) unsigned char row_smem[];
  __shared__ float red[32];
  uint4* srow = reinterpret_cast<uint4*>(row_smem);
  const int nvec = N / 8;  // 8 bf16 per 16-byte vector
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * N);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 u = xr[i];
      srow[i] = u;
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float a = __uint_as_float(w[t] << 16), b = __uint_as_float(w[t] & 0xFFFF0000u);
        ss += a * a + b * b;
      }
    }
    ss = block_reduce<false>(ss, red);   // also orders the shared-memory writes before the reads below
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
    float mx = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 u = srow[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        mx = fmaxf(mx, fabsf(__uint_as_float(w[t] << 16) * rstd));
        mx = fmaxf(mx, fabsf(__uint_as_float(w[t] & 0xFFFF0000u) * rstd));
      }
    }
    mx = block_reduce<true>(mx, red);
    const float scale = mx / 127.0f + 1e-8f;
    uint4* qr = reinterpret_cast<uint4*>(xq + row * N);
    for (int i = threadIdx.x; i < nvec / 2; i += blockDim.x) {   // 16 int8 per 16-byte store
      uint32_t o[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint4 u = srow[2 * i + h];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; t += 2) {
          float f[4] = {__uint_as_float(w[t] << 16), __uint_as_float(w[t] & 0xFFFF0000u),
                        __uint_as_float(w[t + 1] << 16), __uint_as_float(w[t + 1] & 0xFFFF0000u)};
          uint32_t packed = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float qv = roundf(__fdiv_rn(f[k] * rstd, scale));   // the reference's exact quotient, half away from zero
            qv = fminf(fmaxf(qv, -128.0f), 127.0f);
            packed |= (static_cast<uint32_t>(static_cast<int>(qv)) & 0xFFu) << (8 * k);
          }
          o[h * 2 + t / 2] = packed;
        }
      }
      qr[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (threadIdx.x == 0) scale_out[row] = scale;
    __syncthreads();  // the next row overwrites the staged one
  }
}

// The same with the row held in registers instead of shared memory: each thread keeps VPT 16-byte
// vectors (8 bf16 each) of the row, the sum of squares and the absolute maximum are reduced
// together (max|x * rstd| == max|x| * rstd: rounding is monotone and rstd > 0), and the int8 row is
// written from the registers.  One HBM read, one write, two block-wide reductions per row; the
// next row a block will take is loaded before the current one is processed.  Rounding uses
// full-rate instructions only: q + 1.5 * 2^23 leaves round-to-nearest-even(q) in the low mantissa
// bits, and a value within 1e-4 of a tie k + 0.5 (rare) is redone with the exact quotient.
// The reference's quantised value, round(normed / scale) with the exact quotient; out of line so the
// rare elements that need it do not cost the common path registers.
__device__ __forceinline__ float exact_quotient_rounded(float normed, float scale) {
  return roundf(__fdiv_rn(normed, scale));
}

// Sum and maximum over the block with one pair of barriers.
__device__ __forceinline__ void block_reduce_sum_max(float& s, float& m, float2* red) {
  s = warp_sum(s);
  m = warp_max(m);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = make_float2(s, m);
  __syncthreads();
  const float2 r = (l < nw) ? red[l] : make_float2(0.0f, 0.0f);
  s = warp_sum(r.x);
  m = warp_max(r.y);
}

// Up to 4 vectors per thread run in blocks of at most 256 threads, four of them per SM (64
// registers): the kernel is bound by instruction issue and by the two barriers per row, and a
// fourth resident block hides more of both than the registers it costs.
template <int VPT>
__global__ void __launch_bounds__(VPT < 8 ? 256 : 512, VPT < 8 ? 4 : 1)
rstd_quant_reg_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ scale_out,
                      int8_t* __restrict__ xq, long long rows, int N, float eps) {
  __shared__ float2 red[32];
  const int nvec = N / 8;
  auto load_row = [&](uint4 (&dst)[VPT], long long row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * N);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      dst[k] = (i < nvec) ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  uint4 v[VPT], vn[VPT];
  if (blockIdx.x < rows) load_row(v, blockIdx.x);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    // the next row's loads are in flight while this one is reduced and quantised
    const long long next = row + gridDim.x;
    if (next < rows) load_row(vn, next);
    float ss = 0.0f, amax = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float a = __uint_as_float(w[t] << 16), b = __uint_as_float(w[t] & 0xFFFF0000u);
        ss += a * a + b * b;
        amax = fmaxf(amax, fmaxf(fabsf(a), fabsf(b)));
      }
    }
    block_reduce_sum_max(ss, amax, red);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
    const float scale = (amax * rstd) / 127.0f + 1e-8f;
    const float inv_scale = 1.0f / scale;   // one division per row; the elements multiply
    uint2* qr = reinterpret_cast<uint2*>(xq + row * N);   // 8 int8 per vector
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
        // |x * rstd| <= amax * rstd < 127 * scale, so q stays inside [-127.5, 127.5]: no clamp needed
        const float kMagic = 12582912.0f;   // 1.5 * 2^23: q + kMagic holds rne(q) in its low mantissa bits
        // q = (x * rstd) * (1 / scale) is within 1.5e-5 of the reference's (x * rstd) / scale (|q| < 128), which
        // decides the rounded value except within that distance of k + 0.5: those few are redone with
        // the exact quotient and rounded half away from zero, so the int8 values equal the
        // reference's whenever rstd does.
        const float kTieWindow = 0.49998f;   // 0.5 - 2e-5: beyond twice the error bound of the product
        float q[8], m[8];
        bool near_tie = false;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          q[2 * t] = (__uint_as_float(w[t] << 16) * rstd) * inv_scale;
          q[2 * t + 1] = (__uint_as_float(w[t] & 0xFFFF0000u) * rstd) * inv_scale;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          m[e] = q[e] + kMagic;
          near_tie |= fabsf(q[e] - (m[e] - kMagic)) > kTieWindow;
        }
        if (near_tie) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (fabsf(q[e] - (m[e] - kMagic)) > kTieWindow) {
              const uint32_t we = w[e >> 1];
              const float xe = (e & 1) ? __uint_as_float(we & 0xFFFF0000u) : __uint_as_float(we << 16);
              m[e] = exact_quotient_rounded(xe * rstd, scale) + kMagic;
            }
        }
        // the low byte of (integer + kMagic)'s bit pattern is the integer's two's-complement byte:
        // three byte permutes gather four of them
        uint32_t o[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t lo = __byte_perm(__float_as_uint(m[4 * h]), __float_as_uint(m[4 * h + 1]), 0x0040);
          const uint32_t hi = __byte_perm(__float_as_uint(m[4 * h + 2]), __float_as_uint(m[4 * h + 3]), 0x0040);
          o[h] = __byte_perm(lo, hi, 0x5410);
        }
        qr[i] = make_uint2(o[0], o[1]);
      }
    }
    if (threadIdx.x == 0) scale_out[row] = scale;
#pragma unroll
    for (int k = 0; k < VPT; ++k) v[k] = vn[k];
  }
}

// rstd[l*M+m] = 1/sqrt(sum_u partials[l][u][m] / N + eps): the finishing pass over the row_sumsq
// side output of a fused GEMM.  One thread per row; consecutive threads read consecutive floats.
__global__ void __launch_bounds__(256) reduce_partials_rsqrt_kernel(const float* __restrict__ partials,
                                                                    float* __restrict__ rstd, int M, int units,
                                                                    long long rows, float inv_n, float eps) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  const long long l = i / M;
  const int m = static_cast<int>(i - l * M);
  const float* p = partials + l * units * static_cast<long long>(M) + m;
  float ss = 0.0f;
  for (int u = 0; u < units; ++u) ss += p[static_cast<long long>(u) * M];
  rstd[i] = 1.0f / sqrtf(ss * inv_n + eps);
}

}  // namespace sa
}  // namespace xf

using xf::sa::Args;
using namespace xf::sa;

static Args mk(void* out, const void* in, int M, int N, int L) {
  Args a = {};
  a.out = out;
  a.in = in;
  a.rows = static_cast<long long>(M) * L;
  a.M = M;
  a.N = N;
  return a;
}

extern "C" {

xf_status xf_sa_scale_rows(void* D, const float* scale, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.rowv = scale;
  if (!scale) { xf::set_error("scale_rows: null scale"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_SCALE_ROWS>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_scale_cols(void* D, const float* scale, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.colv = scale;
  if (!scale) { xf::set_error("scale_cols: null scale"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_SCALE_COLS>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_add_residual(void* D, const void* residual, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.mat = residual;
  if (!residual) { xf::set_error("add_residual: null residual"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_ADD_RESIDUAL>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_residual_gamma(void* D, const void* residual, const float* gamma, int M, int N,
                               int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.mat = residual;
  a.colv = gamma;
  if (!residual || !gamma) { xf::set_error("residual_gamma: null operand"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_RESIDUAL_GAMMA>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_swiglu(void* D, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  return launch<OP_SWIGLU>(a, true, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_geglu(void* D, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  return launch<OP_GEGLU>(a, true, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_rope(void* out, const void* in, const float* cos_sin, int M, int N, int L,
                     void* stream) {
  Args a = mk(out, in, M, N, L);
  a.cos_sin = cos_sin;
  if (!cos_sin) { xf::set_error("rope: null cos_sin"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_ROPE>(a, true, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_rope_scaled(void* out, const void* in, const float* scale, const float* cos_sin,
                            int M, int N, int L, void* stream) {
  Args a = mk(out, in, M, N, L);
  a.rowv = scale;
  a.cos_sin = cos_sin;
  if (!scale || !cos_sin) { xf::set_error("rope_scaled: null operand"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_ROPE_SCALED>(a, true, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_unary(void* D, int unary, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.unary = unary;
  if (unary < XF_UNARY_NONE || unary > XF_UNARY_EXP) {
    xf::set_error("unary: unknown op %d", unary);
    return XF_ERR_NOT_SUPPORTED;
  }
  return launch<OP_UNARY>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_bias_add(void* D, const float* bias, int M, int N, int L, void* stream) {
  Args a = mk(D, D, M, N, L);
  a.colv = bias;
  if (!bias) { xf::set_error("bias_add: null bias"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_BIAS_ADD>(a, false, static_cast<cudaStream_t>(stream));
}

xf_status xf_sa_dequant_w8a8(void* out, const int32_t* acc, const float* scale_token,
                             const float* scale_channel, int M, int N, int L, void* stream) {
  Args a = mk(out, acc, M, N, L);
  a.rowv = scale_token;
  a.colv = scale_channel;
  if (!scale_token || !scale_channel) { xf::set_error("dequant_w8a8: null scale"); return XF_ERR_INVALID_PROBLEM; }
  return launch<OP_DEQUANT>(a, false, static_cast<cudaStream_t>(stream));
}

static xf_status launch_rstd(const void* x, float* out, int8_t* xq, int M, int N, int L, float eps,
                             void* stream) {
  if (!x || !out || M <= 0 || N <= 0 || L <= 0) {
    xf::set_error("compute_rstd: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  const long long rows = static_cast<long long>(M) * L;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long grid = rows < static_cast<long long>(sms) * 8 ? rows : static_cast<long long>(sms) * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t row_bytes = static_cast<size_t>(N) * 2;
  const bool one_pass = xq && (N % 16 == 0) && row_bytes <= 96 * 1024 &&
                        (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15) == 0;
  const int nvec = N / 8;
  const bool in_regs = xq && (N % 8 == 0) && nvec <= 4096 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(xq) & 7) == 0;
  if (in_regs) {
    // the fewest vectors per thread that keep the block at 256 threads or fewer (many rows in
    // flight per SM); rows beyond 8 x 256 vectors take 8 per thread and up to 512 threads
    const auto* xb = static_cast<const __nv_bfloat16*>(x);
    const int g = static_cast<int>(grid);
    int vpt = 1;
    while (vpt < 8 && (nvec + vpt - 1) / vpt > 256) vpt *= 2;
    int threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32;
    if (threads < 64) threads = 64;
    switch (vpt) {
      case 1: xf::sa::rstd_quant_reg_kernel<1><<<g, threads, 0, st>>>(xb, out, xq, rows, N, eps); break;
      case 2: xf::sa::rstd_quant_reg_kernel<2><<<g, threads, 0, st>>>(xb, out, xq, rows, N, eps); break;
      case 4: xf::sa::rstd_quant_reg_kernel<4><<<g, threads, 0, st>>>(xb, out, xq, rows, N, eps); break;
      default: xf::sa::rstd_quant_reg_kernel<8><<<g, threads, 0, st>>>(xb, out, xq, rows, N, eps); break;
    }
  } else if (one_pass) {
    if (row_bytes > 48 * 1024)
      cudaFuncSetAttribute(xf::sa::rstd_quant_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(row_bytes));
    // enough threads per block that a few staged rows fill the SM's thread slots
    const int threads = row_bytes > 32 * 1024 ? 1024 : (row_bytes > 16 * 1024 ? 512 : 256);
    xf::sa::rstd_quant_smem_kernel<<<static_cast<int>(grid), threads, row_bytes, st>>>(
        static_cast<const __nv_bfloat16*>(x), out, xq, rows, N, eps);
  } else if (xq)
    xf::sa::rstd_kernel<true><<<static_cast<int>(grid), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), out, xq, rows, N, eps);
  else
    xf::sa::rstd_kernel<false><<<static_cast<int>(grid), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), out, nullptr, rows, N, eps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    xf::set_error("compute_rstd launch failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

xf_status xf_compute_rstd(const void* x, float* rstd, int M, int N, int L, float eps, void* stream) {
  return launch_rstd(x, rstd, nullptr, M, N, L, eps, stream);
}

xf_status xf_compute_rstd_and_quantize(const void* x, int8_t* xq, float* scale_token, int M, int N,
                                       int L, float eps, void* stream) {
  if (!xq) {
    xf::set_error("compute_rstd_and_quantize: null int8 output");
    return XF_ERR_INVALID_PROBLEM;
  }
  return launch_rstd(x, scale_token, xq, M, N, L, eps, stream);
}

size_t xf_row_sumsq_count(int M, int N, int L) {
  if (M <= 0 || N <= 0 || L <= 0) return 0;
  return static_cast<size_t>(L) * static_cast<size_t>((N + 31) / 32) * static_cast<size_t>(M);
}

xf_status xf_reduce_partials_rsqrt(const float* partials, float* rstd, int M, int N, int L, float eps,
                                   void* stream) {
  if (!partials || !rstd || M <= 0 || N <= 0 || L <= 0) {
    xf::set_error("reduce_partials_rsqrt: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  const long long rows = static_cast<long long>(M) * L;
  const int grid = static_cast<int>((rows + 255) / 256);
  xf::sa::reduce_partials_rsqrt_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partials, rstd, M, (N + 31) / 32, rows, 1.0f / static_cast<float>(N), eps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    xf::set_error("reduce_partials_rsqrt launch failed: %s", cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

}  // extern "C"
