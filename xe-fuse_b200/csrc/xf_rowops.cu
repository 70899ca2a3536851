// Row-wise and merged elementwise passes in the style of an inference engine's stand-alone
// kernels: RMSNorm with a bf16 weight, residual-add + RMSNorm, act(gate) * up over [M, 2d] halves,
// NeoX-style rotary embedding over [M, heads, head_size], and the int8 forms that read an int32
// GEMM accumulator and apply the W8A8 dequantisation and the activation / rotation in one pass.
//
// They are the "engine-equivalent" comparison arm of the reference's generated pipelines
// (include/xe-fuse/standalone/vllm_ops.hpp:33-346): bare GEMM -> one of these -> bare GEMM, against
// the fused epilogues.  All are HBM-bound.  Each kernel reads every input element once: the
// normalising kernels keep the row in shared memory between the sum of squares and the scaling,
// the others move 16-byte vectors through registers.  Arithmetic is fp32 on bf16/int32 data with
// one round-to-nearest-even back to bf16, in the reference's operation order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/xefuse_b200.h"
#include "xf_host_util.h"

namespace xf {
namespace rowops {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = (l < nw) ? red[l] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// out[m,:] = bf16( x[m,:] * rsqrt(mean(x[m,:]^2) + eps) * weight[:] ), x = input, or for ADD
// x = bf16(input + residual) which is also written back to residual (the sum of squares uses the
// unrounded sum, the scaling the rounded one, as the reference's two loops do).
// One block (256-1024 threads) per row, the row staged in shared memory as 16-byte vectors: one
// HBM read per element.
// out may alias input.
template <bool ADD>
__global__ void __launch_bounds__(1024) rmsnorm_smem_kernel(__nv_bfloat16* out, const __nv_bfloat16* input,
                                                           __nv_bfloat16* residual,
                                                           const __nv_bfloat16* __restrict__ weight,
                                                           long long rows, int N, float eps) {
  extern __shared__ __align__(16) unsigned char row_smem[];
  __shared__ float red[32];
  uint4* srow = reinterpret_cast<uint4*>(row_smem);
  const int nvec = N / 8;
  const uint4* wv = reinterpret_cast<const uint4*>(weight);
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(input + row * N);
    uint4* rr = ADD ? reinterpret_cast<uint4*>(residual + row * N) : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      uint4 u = xr[i];
      if (ADD) {
        const uint4 r = rr[i];
        const uint32_t a[4] = {u.x, u.y, u.z, u.w}, b[4] = {r.x, r.y, r.z, r.w};
        uint32_t o[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float s0 = bf_lo(a[t]) + bf_lo(b[t]), s1 = bf_hi(a[t]) + bf_hi(b[t]);
          ss += s0 * s0 + s1 * s1;
          o[t] = pack2(s0, s1);
        }
        u = make_uint4(o[0], o[1], o[2], o[3]);
        rr[i] = u;
      } else {
        const uint32_t a[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) ss += bf_lo(a[t]) * bf_lo(a[t]) + bf_hi(a[t]) * bf_hi(a[t]);
      }
      srow[i] = u;
    }
    ss = block_sum(ss, red);   // its barriers also order the staging writes before the reads below
    const float s = rsqrtf(ss / static_cast<float>(N) + eps);
    uint4* orow = reinterpret_cast<uint4*>(out + row * N);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 u = srow[i], w = wv[i];
      const uint32_t a[4] = {u.x, u.y, u.z, u.w}, g[4] = {w.x, w.y, w.z, w.w};
      uint32_t o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
        o[t] = pack2(bf_lo(a[t]) * s * bf_lo(g[t]), bf_hi(a[t]) * s * bf_hi(g[t]));
      orow[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();   // the next row overwrites the staged one
  }
}

// The same without staging or vectors, for rows that are unaligned, ragged or larger than shared
// memory: two passes over global memory.
template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_plain_kernel(__nv_bfloat16* out, const __nv_bfloat16* input,
                                                            __nv_bfloat16* residual,
                                                            const __nv_bfloat16* __restrict__ weight,
                                                            long long rows, int N, float eps) {
  __shared__ float red[32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = input + row * N;
    __nv_bfloat16* rr = ADD ? residual + row * N : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < N; i += 256) {
      float x = __bfloat162float(xr[i]);
      if (ADD) {
        x += __bfloat162float(rr[i]);
        rr[i] = __float2bfloat16_rn(x);
      }
      ss += x * x;
    }
    ss = block_sum(ss, red);
    const float s = rsqrtf(ss / static_cast<float>(N) + eps);
    const __nv_bfloat16* src = ADD ? rr : xr;
    __nv_bfloat16* orow = out + row * N;
    for (int i = threadIdx.x; i < N; i += 256)
      orow[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * s * __bfloat162float(weight[i]));
    __syncthreads();
  }
}

__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }
// erf-GeLU, g * 0.5 * (1 + erf(g / sqrt 2)), with erf from the five-term rational approximation of
// Abramowitz & Stegun 7.1.26 (absolute error below 1.5e-7): 1 - erf(z) = P(t) exp(-z^2),
// t = 1 / (1 + p z), z >= 0.  For negative g the factor 1 + erf is formed directly as P(t) exp(-z^2),
// so the far tail does not cancel.  A third of the instructions of erff().
__device__ __forceinline__ float gelu_f(float g) {
  const float z = fabsf(g) * 0.7071067811865475f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  const float pe = p * t * __expf(-z * z);         // 1 - erf(z)
  return g * 0.5f * (g >= 0.0f ? 2.0f - pe : pe);
}

// out[m, i] = act(in[m, i]) * in[m, d + i]; in is [M, 2d] (gate half, then up half), out [M, d].
// VEC: 8 columns per thread per step (16-byte loads and stores).  The reference's pipelines call
// this with out == in; rows then overwrite one another's inputs exactly as they do there, so no
// no-alias promise is made to the compiler.
template <bool GELU, bool VEC>
__global__ void __launch_bounds__(256) act_and_mul_kernel(__nv_bfloat16* out, const __nv_bfloat16* in, int d,
                                                          long long M) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (VEC) {
    const int dv = d / 8;
    const long long total = M * dv;
    for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total; w += stride) {
      const long long row = w / dv;
      const int v = static_cast<int>(w - row * dv);
      const uint4* gp = reinterpret_cast<const uint4*>(in + row * 2 * d) + v;
      const uint4 g = gp[0], u = gp[dv];
      const uint32_t ga[4] = {g.x, g.y, g.z, g.w}, ua[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float g0 = bf_lo(ga[t]), g1 = bf_hi(ga[t]);
        const float a0 = GELU ? gelu_f(g0) : silu_f(g0), a1 = GELU ? gelu_f(g1) : silu_f(g1);
        o[t] = pack2(a0 * bf_lo(ua[t]), a1 * bf_hi(ua[t]));
      }
      reinterpret_cast<uint4*>(out + row * d)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    const long long total = M * d;
    for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total; w += stride) {
      const long long row = w / d;
      const int i = static_cast<int>(w - row * d);
      const float g = __bfloat162float(in[row * 2 * d + i]), u = __bfloat162float(in[row * 2 * d + d + i]);
      out[row * d + i] = __float2bfloat16_rn((GELU ? gelu_f(g) : silu_f(g)) * u);
    }
  }
}

// NeoX-style rotary embedding, in place.  data is [M, heads, head_size]; within a head the pair is
// (x, y) = (h[j], h[rot_dim/2 + j]) and becomes (x c - y s, y c + x s) with c = cache[m, j],
// s = cache[m, rot_dim/2 + j].  One launch covers the query heads and, if given, the key heads.
// VEC: 8 values of j per thread per step.
template <bool VEC>
__global__ void __launch_bounds__(256) rotary_neox_kernel(__nv_bfloat16* query, __nv_bfloat16* key,
                                                          const float* __restrict__ cache, int head_size,
                                                          int num_heads, int num_kv_heads, int rot_dim,
                                                          long long M) {
  const int embed = rot_dim / 2;
  const int heads_all = num_heads + (key ? num_kv_heads : 0);
  const int per_head = VEC ? embed / 8 : embed;
  const long long total = M * heads_all * per_head;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total; w += stride) {
    const int j = static_cast<int>(w % per_head);
    const long long th = w / per_head;
    const int head = static_cast<int>(th % heads_all);
    const long long tok = th / heads_all;
    __nv_bfloat16* base = head < num_heads
                              ? query + (tok * num_heads + head) * head_size
                              : key + (tok * num_kv_heads + (head - num_heads)) * head_size;
    const float* cp = cache + tok * rot_dim;
    if (VEC) {
      uint4* xp = reinterpret_cast<uint4*>(base) + j;
      uint4* yp = reinterpret_cast<uint4*>(base + embed) + j;
      const uint4 xv = *xp, yv = *yp;
      const float4 c0 = reinterpret_cast<const float4*>(cp)[2 * j], c1 = reinterpret_cast<const float4*>(cp)[2 * j + 1];
      const float4 s0 = reinterpret_cast<const float4*>(cp + embed)[2 * j],
                   s1 = reinterpret_cast<const float4*>(cp + embed)[2 * j + 1];
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const uint32_t xa[4] = {xv.x, xv.y, xv.z, xv.w}, ya[4] = {yv.x, yv.y, yv.z, yv.w};
      uint32_t xo[4], yo[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float x0 = bf_lo(xa[t]), x1 = bf_hi(xa[t]), y0 = bf_lo(ya[t]), y1 = bf_hi(ya[t]);
        xo[t] = pack2(x0 * c[2 * t] - y0 * s[2 * t], x1 * c[2 * t + 1] - y1 * s[2 * t + 1]);
        yo[t] = pack2(y0 * c[2 * t] + x0 * s[2 * t], y1 * c[2 * t + 1] + x1 * s[2 * t + 1]);
      }
      *xp = make_uint4(xo[0], xo[1], xo[2], xo[3]);
      *yp = make_uint4(yo[0], yo[1], yo[2], yo[3]);
    } else {
      const float x = __bfloat162float(base[j]), y = __bfloat162float(base[embed + j]);
      const float c = cp[j], s = cp[embed + j];
      base[j] = __float2bfloat16_rn(x * c - y * s);
      base[embed + j] = __float2bfloat16_rn(y * c + x * s);
    }
  }
}

// int32 accumulator [L, M, 2d] -> bf16 [L, M, 2d]: gate = acc[i] st sc[i], up = acc[d+i] st sc[d+i],
// r = act(gate) up, written to both out[i] and out[d+i].  VEC: 4 columns per thread per step.
template <bool GELU, bool VEC>
__global__ void __launch_bounds__(256) dequant_act_mul_kernel(__nv_bfloat16* __restrict__ out,
                                                              const int32_t* __restrict__ acc,
                                                              const float* __restrict__ scale_token,
                                                              const float* __restrict__ scale_channel,
                                                              int d, int M, long long rows) {
  const int N = 2 * d;
  const int per_row = VEC ? d / 4 : d;
  const long long total = rows * per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total; w += stride) {
    const long long row = w / per_row;          // l * M + m
    const int v = static_cast<int>(w - row * per_row);
    const long long l = row / M;
    const float st = scale_token[row];
    const int32_t* ar = acc + row * N;
    const float* sc = scale_channel + l * N;
    __nv_bfloat16* orow = out + row * N;
    if (VEC) {
      const int4 g = reinterpret_cast<const int4*>(ar)[v], u = reinterpret_cast<const int4*>(ar + d)[v];
      const float4 sg = reinterpret_cast<const float4*>(sc)[v], su = reinterpret_cast<const float4*>(sc + d)[v];
      const int gi[4] = {g.x, g.y, g.z, g.w}, ui[4] = {u.x, u.y, u.z, u.w};
      const float sgf[4] = {sg.x, sg.y, sg.z, sg.w}, suf[4] = {su.x, su.y, su.z, su.w};
      float r[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float gate = static_cast<float>(gi[t]) * st * sgf[t];
        const float up = static_cast<float>(ui[t]) * st * suf[t];
        r[t] = (GELU ? gelu_f(gate) : silu_f(gate)) * up;
      }
      const uint2 o = make_uint2(pack2(r[0], r[1]), pack2(r[2], r[3]));
      reinterpret_cast<uint2*>(orow)[v] = o;
      reinterpret_cast<uint2*>(orow + d)[v] = o;
    } else {
      const float gate = static_cast<float>(ar[v]) * st * sc[v];
      const float up = static_cast<float>(ar[d + v]) * st * sc[d + v];
      const __nv_bfloat16 r = __float2bfloat16_rn((GELU ? gelu_f(gate) : silu_f(gate)) * up);
      orow[v] = r;
      orow[d + v] = r;
    }
  }
}

// int32 accumulator [L, M, N] -> bf16 with the W8A8 dequantisation and the interleaved-pair
// rotation: x = acc st sc; (e, o) = (x[2k], x[2k+1]) -> (e c + o s, -e s + o c) with
// c = cos_sin[l, m, 2k], s = cos_sin[l, m, 2k+1]; a last unpaired column is only dequantised.
// One pair per thread per step; VEC: four pairs (two 16-byte accumulator loads, one 16-byte store).
template <bool VEC>
__global__ void __launch_bounds__(256) dequant_rotary_kernel(__nv_bfloat16* __restrict__ out,
                                                             const int32_t* __restrict__ acc,
                                                             const float* __restrict__ scale_token,
                                                             const float* __restrict__ scale_channel,
                                                             const float* __restrict__ cos_sin, int M, int N,
                                                             long long rows) {
  const int per_row = VEC ? N / 8 : (N + 1) / 2;
  const long long total = rows * per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; w < total; w += stride) {
    const long long row = w / per_row;
    const int v = static_cast<int>(w - row * per_row);
    const long long l = row / M;
    const float st = scale_token[row];
    const long long base = row * N;
    const float* sc = scale_channel + l * N;
    if (VEC) {
      const int4 a0 = reinterpret_cast<const int4*>(acc + base)[2 * v], a1 = reinterpret_cast<const int4*>(acc + base)[2 * v + 1];
      const float4 s0 = reinterpret_cast<const float4*>(sc)[2 * v], s1 = reinterpret_cast<const float4*>(sc)[2 * v + 1];
      const float4 c0 = reinterpret_cast<const float4*>(cos_sin + base)[2 * v],
                   c1 = reinterpret_cast<const float4*>(cos_sin + base)[2 * v + 1];
      const int ai[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float sf[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      const float cf[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      uint32_t o[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float e = static_cast<float>(ai[2 * t]) * st * sf[2 * t];
        const float od = static_cast<float>(ai[2 * t + 1]) * st * sf[2 * t + 1];
        const float c = cf[2 * t], s = cf[2 * t + 1];
        o[t] = pack2(e * c + od * s, -e * s + od * c);
      }
      reinterpret_cast<uint4*>(out + base)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
      const int ce = 2 * v, co = ce + 1;
      const float e = static_cast<float>(acc[base + ce]) * st * sc[ce];
      if (co >= N) {
        out[base + ce] = __float2bfloat16_rn(e);
        continue;
      }
      const float od = static_cast<float>(acc[base + co]) * st * sc[co];
      const float c = cos_sin[base + ce], s = cos_sin[base + co];
      out[base + ce] = __float2bfloat16_rn(e * c + od * s);
      out[base + co] = __float2bfloat16_rn(-e * s + od * c);
    }
  }
}

static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Blocks for a grid-stride kernel: whole waves of the SM count, 8 blocks of 256 threads per SM.
static int wave_grid(long long work_items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long blocks = (work_items + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

static xf_status launched(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s launch failed: %s", what, cudaGetErrorString(e));
    return XF_ERR_INTERNAL;
  }
  return XF_SUCCESS;
}

template <bool ADD>
static xf_status launch_rmsnorm(void* out, const void* input, void* residual, const void* weight, int M,
                                int N, float eps, void* stream) {
  if (!out || !input || !weight || (ADD && !residual) || M <= 0 || N <= 0) {
    set_error("rms_norm: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = M;
  const int grid = wave_grid(rows * 256);
  const size_t row_bytes = static_cast<size_t>(N) * 2;
  const bool staged = (N % 8 == 0) && row_bytes <= 96 * 1024 && al16(out) && al16(input) && al16(weight) &&
                      (!ADD || al16(residual));
  auto* o = static_cast<__nv_bfloat16*>(out);
  auto* in = static_cast<const __nv_bfloat16*>(input);
  auto* res = static_cast<__nv_bfloat16*>(residual);
  auto* w = static_cast<const __nv_bfloat16*>(weight);
  if (staged) {
    if (row_bytes > 48 * 1024)
      cudaFuncSetAttribute(rmsnorm_smem_kernel<ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(row_bytes));
    // enough threads per block that the few staged rows an SM can hold fill its thread slots
    const int threads = row_bytes > 32 * 1024 ? 1024 : (row_bytes > 16 * 1024 ? 512 : 256);
    rmsnorm_smem_kernel<ADD><<<grid, threads, row_bytes, st>>>(o, in, res, w, rows, N, eps);
  } else {
    rmsnorm_plain_kernel<ADD><<<grid, 256, 0, st>>>(o, in, res, w, rows, N, eps);
  }
  return launched(ADD ? "fused_add_rms_norm" : "rms_norm");
}

}  // namespace rowops
}  // namespace xf

extern "C" {

using namespace xf::rowops;
typedef __nv_bfloat16 bf16_t;

xf_status xf_ve_rms_norm(void* out, const void* input, const void* weight, int M, int N, float eps,
                         void* stream) {
  return launch_rmsnorm<false>(out, input, nullptr, weight, M, N, eps, stream);
}

xf_status xf_ve_fused_add_rms_norm(void* input, void* residual, const void* weight, int M, int N, float eps,
                                   void* stream) {
  return launch_rmsnorm<true>(input, input, residual, weight, M, N, eps, stream);
}

xf_status xf_ve_act_and_mul(void* out, const void* input, int d, int M, int gelu, void* stream) {
  if (!out || !input || d <= 0 || M <= 0) {
    xf::set_error("act_and_mul: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* o = static_cast<bf16_t*>(out);
  auto* in = static_cast<const bf16_t*>(input);
  const bool vec = (d % 8 == 0) && al16(out) && al16(input);
  const int grid = wave_grid(static_cast<long long>(M) * (vec ? d / 8 : d));
  if (vec) {
    if (gelu) act_and_mul_kernel<true, true><<<grid, 256, 0, st>>>(o, in, d, M);
    else act_and_mul_kernel<false, true><<<grid, 256, 0, st>>>(o, in, d, M);
  } else {
    if (gelu) act_and_mul_kernel<true, false><<<grid, 256, 0, st>>>(o, in, d, M);
    else act_and_mul_kernel<false, false><<<grid, 256, 0, st>>>(o, in, d, M);
  }
  return launched("act_and_mul");
}

xf_status xf_ve_rotary_embedding(void* query, void* key, const float* cos_sin_cache, int head_size,
                                 int num_heads, int num_kv_heads, int rot_dim, int M, void* stream) {
  if (!query || !cos_sin_cache || head_size <= 0 || num_heads <= 0 || M <= 0 || rot_dim <= 0 ||
      (rot_dim & 1) || rot_dim > head_size || (key && num_kv_heads <= 0)) {
    xf::set_error("rotary_embedding: bad arguments (rot_dim must be even and <= head_size)");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int embed = rot_dim / 2;
  // 16-byte vectors need every head base, the y half and the cache rows on 16-byte boundaries
  const bool vec = (embed % 8 == 0) && (head_size % 8 == 0) && al16(query) && (!key || al16(key)) &&
                   al16(cos_sin_cache);
  const int heads_all = num_heads + (key ? num_kv_heads : 0);
  const int grid = wave_grid(static_cast<long long>(M) * heads_all * (vec ? embed / 8 : embed));
  auto* q = static_cast<bf16_t*>(query);
  auto* k = static_cast<bf16_t*>(key);
  if (vec) rotary_neox_kernel<true><<<grid, 256, 0, st>>>(q, k, cos_sin_cache, head_size, num_heads, num_kv_heads, rot_dim, M);
  else rotary_neox_kernel<false><<<grid, 256, 0, st>>>(q, k, cos_sin_cache, head_size, num_heads, num_kv_heads, rot_dim, M);
  return launched("rotary_embedding");
}

xf_status xf_ve_dequant_act_mul(void* out, const int32_t* acc, const float* scale_token,
                                const float* scale_channel, int d, int M, int L, int gelu, void* stream) {
  if (!out || !acc || !scale_token || !scale_channel || d <= 0 || M <= 0 || L <= 0) {
    xf::set_error("dequant_act_mul: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = static_cast<long long>(M) * L;
  const bool vec = (d % 4 == 0) && al16(acc) && al16(scale_channel) && al16(out);   // out: 8-byte stores
  const int grid = wave_grid(rows * (vec ? d / 4 : d));
  auto* o = static_cast<bf16_t*>(out);
  if (vec) {
    if (gelu) dequant_act_mul_kernel<true, true><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, d, M, rows);
    else dequant_act_mul_kernel<false, true><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, d, M, rows);
  } else {
    if (gelu) dequant_act_mul_kernel<true, false><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, d, M, rows);
    else dequant_act_mul_kernel<false, false><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, d, M, rows);
  }
  return launched("dequant_act_mul");
}

xf_status xf_ve_dequant_rotary(void* out, const int32_t* acc, const float* scale_token,
                               const float* scale_channel, const float* cos_sin, int M, int N, int L,
                               void* stream) {
  if (!out || !acc || !scale_token || !scale_channel || !cos_sin || M <= 0 || N <= 0 || L <= 0) {
    xf::set_error("dequant_rotary: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = static_cast<long long>(M) * L;
  const bool vec = (N % 8 == 0) && al16(acc) && al16(scale_channel) && al16(cos_sin) && al16(out);
  const int grid = wave_grid(rows * (vec ? N / 8 : (N + 1) / 2));
  auto* o = static_cast<bf16_t*>(out);
  if (vec) dequant_rotary_kernel<true><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, cos_sin, M, N, rows);
  else dequant_rotary_kernel<false><<<grid, 256, 0, st>>>(o, acc, scale_token, scale_channel, cos_sin, M, N, rows);
  return launched("dequant_rotary");
}

}  // extern "C"
