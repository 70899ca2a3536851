// Device utilities behind the harness headers of the front end (initialize_block, GemmComplex,
// BlockCompareRelativelyEqual).  They rebuild expected results the way the reference's harness
// mains do -- on the device, with deliberately simple kernels -- and are not part of the fused path.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/xefuse_b200.h"
#include "xf_host_util.h"
#include "xf_params.h"

namespace xf {
namespace harness {

__device__ __forceinline__ uint64_t mix64(uint64_t x) {  // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <class T> __device__ __forceinline__ T from_int(int v);
template <> __device__ __forceinline__ float from_int<float>(int v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_int<__nv_bfloat16>(int v) { return __float2bfloat16_rn(static_cast<float>(v)); }
template <> __device__ __forceinline__ int8_t from_int<int8_t>(int v) { return static_cast<int8_t>(v); }
template <> __device__ __forceinline__ int32_t from_int<int32_t>(int v) { return v; }

template <class T>
__global__ void fill_uniform_kernel(T* p, long long n, uint64_t seed, int lo, int span) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += gridDim.x * 256LL) {
    const uint64_t h = mix64(seed * 0x100000001B3ull + static_cast<uint64_t>(i));
    p[i] = from_int<T>(lo + static_cast<int>(h % static_cast<uint64_t>(span)));
  }
}

template <class T> __device__ __forceinline__ float to_f(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ int32_t from_f<int32_t>(float v) { return static_cast<int32_t>(v); }
template <> __device__ __forceinline__ int8_t from_f<int8_t>(float v) { return static_cast<int8_t>(v); }

// D[m,n] = alpha * sum_k A[m,k]*B[k,n] + beta*C[m,n]; 32x32 output tile per block, k in order.
// Each 32-term block of products is summed in fp32 and the blocks in fp64, so the reference carries
// no accumulation error of its own to speak of (and integer inputs stay exact far beyond 2^24).
template <class TA, class TC, class TD>
__global__ void __launch_bounds__(1024) ref_gemm_kernel(const TA* A, long long lda, long long ba, const TA* B,
                                                        long long ldb, long long bb, const TC* C,
                                                        long long ldc, long long bc, TD* D, long long ldd,
                                                        long long bd, int M, int N, int K, float alpha,
                                                        float beta) {
  __shared__ float sa[32][33];
  __shared__ float sb[32][33];
  const int l = blockIdx.z;
  const int m = blockIdx.y * 32 + threadIdx.y;
  const int n = blockIdx.x * 32 + threadIdx.x;
  A += l * ba; B += l * bb; D += l * bd;
  if (C) C += l * bc;
  double acc = 0.0;
  for (int k0 = 0; k0 < K; k0 += 32) {
    const int ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
    sa[threadIdx.y][threadIdx.x] = (m < M && ka < K) ? to_f(A[(long long)m * lda + ka]) : 0.f;
    sb[threadIdx.y][threadIdx.x] = (kb < K && n < N) ? to_f(B[(long long)kb * ldb + n]) : 0.f;
    __syncthreads();
    float part = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) part = fmaf(sa[threadIdx.y][k], sb[k][threadIdx.x], part);
    acc += static_cast<double>(part);
    __syncthreads();
  }
  if (m < M && n < N) {
    double v = static_cast<double>(alpha) * acc;
    if (C && beta != 0.f) v += static_cast<double>(beta) * to_f(C[(long long)m * ldc + n]);
    if constexpr (sizeof(TD) == 4 && !std::is_same<TD, float>::value)
      D[(long long)m * ldd + n] = static_cast<TD>(llrint(v));   // int32 output: exact
    else
      D[(long long)m * ldd + n] = from_f<TD>(static_cast<float>(v));
  }
}

__device__ unsigned long long g_mismatches;
__device__ unsigned long long g_first_mismatch;
// the first kListMax disagreements found (in no particular order), for the verbose listing
static const int kListMax = 64;
__device__ unsigned int g_list_count;
__device__ unsigned long long g_list_index[kListMax];
__device__ float g_list_a[kListMax];
__device__ float g_list_b[kListMax];

template <class T>
__global__ void compare_kernel(const T* a, const T* b, long long n, float eps, float floor_) {
  unsigned long long local = 0;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += gridDim.x * 256LL) {
    const float x = to_f(a[i]), y = to_f(b[i]);
    bool ok;
    if (x == y) ok = true;
    else {
      const float d = fabsf(x - y);
      if (x == 0.f || y == 0.f || (fabsf(x) + fabsf(y)) < floor_) ok = d < eps * floor_;
      else ok = d < eps * (fabsf(x) + fabsf(y));
      if (!(d == d)) ok = false;  // NaN
    }
    if (!ok) {
      ++local;
      atomicMin(&g_first_mismatch, static_cast<unsigned long long>(i));
      const unsigned int slot = atomicAdd(&g_list_count, 1u);
      if (slot < kListMax) {
        g_list_index[slot] = static_cast<unsigned long long>(i);
        g_list_a[slot] = x;
        g_list_b[slot] = y;
      }
    }
  }
  if (local) atomicAdd(&g_mismatches, local);
}

static int grid_for(long long n) {
  long long b = (n + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace harness
}  // namespace xf

using namespace xf::harness;

extern "C" {

xf_status xf_harness_fill_uniform(int dtype, void* ptr, long long n, uint64_t seed, int lo, int hi,
                                  void* stream) {
  if (n == 0) return XF_SUCCESS;
  if (!ptr || n < 0 || hi < lo) {
    xf::set_error("fill_uniform: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int span = hi - lo + 1;
  switch (dtype) {
    case XF_DT_BF16: fill_uniform_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<__nv_bfloat16*>(ptr), n, seed, lo, span); break;
    case XF_DT_F32: fill_uniform_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<float*>(ptr), n, seed, lo, span); break;
    case XF_DT_S8: fill_uniform_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<int8_t*>(ptr), n, seed, lo, span); break;
    case XF_DT_S32: fill_uniform_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<int32_t*>(ptr), n, seed, lo, span); break;
    default: xf::set_error("fill_uniform: unknown dtype %d", dtype); return XF_ERR_INVALID_DATA_TYPE;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { xf::set_error("fill_uniform launch: %s", cudaGetErrorString(e)); return XF_ERR_INTERNAL; }
  return XF_SUCCESS;
}

#define XF_REF_GEMM(TA, TC, TD)                                                                     \
  ref_gemm_kernel<TA, TC, TD><<<grid, block, 0, st>>>(static_cast<const TA*>(A), lda, batch_a,      \
      static_cast<const TA*>(B), ldb, batch_b, static_cast<const TC*>(C), ldc, batch_c,             \
      static_cast<TD*>(D), ldd, batch_d, M, N, K, alpha, beta)

xf_status xf_harness_ref_gemm(int dtype_a, const void* A, int64_t lda, int64_t batch_a, int dtype_b,
                              const void* B, int64_t ldb, int64_t batch_b, int dtype_c, const void* C,
                              int64_t ldc, int64_t batch_c, int dtype_d, void* D, int64_t ldd,
                              int64_t batch_d, int M, int N, int K, int L, float alpha, float beta,
                              void* stream) {
  if (!A || !B || !D || M <= 0 || N <= 0 || K <= 0 || L <= 0) {
    xf::set_error("ref_gemm: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  if (dtype_a != dtype_b) { xf::set_error("ref_gemm: A and B dtypes differ"); return XF_ERR_INVALID_DATA_TYPE; }
  // C aliases D in the harness calls (beta = 0); only same-typed C/D pairs are instantiated
  if (beta == 0.f) C = nullptr;
  else if (dtype_c != dtype_d) { xf::set_error("ref_gemm: C and D dtypes differ"); return XF_ERR_INVALID_DATA_TYPE; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((N + 31) / 32, (M + 31) / 32, L), block(32, 32, 1);
  if (dtype_a == XF_DT_BF16 && dtype_d == XF_DT_BF16) XF_REF_GEMM(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (dtype_a == XF_DT_BF16 && dtype_d == XF_DT_F32) XF_REF_GEMM(__nv_bfloat16, float, float);
  else if (dtype_a == XF_DT_S8 && dtype_d == XF_DT_F32) XF_REF_GEMM(int8_t, float, float);
  else if (dtype_a == XF_DT_S8 && dtype_d == XF_DT_S32) XF_REF_GEMM(int8_t, int32_t, int32_t);
  else if (dtype_a == XF_DT_F32 && dtype_d == XF_DT_F32) XF_REF_GEMM(float, float, float);
  else { xf::set_error("ref_gemm: unsupported dtype combination %d -> %d", dtype_a, dtype_d); return XF_ERR_INVALID_DATA_TYPE; }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { xf::set_error("ref_gemm launch: %s", cudaGetErrorString(e)); return XF_ERR_INTERNAL; }
  return XF_SUCCESS;
}

xf_status xf_harness_compare(int dtype, const void* a, const void* b, long long n, float epsilon,
                             float nonzero_floor, long long* mismatches, void* stream) {
  if (!mismatches || (n > 0 && (!a || !b)) || n < 0) {
    xf::set_error("compare: bad arguments");
    return XF_ERR_INVALID_PROBLEM;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long zero = 0, none = ~0ull;
  cudaError_t e = cudaMemcpyToSymbolAsync(g_mismatches, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess)
    e = cudaMemcpyToSymbolAsync(g_first_mismatch, &none, sizeof(none), 0, cudaMemcpyHostToDevice, st);
  unsigned int zero32 = 0;
  if (e == cudaSuccess)
    e = cudaMemcpyToSymbolAsync(g_list_count, &zero32, sizeof(zero32), 0, cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) { xf::set_error("compare: %s", cudaGetErrorString(e)); return XF_ERR_INTERNAL; }
  if (n > 0) {
    switch (dtype) {
      case XF_DT_BF16: compare_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), n, epsilon, nonzero_floor); break;
      case XF_DT_F32: compare_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<const float*>(a), static_cast<const float*>(b), n, epsilon, nonzero_floor); break;
      case XF_DT_S32: compare_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<const int32_t*>(a), static_cast<const int32_t*>(b), n, epsilon, nonzero_floor); break;
      case XF_DT_S8: compare_kernel<<<grid_for(n), 256, 0, st>>>(static_cast<const int8_t*>(a), static_cast<const int8_t*>(b), n, epsilon, nonzero_floor); break;
      default: xf::set_error("compare: unknown dtype %d", dtype); return XF_ERR_INVALID_DATA_TYPE;
    }
  }
  unsigned long long out = 0;
  e = cudaMemcpyFromSymbolAsync(&out, g_mismatches, sizeof(out), 0, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { xf::set_error("compare: %s", cudaGetErrorString(e)); return XF_ERR_INTERNAL; }
  *mismatches = static_cast<long long>(out);
  if (out != 0 && getenv("XF_HARNESS_VERBOSE")) {
    // diagnostic for harness runs: which elements disagree and what the two values are
    // (XF_HARNESS_VERBOSE=1; up to 64 of them, sorted by index)
    unsigned int cnt = 0;
    static unsigned long long idx[kListMax];
    static float va[kListMax], vb[kListMax];
    cudaMemcpyFromSymbol(&cnt, g_list_count, sizeof(cnt));
    cudaMemcpyFromSymbol(idx, g_list_index, sizeof(idx));
    cudaMemcpyFromSymbol(va, g_list_a, sizeof(va));
    cudaMemcpyFromSymbol(vb, g_list_b, sizeof(vb));
    if (cnt > (unsigned int)kListMax) cnt = kListMax;
    fprintf(stderr, "compare: %llu of %lld elements differ (eps %g, floor %g)\n", out, n, epsilon, nonzero_floor);
    for (unsigned int i = 0; i < cnt; ++i) {   // selection sort: at most 64 entries
      unsigned int m = i;
      for (unsigned int j = i + 1; j < cnt; ++j) if (idx[j] < idx[m]) m = j;
      unsigned long long ti = idx[i]; idx[i] = idx[m]; idx[m] = ti;
      float ta = va[i]; va[i] = va[m]; va[m] = ta;
      float tb = vb[i]; vb[i] = vb[m]; vb[m] = tb;
      fprintf(stderr, "  [%llu] expected %.9g got %.9g\n", idx[i], va[i], vb[i]);
    }
  }
  return XF_SUCCESS;
}

}  // extern "C"
