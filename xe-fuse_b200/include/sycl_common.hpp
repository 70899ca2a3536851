// Queue vocabulary of the harness mains on a CUDA back end.
//
// The reference's harnesses drive the device through a default in-order queue
// (compat::get_default_queue(), compat::wait()) and rebuild expected values with
// queue.parallel_for(range, lambda) over device pointers.  Here the queue is the default CUDA
// stream; parallel_for synchronises the device and runs the lambda on the host cores, which works
// because harness buffers are managed memory (cutlass/util/device_memory.h).  Only what the
// harnesses use exists.
#pragma once
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>

namespace sycl {

template <int Dims = 1>
struct range {
  size_t extent[Dims > 0 ? Dims : 1];
  range(size_t n0) { extent[0] = n0; }
  size_t operator[](int i) const { return extent[i]; }
  size_t size() const { size_t s = 1; for (int i = 0; i < Dims; ++i) s *= extent[i]; return s; }
};

template <int Dims = 1>
struct id {
  size_t index[Dims > 0 ? Dims : 1];
  size_t operator[](int i) const { return index[i]; }
  operator size_t() const { return index[0]; }
};

inline float exp(float x) { return std::exp(x); }
inline float log(float x) { return std::log(x); }
inline float erf(float x) { return std::erf(x); }
inline float tanh(float x) { return std::tanh(x); }
inline float sqrt(float x) { return std::sqrt(x); }
inline float rsqrt(float x) { return 1.0f / std::sqrt(x); }
inline float fabs(float x) { return std::fabs(x); }
inline float fmax(float a, float b) { return std::fmax(a, b); }
inline float fmin(float a, float b) { return std::fmin(a, b); }
inline float round(float x) { return std::round(x); }
inline float pow(float a, float b) { return std::pow(a, b); }

class queue {
 public:
  void wait() { cudaDeviceSynchronize(); }
  void wait_and_throw() { wait(); }
  queue& memcpy(void* dst, const void* src, size_t bytes) {
    cudaMemcpy(dst, src, bytes, cudaMemcpyDefault);
    return *this;
  }
  queue& memset(void* dst, int value, size_t bytes) {
    cudaMemset(dst, value, bytes);
    return *this;
  }
  // Host execution over managed memory; the device is idle while it runs.
  template <class F>
  queue& parallel_for(range<1> r, F f) {
    cudaDeviceSynchronize();
    const long long n = static_cast<long long>(r[0]);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
      id<1> ix;
      ix.index[0] = static_cast<size_t>(i);
      f(ix);
    }
    return *this;
  }
};

}  // namespace sycl

namespace compat {
inline sycl::queue& get_default_queue() {
  static sycl::queue q;
  return q;
}
inline void wait() { cudaDeviceSynchronize(); }
inline void wait_and_throw() { cudaDeviceSynchronize(); }
}  // namespace compat
namespace syclcompat = compat;
