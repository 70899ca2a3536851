// Device buffers for the harness mains: cutlass::DeviceAllocation<T> and
// cutlass::device_memory::allocation<T>.  Buffers are CUDA managed memory, resident on the GPU
// (they are prefetched there on allocation): kernels run at device-memory speed, and host-side
// verification code that dereferences block.get() -- as the reference's harnesses do inside their
// parallel_for lambdas -- still works.
#pragma once
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdio>
#include <cstdlib>

namespace cutlass {
namespace device_memory {

inline void* allocate_bytes(size_t bytes) {
  if (bytes == 0) return nullptr;
  void* p = nullptr;
  cudaError_t e = cudaMallocManaged(&p, bytes, cudaMemAttachGlobal);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "device allocation of %zu bytes failed: %s\n", bytes, cudaGetErrorString(e));
    std::abort();
  }
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaMemPrefetchAsync(p, bytes, dev, 0);
  return p;
}
inline void free_bytes(void* p) { if (p) cudaFree(p); }

template <class T>
class allocation {
 public:
  allocation() = default;
  explicit allocation(size_t n) { reset(n); }
  allocation(allocation const&) = delete;
  allocation& operator=(allocation const&) = delete;
  allocation(allocation&& o) noexcept : ptr_(o.ptr_), n_(o.n_) { o.ptr_ = nullptr; o.n_ = 0; }
  allocation& operator=(allocation&& o) noexcept {
    if (this != &o) { free_bytes(ptr_); ptr_ = o.ptr_; n_ = o.n_; o.ptr_ = nullptr; o.n_ = 0; }
    return *this;
  }
  ~allocation() { free_bytes(ptr_); }
  void reset(size_t n = 0) {
    free_bytes(ptr_);
    n_ = n;
    ptr_ = static_cast<T*>(allocate_bytes(n * sizeof(T)));
  }
  T* get() const { return ptr_; }
  size_t size() const { return n_; }
  size_t bytes() const { return n_ * sizeof(T); }
  void copy_from_host(T const* src, size_t n) { cudaMemcpy(ptr_, src, n * sizeof(T), cudaMemcpyDefault); }
  void copy_from_host(T const* src) { copy_from_host(src, n_); }
  void copy_to_host(T* dst, size_t n) const { cudaMemcpy(dst, ptr_, n * sizeof(T), cudaMemcpyDefault); }
  void copy_to_host(T* dst) const { copy_to_host(dst, n_); }
 private:
  T* ptr_ = nullptr;
  size_t n_ = 0;
};

}  // namespace device_memory

template <class T>
using DeviceAllocation = device_memory::allocation<T>;

}  // namespace cutlass
