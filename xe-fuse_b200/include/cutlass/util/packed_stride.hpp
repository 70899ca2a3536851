// make_cute_packed_stride: strides of a densely packed (rows, cols, batch) tensor for the two
// stride patterns the GEMM API uses.  The batch stride is 0 when there is a single batch.
#pragma once
#include "xefuse/frontend.hpp"

namespace cutlass {

// major mode second:  (M,K,L) row-major, K contiguous  -> {K, 1, M*K}
template <class IntT, class ShapeT>
cute::Stride<IntT, cute::Int<1>, int64_t>
make_cute_packed_stride(cute::Stride<IntT, cute::Int<1>, int64_t> s, ShapeT const& shape_mkl) {
  std::get<0>(s) = static_cast<IntT>(std::get<1>(shape_mkl));
  const int64_t batches = static_cast<int64_t>(std::get<2>(shape_mkl));
  std::get<2>(s) = batches > 1 ? static_cast<int64_t>(std::get<0>(shape_mkl)) * std::get<1>(shape_mkl) : 0;
  return s;
}

// major mode first:  (N,K,L) with N contiguous (row-major [K,N] storage) -> {1, N, N*K}
template <class IntT, class ShapeT>
cute::Stride<cute::Int<1>, IntT, int64_t>
make_cute_packed_stride(cute::Stride<cute::Int<1>, IntT, int64_t> s, ShapeT const& shape_nkl) {
  std::get<1>(s) = static_cast<IntT>(std::get<0>(shape_nkl));
  const int64_t batches = static_cast<int64_t>(std::get<2>(shape_nkl));
  std::get<2>(s) = batches > 1 ? static_cast<int64_t>(std::get<0>(shape_nkl)) * std::get<1>(shape_nkl) : 0;
  return s;
}

}  // namespace cutlass
