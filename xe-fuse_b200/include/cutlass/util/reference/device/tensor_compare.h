// cutlass::reference::device::BlockCompareRelativelyEqual / BlockCompareEqual over device buffers.
// Two values a, b are relatively equal when a == b; or, if either is zero or |a| + |b| is below
// nonzero_floor, when |a-b| < epsilon * nonzero_floor; otherwise when |a-b| < epsilon * (|a| + |b|).
// (The comparator the reference's harnesses call lives in intel/sycl-tla, which is not part of the
// reference tree; this is the usual relative test with an absolute floor near zero.)
#pragma once
#include "xefuse/frontend.hpp"

namespace cutlass::reference::device {

template <class Element>
bool BlockCompareRelativelyEqual(Element const* a, Element const* b, size_t count, Element epsilon,
                                 Element nonzero_floor, int /*grid*/ = 0, int /*block*/ = 0) {
  long long mismatches = -1;
  xf_status s = xf_harness_compare(xefuse::DType<Element>::value, a, b, static_cast<long long>(count),
                                   float(epsilon), float(nonzero_floor), &mismatches, nullptr);
  if (s != XF_SUCCESS) {
    std::fprintf(stderr, "BlockCompareRelativelyEqual: %s\n", xf_last_error_string());
    return false;
  }
  return mismatches == 0;
}

template <class Element>
bool BlockCompareEqual(Element const* a, Element const* b, size_t count, int = 0, int = 0) {
  long long mismatches = -1;
  xf_status s = xf_harness_compare(xefuse::DType<Element>::value, a, b, static_cast<long long>(count),
                                   0.f, 0.f, &mismatches, nullptr);
  return s == XF_SUCCESS && mismatches == 0;
}

}  // namespace cutlass::reference::device
