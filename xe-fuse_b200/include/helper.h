// Harness helpers: CUTLASS_CHECK (abort on a failed status) and initialize_block (deterministic
// seeded fill of a device buffer: small integers, so fp32 accumulation of products is exact).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <iostream>

#include "cutlass/util/device_memory.h"
#include "xefuse/frontend.hpp"

#define CUTLASS_CHECK(status)                                                                   \
  {                                                                                             \
    cutlass::Status error_ = (status);                                                          \
    if (error_ != cutlass::Status::kSuccess) {                                                  \
      std::cerr << "Got cutlass error: " << cutlass::cutlassGetStatusString(error_) << " at: "  \
                << __LINE__ << " (" << xf_last_error_string() << ")" << std::endl;              \
      std::exit(EXIT_FAILURE);                                                                  \
    }                                                                                           \
  }

// Uniform integers in [-8, 8] for 16/32-bit element types, [-2, 2] for 8-bit ones.
template <class Element>
bool initialize_block(cutlass::DeviceAllocation<Element>& block, uint64_t seed = 2023) {
  const int hi = sizeof(Element) == 1 ? 2 : 8;
  xf_status s = xf_harness_fill_uniform(xefuse::DType<Element>::value, block.get(),
                                        static_cast<long long>(block.size()), seed, -hi, hi, nullptr);
  if (s != XF_SUCCESS) std::fprintf(stderr, "initialize_block: %s\n", xf_last_error_string());
  return s == XF_SUCCESS;
}
