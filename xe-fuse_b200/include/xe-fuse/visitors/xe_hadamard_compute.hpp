// Walsh-Hadamard output node (QuaRot).  The name exists so that code spelling it compiles; the
// B200 library does not implement it: a tree containing it is refused with kErrorNotSupported.
#pragma once

#include "xefuse/frontend.hpp"

namespace xe_fuse {
template <int GroupSize = 16>
struct XeHadamardCompute { struct Arguments {}; };
}  // namespace xe_fuse
