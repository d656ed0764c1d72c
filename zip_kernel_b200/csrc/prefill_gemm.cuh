// Kernel 2 (tensor-core path) - placeholder until the tcgen05 kernel lands.
#pragma once
#include "common.cuh"
namespace w4a4 {
namespace pre {
inline bool supported(int, int, int) { return false; }
}  // namespace pre
}  // namespace w4a4
