// Host program (built by tests/test_descriptors.py with nvcc, runs without a GPU): prints the
// tcgen05 instruction descriptors the kernels use, so that an accidental edit of the bit
// layout in csrc/tc_common.cuh shows up in the CPU test tier.
#include <cstdio>

#include "tc_common.cuh"

int main() {
  std::printf("%u\n", tc::make_idesc_bf16(128, 256, false, false));  // GEMM, both K-major
  std::printf("%u\n", tc::make_idesc_bf16(128, 256, true, true));    // wgrad, both MN-major
  std::printf("%u\n", tc::make_idesc_bf16(128, 64, false, false));   // attention S = Q K^T
  std::printf("%u\n", tc::make_idesc_bf16(128, 128, false, true));   // attention O += P V
  return 0;
}
