// Sanitizer driver for the C++ CPU codec: built by tests/test_sanitizers_cpu.py with
// -fsanitize=address,undefined (and, separately, -fsanitize=thread) and run to completion.
// It walks odd sizes around block and byte boundaries, every bitwidth, both rounding modes,
// one to four threads, with output buffers allocated at their exact sizes so that any write
// past the end is caught, and checks that the packed bytes and scales do not depend on the
// thread count and that unpack(dequantize) of pack(quantize) stays within one step.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

extern "C" {
long long bcom_cpu_packed_nbytes(long long n, int bits);
int bcom_cpu_blockwise_quantize_pack_mt(const float* x, long long n, int bits, int block,
                                        int stochastic, unsigned int key, unsigned int idx_offset,
                                        uint8_t* packed, uint16_t* scales, int threads);
int bcom_cpu_blockwise_unpack_dequantize_mt(const uint8_t* packed, const uint16_t* scales,
                                            int bits, long long n, int block, float* out,
                                            int threads);
}

static uint32_t lcg(uint32_t& s) { return s = s * 1664525u + 1013904223u; }

static int run_case(long long n, int bits, int block, int stochastic) {
  std::vector<float> x((size_t)n);
  uint32_t seed = (uint32_t)(n * 31 + bits * 7 + block);
  for (auto& v : x) v = ((int)(lcg(seed) >> 8) % 2001 - 1000) * 1e-3f;
  if (n > 5) x[3] = 0.0f;
  const long long nb = bcom_cpu_packed_nbytes(n, bits);
  const long long ns = (n + block - 1) / block;
  std::vector<uint8_t> ref;
  std::vector<uint16_t> ref_s;
  for (int threads = 1; threads <= 4; ++threads) {
    std::vector<uint8_t> packed((size_t)nb);      // exact size: overruns trip the sanitizer
    std::vector<uint16_t> scales((size_t)ns);
    if (bcom_cpu_blockwise_quantize_pack_mt(x.data(), n, bits, block, stochastic, 0x1234u, 17u,
                                            packed.data(), scales.data(), threads))
      return 1;
    if (threads == 1) {
      ref = packed;
      ref_s = scales;
    } else if (packed != ref || scales != ref_s) {
      std::fprintf(stderr, "thread count changes the result: n=%lld bits=%d block=%d\n", n, bits,
                   block);
      return 2;
    }
    std::vector<float> out((size_t)n);
    if (bcom_cpu_blockwise_unpack_dequantize_mt(packed.data(), scales.data(), bits, n, block,
                                                out.data(), threads))
      return 3;
    if (bits >= 2) {
      const float qmax = (float)((1 << (bits - 1)) - 1);
      for (long long b0 = 0; b0 < n; b0 += block) {
        float m = 0.0f;
        for (long long i = b0; i < n && i < b0 + block; ++i) m = std::fmax(m, std::fabs(x[i]));
        const float step = m / qmax * 1.01f + 1e-7f;
        for (long long i = b0; i < n && i < b0 + block; ++i)
          // one rounding step, plus the fp16 rounding of the scale (relative 2^-11 for
          // normal scales, absolute 2^-25 for subnormal ones) carried by a code of up to qmax
          if (std::fabs(out[i] - x[i]) >
              step * (stochastic ? 1.0f : 0.51f) + 1e-3f * m + qmax * 3.0e-8f) {
            std::fprintf(stderr, "error too large: n=%lld bits=%d block=%d i=%lld %g vs %g\n", n,
                         bits, block, i, out[i], x[i]);
            return 4;
          }
      }
    }
  }
  return 0;
}

int main() {
  const int bit_list[] = {1, 2, 4, 8, 12, 16};
  const int blocks[] = {1, 7, 8, 24, 256, 1000};
  const long long sizes[] = {0, 1, 2, 7, 8, 9, 255, 256, 257, 1001, 4099, 70001, 300007};
  long long cases = 0;
  for (int bits : bit_list)
    for (int block : blocks)
      for (long long n : sizes)
        for (int sr = 0; sr < 2; ++sr) {
          if (n > 100000 && block < 8) continue;  // keep the run short
          const int rc = run_case(n, bits, block, sr);
          if (rc) return rc;
          ++cases;
        }
  std::printf("ok %lld cases\n", cases);
  return 0;
}
