/* Calling the codec from plain C: quantize a buffer to 4 bits with fp16 block scales, restore
 * it, print the packed size and the largest error.  The CUDA libraries expose the same kind
 * of C symbols (raw pointers plus a stream), see bitscom_b200/csrc/symm.h.
 *
 *   cc examples/cpu_codec_example.c -L<dir with libbcom_cpu.so> -lbcom_cpu -lm -o example
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

long long bcom_cpu_packed_nbytes(long long n, int bits);
int bcom_cpu_blockwise_quantize_pack_mt(const float* x, long long n, int bits, int block,
                                        int stochastic, unsigned int key, unsigned int idx_offset,
                                        uint8_t* packed, uint16_t* scales, int threads);
int bcom_cpu_blockwise_unpack_dequantize_mt(const uint8_t* packed, const uint16_t* scales,
                                            int bits, long long n, int block, float* out,
                                            int threads);

int main(void) {
  const long long n = 100000;
  const int bits = 4, block = 256;
  float* x = malloc(sizeof(float) * n);
  float* y = malloc(sizeof(float) * n);
  for (long long i = 0; i < n; ++i) x[i] = sinf(0.001f * (float)i) * 1e-3f;
  const long long nbytes = bcom_cpu_packed_nbytes(n, bits);
  const long long nblocks = (n + block - 1) / block;
  uint8_t* packed = malloc((size_t)nbytes);
  uint16_t* scales = malloc(sizeof(uint16_t) * (size_t)nblocks);
  if (bcom_cpu_blockwise_quantize_pack_mt(x, n, bits, block, 0, 0u, 0u, packed, scales, 2) ||
      bcom_cpu_blockwise_unpack_dequantize_mt(packed, scales, bits, n, block, y, 2)) {
    fprintf(stderr, "codec rejected its arguments\n");
    return 1;
  }
  float worst = 0.0f;
  for (long long i = 0; i < n; ++i) worst = fmaxf(worst, fabsf(x[i] - y[i]));
  printf("%lld floats -> %lld packed bytes + %lld scale bytes, max error %.3g\n", n, nbytes,
         2 * nblocks, worst);
  free(x); free(y); free(packed); free(scales);
  return worst < 1e-3f / 7.0f ? 0 : 2;
}
