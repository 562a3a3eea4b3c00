// CPU codec: blockwise quantize + pack and unpack + dequantize for fp32 buffers, all six
// bitwidths, nearest and seeded stochastic rounding — a bit-exact C++ twin of the host
// quantizer (bitscom_b200/quantization.py, which restates reference
// python/bitscom/quantization.py:102-150,311-390).  It serves CPU ranks (gloo plumbing
// path, fault-injection harness) and is the timed CPU baseline; the reference has no native
// CPU codec, its CPU path is ~15 torch ops per call.
//
// Plain C++17, no CUDA.  The inner loops are written branch-free over short spans so that
// the compiler vectorises them (cloned for AVX2 and the baseline ISA, chosen at load time);
// large tensors are split over `threads` std::threads at boundaries that are whole blocks and
// whole packed bytes.  Rounding never goes through the conversion instructions' modes: the
// 2^23 magic-number add gives round-half-even and a truncating convert gives floor for the
// non-negative ratios, both exactly.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

// (BCOM_NO_CLONES: the load-time resolver of cloned functions runs before ThreadSanitizer's
// runtime is up, so sanitizer builds switch the clones off)
#if defined(__GNUC__) && defined(__x86_64__) && !defined(BCOM_NO_CLONES)
#define BCOM_CLONES __attribute__((target_clones("avx2", "default")))
#else
#define BCOM_CLONES
#endif

namespace {

inline void bounds(int bits, int* qmin, int* qmax) {
  if (bits == 1) { *qmin = 0; *qmax = 1; return; }
  *qmax = (1 << (bits - 1)) - 1;
  *qmin = -(1 << (bits - 1));
}

// IEEE binary16 round-to-nearest-even conversion and back
inline uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7FFFFFFFu;
  if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((x > 0x7F800000u) ? 0x200u : 0));
  if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to infinity
  if (x < 0x33000001u) return (uint16_t)sign;               // rounds to zero
  int exp = (int)(x >> 23) - 127;
  uint32_t man = (x & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t half_exp;
  if (exp < -14) {            // subnormal half
    shift = 13 + (-14 - exp);
    half_exp = 0;
  } else {
    shift = 13;
    half_exp = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t half_man = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half_man & 1u))) ++half_man;
  return (uint16_t)(sign | (half_exp + half_man));  // a carry moves into the exponent
}

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7F800000u | (man << 13);
  } else {
    x = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

inline uint32_t sr_bits(uint32_t key, uint32_t idx) {
  uint32_t h = (idx >> 1) * 0x9E3779B1u + key;
  h ^= h >> 16;
  h *= 0x21F0AAADu;
  h ^= h >> 15;
  h *= 0x735A2D97u;
  h ^= h >> 15;
  return (idx & 1u) ? (h >> 16) : (h & 0xFFFFu);
}

inline long long packed_nbytes(long long n, int bits) {
  if (bits == 12) return 3 * ((n + 1) / 2);
  if (bits == 16) return 2 * n;
  return (n * bits + 7) / 8;
}

inline void put_code(uint8_t* packed, long long i, uint32_t code, int bits) {
  if (bits <= 8) {
    const int per = 8 / bits;
    packed[i / per] |= (uint8_t)(code << ((i % per) * bits));
  } else if (bits == 12) {
    uint8_t* t = packed + (i / 2) * 3;
    if ((i & 1) == 0) {
      t[0] = (uint8_t)(code & 0xFF);
      t[1] |= (uint8_t)((code >> 8) & 0x0F);
    } else {
      t[1] |= (uint8_t)((code & 0x0F) << 4);
      t[2] = (uint8_t)((code >> 4) & 0xFF);
    }
  } else {
    packed[2 * i] = (uint8_t)(code & 0xFF);
    packed[2 * i + 1] = (uint8_t)((code >> 8) & 0xFF);
  }
}

inline uint32_t get_code(const uint8_t* packed, long long i, int bits) {
  if (bits <= 8) {
    const int per = 8 / bits;
    return (packed[i / per] >> ((i % per) * bits)) & ((1u << bits) - 1u);
  }
  if (bits == 12) {
    const uint8_t* t = packed + (i / 2) * 3;
    return (i & 1) == 0 ? ((uint32_t)t[0] | (((uint32_t)t[1] & 0x0F) << 8))
                        : ((((uint32_t)t[1] >> 4) & 0x0F) | ((uint32_t)t[2] << 4));
  }
  return (uint32_t)packed[2 * i] | ((uint32_t)packed[2 * i + 1] << 8);
}

constexpr int kSpan = 256;  // elements handled per inner call (a block is cut into spans)

// Largest magnitude of a span; NaN if the span holds one (the host quantizer's amax
// propagates NaN, which then selects the scale 1.0 for the block).
BCOM_CLONES float span_absmax(const float* x, int len) {
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int nan[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= len; i += 8)
    for (int l = 0; l < 8; ++l) {
      const float a = std::fabs(x[i + l]);
      lane[l] = a > lane[l] ? a : lane[l];
      nan[l] |= a != a;
    }
  float m = 0.0f;
  int any_nan = 0;
  for (int l = 0; l < 8; ++l) {
    m = lane[l] > m ? lane[l] : m;
    any_nan |= nan[l];
  }
  for (; i < len; ++i) {
    const float a = std::fabs(x[i]);
    m = a > m ? a : m;
    any_nan |= a != a;
  }
  return any_nan ? std::nanf("") : m;
}

// codes[i] = (q - qmin) & mask for len <= kSpan values that share the scale sf
template <bool SR>
BCOM_CLONES void span_quantize(const float* x, int len, float sf, int bits, int qmin, int qmax,
                               uint32_t key, uint32_t idx0, uint16_t* codes) {
  const float fmin = (float)qmin, fmax = (float)qmax;
  const uint32_t mask = (1u << bits) - 1u;
  const bool one_bit = bits == 1;
  for (int i = 0; i < len; ++i) {
    const float v = x[i];
    const float nrm = std::fabs(v) / sf;
    float mag;
    if (SR) {
      // floor of a non-negative ratio; ratios >= 2^23 (and inf / NaN) are already integral
      const float lo = nrm < 8388608.0f ? (float)(int)nrm : nrm;
      float p = nrm - lo;
      p = p < 0.0f ? 0.0f : (p > 1.0f ? 1.0f : p);
      const float u = (float)sr_bits(key, idx0 + (uint32_t)i) * (1.0f / 65536.0f);
      mag = u < p ? lo + 1.0f : lo;
    } else {
      // round half to even: exact for ratios below 2^22, larger ones are integral already
      const float r = (nrm + 12582912.0f) - 12582912.0f;
      mag = nrm < 4194304.0f ? r : nrm;
    }
    const float sgn = (float)((v > 0.0f) - (v < 0.0f));
    float s = one_bit ? mag : mag * sgn;
    s = s < fmin ? fmin : (s > fmax ? fmax : s);  // NaN falls through both tests
    const int q = s != s ? 0 : (int)s;
    codes[i] = (uint16_t)((uint32_t)(q - qmin) & mask);
  }
}

// whole-byte packers: i0 and len are multiples of 8 for bits <= 8, of 2 for 12 bits
BCOM_CLONES void span_pack(const uint16_t* c, long long i0, int len, int bits, uint8_t* packed) {
  if (bits == 8) {
    uint8_t* o = packed + i0;
    for (int i = 0; i < len; ++i) o[i] = (uint8_t)c[i];
  } else if (bits == 4) {
    uint8_t* o = packed + i0 / 2;
    for (int i = 0; i < len / 2; ++i) o[i] = (uint8_t)(c[2 * i] | (c[2 * i + 1] << 4));
  } else if (bits == 2) {
    uint8_t* o = packed + i0 / 4;
    for (int i = 0; i < len / 4; ++i)
      o[i] = (uint8_t)(c[4 * i] | (c[4 * i + 1] << 2) | (c[4 * i + 2] << 4) | (c[4 * i + 3] << 6));
  } else if (bits == 1) {
    uint8_t* o = packed + i0 / 8;
    for (int i = 0; i < len / 8; ++i) {
      uint32_t b = 0;
      for (int k = 0; k < 8; ++k) b |= (uint32_t)c[8 * i + k] << k;
      o[i] = (uint8_t)b;
    }
  } else if (bits == 12) {
    uint8_t* o = packed + (i0 / 2) * 3;
    for (int i = 0; i < len / 2; ++i) {
      const uint32_t a = c[2 * i], b = c[2 * i + 1];
      o[3 * i] = (uint8_t)(a & 0xFF);
      o[3 * i + 1] = (uint8_t)(((a >> 8) & 0x0F) | ((b & 0x0F) << 4));
      o[3 * i + 2] = (uint8_t)(b >> 4);
    }
  } else {
    uint8_t* o = packed + 2 * i0;
    for (int i = 0; i < len; ++i) {
      o[2 * i] = (uint8_t)(c[i] & 0xFF);
      o[2 * i + 1] = (uint8_t)(c[i] >> 8);
    }
  }
}

BCOM_CLONES void span_unpack(const uint8_t* packed, long long i0, int len, int bits,
                             uint16_t* c) {
  if (bits == 8) {
    const uint8_t* p = packed + i0;
    for (int i = 0; i < len; ++i) c[i] = p[i];
  } else if (bits == 4) {
    const uint8_t* p = packed + i0 / 2;
    for (int i = 0; i < len / 2; ++i) {
      c[2 * i] = p[i] & 0x0F;
      c[2 * i + 1] = p[i] >> 4;
    }
  } else if (bits == 2) {
    const uint8_t* p = packed + i0 / 4;
    for (int i = 0; i < len / 4; ++i)
      for (int k = 0; k < 4; ++k) c[4 * i + k] = (p[i] >> (2 * k)) & 3;
  } else if (bits == 1) {
    const uint8_t* p = packed + i0 / 8;
    for (int i = 0; i < len / 8; ++i)
      for (int k = 0; k < 8; ++k) c[8 * i + k] = (p[i] >> k) & 1;
  } else if (bits == 12) {
    const uint8_t* p = packed + (i0 / 2) * 3;
    for (int i = 0; i < len / 2; ++i) {
      c[2 * i] = (uint16_t)(p[3 * i] | ((p[3 * i + 1] & 0x0F) << 8));
      c[2 * i + 1] = (uint16_t)((p[3 * i + 1] >> 4) | (p[3 * i + 2] << 4));
    }
  } else {
    const uint8_t* p = packed + 2 * i0;
    for (int i = 0; i < len; ++i) c[i] = (uint16_t)(p[2 * i] | (p[2 * i + 1] << 8));
  }
}

BCOM_CLONES void span_scale(const uint16_t* c, int len, int qmin, float sf, float* out) {
  for (int i = 0; i < len; ++i) out[i] = (float)((int)c[i] + qmin) * sf;
}

inline bool whole_bytes(long long i0, int len, int bits) {
  const int unit = bits <= 8 ? 8 : (bits == 12 ? 2 : 1);
  return i0 % unit == 0 && len % unit == 0;
}

// blocks [blk0, blk1) of the tensor; the caller zeroed `packed`
void quantize_range(const float* x, long long n, int bits, int block, bool stochastic,
                    uint32_t key, uint32_t idx_offset, long long blk0, long long blk1,
                    uint8_t* packed, uint16_t* scales) {
  int qmin, qmax;
  bounds(bits, &qmin, &qmax);
  uint16_t codes[kSpan];
  for (long long blk = blk0; blk < blk1; ++blk) {
    const long long b0 = blk * block;
    const long long b1 = b0 + block < n ? b0 + block : n;
    float m = 0.0f;
    for (long long i = b0; i < b1; i += kSpan) {
      const float a = span_absmax(x + i, (int)(b1 - i < kSpan ? b1 - i : kSpan));
      m = (a > m || a != a) ? a : m;
      if (m != m) break;
    }
    float scale = m / (float)qmax;
    if (!(m > 0.0f)) scale = 1.0f;
    const uint16_t sh = float_to_half(scale);
    scales[blk] = sh;
    const float sf = half_to_float(sh);
    for (long long i = b0; i < b1; i += kSpan) {
      const int len = (int)(b1 - i < kSpan ? b1 - i : kSpan);
      if (stochastic)
        span_quantize<true>(x + i, len, sf, bits, qmin, qmax, key, idx_offset + (uint32_t)i,
                            codes);
      else
        span_quantize<false>(x + i, len, sf, bits, qmin, qmax, 0u, 0u, codes);
      if (whole_bytes(i, len, bits)) {
        span_pack(codes, i, len, bits, packed);
      } else {
        for (int k = 0; k < len; ++k) put_code(packed, i + k, codes[k], bits);
      }
    }
  }
}

void dequantize_range(const uint8_t* packed, const uint16_t* scales, int bits, long long n,
                      int block, long long blk0, long long blk1, float* out) {
  int qmin, qmax;
  bounds(bits, &qmin, &qmax);
  uint16_t codes[kSpan];
  for (long long blk = blk0; blk < blk1; ++blk) {
    const long long b0 = blk * block;
    const long long b1 = b0 + block < n ? b0 + block : n;
    const float sf = half_to_float(scales[blk]);
    for (long long i = b0; i < b1; i += kSpan) {
      const int len = (int)(b1 - i < kSpan ? b1 - i : kSpan);
      if (whole_bytes(i, len, bits)) {
        span_unpack(packed, i, len, bits, codes);
      } else {
        for (int k = 0; k < len; ++k) codes[k] = (uint16_t)get_code(packed, i + k, bits);
      }
      span_scale(codes, len, qmin, sf, out + i);
    }
  }
}

// Splits [0, nblocks) over up to `threads` workers at multiples of `align` blocks (so that no
// two workers share a packed byte) and runs fn(blk0, blk1) on each part.
template <typename F>
void fan_out(long long nblocks, long long align, int threads, long long min_blocks, F fn) {
  long long parts = threads > 1 ? threads : 1;
  if (nblocks < 2 * min_blocks) parts = 1;
  if (parts > nblocks / min_blocks && parts > 1) parts = nblocks / min_blocks;
  if (parts <= 1) {
    fn(0, nblocks);
    return;
  }
  long long per = (nblocks + parts - 1) / parts;
  per = (per + align - 1) / align * align;
  std::vector<std::thread> pool;
  for (long long b = per; b < nblocks; b += per)
    pool.emplace_back(fn, b, b + per < nblocks ? b + per : nblocks);
  fn(0, per < nblocks ? per : nblocks);
  for (auto& t : pool) t.join();
}

inline bool bits_ok(int bits) {
  return bits == 1 || bits == 2 || bits == 4 || bits == 8 || bits == 12 || bits == 16;
}

}  // namespace

extern "C" {

long long bcom_cpu_packed_nbytes(long long n, int bits) { return packed_nbytes(n, bits); }

// x: fp32[n]; packed: uint8[packed_nbytes(n)]; scales: fp16 bits, uint16[ceil(n/block)].
// threads <= 1 runs on the calling thread.  Returns 0, or 1 on bad arguments.
int bcom_cpu_blockwise_quantize_pack_mt(const float* x, long long n, int bits, int block,
                                        int stochastic, unsigned int key,
                                        unsigned int idx_offset, uint8_t* packed,
                                        uint16_t* scales, int threads) {
  if (n < 0 || block <= 0 || !bits_ok(bits)) return 1;
  const long long nblocks = (n + block - 1) / block;
  // 8 blocks always end on a whole packed byte (and on a 12-bit pair)
  const long long min_blocks = (65536 + block - 1) / block;
  fan_out(nblocks, 8, threads, min_blocks, [=](long long b0, long long b1) {
    const long long e0 = b0 * block, e1 = b1 * block < n ? b1 * block : n;
    const long long p0 = packed_nbytes(e0, bits), p1 = packed_nbytes(e1, bits);
    if (p1 > p0) std::memset(packed + p0, 0, (size_t)(p1 - p0));  // n == 0: packed may be null
    quantize_range(x, n, bits, block, stochastic != 0, key, idx_offset, b0, b1, packed, scales);
  });
  return 0;
}

int bcom_cpu_blockwise_quantize_pack(const float* x, long long n, int bits, int block,
                                     int stochastic, unsigned int key, unsigned int idx_offset,
                                     uint8_t* packed, uint16_t* scales) {
  return bcom_cpu_blockwise_quantize_pack_mt(x, n, bits, block, stochastic, key, idx_offset,
                                             packed, scales, 1);
}

int bcom_cpu_blockwise_unpack_dequantize_mt(const uint8_t* packed, const uint16_t* scales,
                                            int bits, long long n, int block, float* out,
                                            int threads) {
  if (n < 0 || block <= 0 || !bits_ok(bits)) return 1;
  const long long nblocks = (n + block - 1) / block;
  const long long min_blocks = (65536 + block - 1) / block;
  fan_out(nblocks, 1, threads, min_blocks, [=](long long b0, long long b1) {
    dequantize_range(packed, scales, bits, n, block, b0, b1, out);
  });
  return 0;
}

int bcom_cpu_blockwise_unpack_dequantize(const uint8_t* packed, const uint16_t* scales, int bits,
                                         long long n, int block, float* out) {
  return bcom_cpu_blockwise_unpack_dequantize_mt(packed, scales, bits, n, block, out, 1);
}

}  // extern "C"
