// CPU codec: blockwise quantize + pack and unpack + dequantize for fp32 buffers, all six
// bitwidths, nearest and seeded stochastic rounding — a bit-exact C++ twin of the host
// quantizer (bitscom_b200/quantization.py, which restates reference
// python/bitscom/quantization.py:102-150,311-390).  It serves CPU ranks (gloo plumbing
// path, fault-injection harness) and is the timed CPU baseline; the reference has no native
// CPU codec, its CPU path is ~15 torch ops per call.
//
// Plain C++17, no CUDA; OpenMP-free on purpose (ranks already run one per process).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

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

inline float sr_uniform(uint32_t key, uint32_t idx) {
  uint32_t h = (idx >> 1) * 0x9E3779B1u + key;
  h ^= h >> 16;
  h *= 0x21F0AAADu;
  h ^= h >> 15;
  h *= 0x735A2D97u;
  h ^= h >> 15;
  const uint32_t bits = (idx & 1u) ? (h >> 16) : (h & 0xFFFFu);
  return (float)bits * (1.0f / 65536.0f);
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

}  // namespace

extern "C" {

long long bcom_cpu_packed_nbytes(long long n, int bits) { return packed_nbytes(n, bits); }

// x: fp32[n]; packed: uint8[packed_nbytes(n)]; scales: fp16 bits, uint16[ceil(n/block)].
// Returns 0, or 1 on bad arguments.
int bcom_cpu_blockwise_quantize_pack(const float* x, long long n, int bits, int block,
                                     int stochastic, unsigned int key, unsigned int idx_offset,
                                     uint8_t* packed, uint16_t* scales) {
  if (n < 0 || block <= 0) return 1;
  if (bits != 1 && bits != 2 && bits != 4 && bits != 8 && bits != 12 && bits != 16) return 1;
  int qmin, qmax;
  bounds(bits, &qmin, &qmax);
  std::memset(packed, 0, (size_t)packed_nbytes(n, bits));
  const uint32_t mask = (1u << bits) - 1u;
  for (long long b0 = 0, blk = 0; b0 < n; b0 += block, ++blk) {
    const long long b1 = b0 + block < n ? b0 + block : n;
    float m = 0.0f;
    for (long long i = b0; i < b1; ++i) {
      const float a = std::fabs(x[i]);
      if (a > m) m = a;
    }
    float scale = m / (float)qmax;
    if (!(m > 0.0f)) scale = 1.0f;
    const uint16_t sh = float_to_half(scale);
    scales[blk] = sh;
    const float sf = half_to_float(sh);
    for (long long i = b0; i < b1; ++i) {
      const float nrm = std::fabs(x[i]) / sf;
      float mag;
      if (stochastic) {
        const float lo = std::floor(nrm);
        float p = nrm - lo;
        p = p < 0.0f ? 0.0f : (p > 1.0f ? 1.0f : p);
        mag = sr_uniform(key, idx_offset + (uint32_t)i) < p ? lo + 1.0f : lo;
      } else {
        mag = std::nearbyintf(nrm);  // default rounding mode: half to even
      }
      float s = mag;
      if (bits != 1) s = mag * (float)((x[i] > 0.0f) - (x[i] < 0.0f));
      int q;
      if (s != s) {
        q = 0;
      } else {
        const float c = s < (float)qmin ? (float)qmin : (s > (float)qmax ? (float)qmax : s);
        q = (int)c;
      }
      put_code(packed, i, (uint32_t)(q - qmin) & mask, bits);
    }
  }
  return 0;
}

int bcom_cpu_blockwise_unpack_dequantize(const uint8_t* packed, const uint16_t* scales, int bits,
                                         long long n, int block, float* out) {
  if (n < 0 || block <= 0) return 1;
  if (bits != 1 && bits != 2 && bits != 4 && bits != 8 && bits != 12 && bits != 16) return 1;
  int qmin, qmax;
  bounds(bits, &qmin, &qmax);
  for (long long i = 0; i < n; ++i) {
    const int q = (int)get_code(packed, i, bits) + qmin;
    out[i] = (float)q * half_to_float(scales[i / block]);
  }
  return 0;
}

}  // extern "C"
