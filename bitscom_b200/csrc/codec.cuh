// Device codec shared by every low-bit kernel in this library (sm_100a).
//
// One thread owns GROUP = 8 consecutive elements.  A quantization block of
// B = 8 * T elements (T a power of two <= 32) therefore lives in T adjacent
// lanes of one warp, and its absmax is a width-T xor-shuffle reduction: no
// shared memory, no block-wide barrier.  Packing happens in registers; eight
// b-bit codes form one b-byte group that is stored with a single instruction
// (b = 4: one 32-bit word per thread, 128 contiguous bytes per warp).
//
// Numerics follow the host quantizer bit for bit (bitscom_b200/quantization.py,
// which restates reference python/bitscom/quantization.py:102-150 and
// cpp/src/lowbit_cuda_kernels.cu:144-250): IEEE division, fp16 round trip of
// the scale, half-to-even rounding, explicit __fmul_rn/__fadd_rn so that the
// compiler cannot contract a multiply and an add into one fma.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace bcom {

constexpr int GROUP = 8;  // elements per thread

template <int BITS> struct Range {
  static constexpr int qmin = BITS == 1 ? 0 : -(1 << (BITS - 1));
  static constexpr int qmax = BITS == 1 ? 1 : (1 << (BITS - 1)) - 1;
};

// bytes occupied by one 8-element group on the wire
template <int BITS> struct GroupBytes { static constexpr int value = BITS; };

// ---------------------------------------------------------------------------
// counter-based uniform stream: same arithmetic as quantization.sr_uniform
// ---------------------------------------------------------------------------
// One 32-bit hash serves TWO consecutive elements (16 random bits each): element idx
// uses the low half of hash(idx >> 1) when idx is even, the high half when odd.
__device__ __forceinline__ uint32_t sr_hash(uint32_t key, uint32_t pair) {
  uint32_t h = pair * 0x9E3779B1u + key;
  h ^= h >> 16;
  h *= 0x21F0AAADu;
  h ^= h >> 15;
  h *= 0x735A2D97u;
  h ^= h >> 15;
  return h;
}
// 16 random bits as the top mantissa bits of a float in [1, 2): u = bits * 2^-16 exactly,
// without an int-to-float conversion
__device__ __forceinline__ float sr_u16(uint32_t bits16) {
  return __uint_as_float(0x3F800000u | (bits16 << 7)) - 1.0f;
}
__device__ __forceinline__ float sr_uniform(uint32_t key, uint32_t idx) {
  const uint32_t h = sr_hash(key, idx >> 1);
  return sr_u16((idx & 1u) ? (h >> 16) : (h & 0xFFFFu));
}

// ---------------------------------------------------------------------------
// typed 8-element loads / stores (vector form: 32-byte aligned fp32, 16-byte aligned 2-byte types)
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// fp32 groups move as ONE 256-bit access (ld/st.global.v8.f32, sm_100): every store
// instruction then writes whole 32-byte sectors, which two 128-bit stores per thread do not
// (each would write half of every sector it touches).  The address must be 32-byte aligned
// for fp32 and 16-byte aligned for the 2-byte types; the launchers check that.
__device__ __forceinline__ void ld256_nc(const float* p, float (&v)[GROUP]) {
  asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]),
                 "=f"(v[6]), "=f"(v[7])
               : "l"(p));
}
__device__ __forceinline__ void ld256(const float* p, float (&v)[GROUP]) {
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]),
                 "=f"(v[6]), "=f"(v[7])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ void st256(float* p, const float (&v)[GROUP]) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0]),
               "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

template <typename T>
__device__ __forceinline__ void load8_vec(const T* __restrict__ p, float (&v)[GROUP]) {
  if constexpr (sizeof(T) == 4) {
    ld256_nc(reinterpret_cast<const float*>(p), v);
  } else {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < GROUP; ++i) v[i] = Elem<T>::to_f(h[i]);
  }
}

// plain (coherent) variant for buffers that are written earlier in the same kernel
template <typename T>
__device__ __forceinline__ void load8_vec_coherent(const T* p, float (&v)[GROUP]) {
  if constexpr (sizeof(T) == 4) {
    ld256(reinterpret_cast<const float*>(p), v);
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < GROUP; ++i) v[i] = Elem<T>::to_f(h[i]);
  }
}

template <typename T>
__device__ __forceinline__ void load8_guard(const T* p, long long base, long long n,
                                            float (&v)[GROUP]) {
#pragma unroll
  for (int i = 0; i < GROUP; ++i)
    v[i] = (base + i < n) ? Elem<T>::to_f(p[base + i]) : 0.0f;
}

template <typename T>
__device__ __forceinline__ void store8_vec(T* p, const float (&v)[GROUP]) {
  if constexpr (sizeof(T) == 4) {
    st256(reinterpret_cast<float*>(p), v);
  } else {
    uint4 raw;
    T* h = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < GROUP; ++i) h[i] = Elem<T>::from_f(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
}

template <typename T>
__device__ __forceinline__ void store8_guard(T* p, long long base, long long n,
                                             const float (&v)[GROUP]) {
#pragma unroll
  for (int i = 0; i < GROUP; ++i)
    if (base + i < n) p[base + i] = Elem<T>::from_f(v[i]);
}

// ---------------------------------------------------------------------------
// block scale: width-T shuffle absmax, IEEE divide, fp16 round trip
// ---------------------------------------------------------------------------
// max that returns NaN when either operand is NaN (fmaxf would drop it).  The host
// quantizer's amax propagates NaN, and a NaN absmax then selects the scale 1.0 for its block
// (reference python/bitscom/quantization.py:126-131), so the block maximum must keep it.
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

__device__ __forceinline__ float absmax8(const float (&v)[GROUP]) {
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < GROUP; ++i) m = max_nan(m, fabsf(v[i]));
  return m;
}

// All 32 lanes of the warp must call this. T = lanes per quantization block.
__device__ __forceinline__ float block_absmax(float m, int lanes_per_block) {
  for (int o = lanes_per_block >> 1; o > 0; o >>= 1)
    m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

template <int BITS>
__device__ __forceinline__ __half scale_from_absmax(float m) {
  float s = __fdiv_rn(m, (float)Range<BITS>::qmax);
  if (!(m > 0.0f)) s = 1.0f;
  return __float2half_rn(s);
}

// ---------------------------------------------------------------------------
// quantize values with a given fp32(fp16 scale); returns signed codes in [qmin, qmax]
// ---------------------------------------------------------------------------
// The kernels are instruction-issue bound, not DRAM bound, so the inner loop avoids the
// quarter-rate conversion unit entirely: floor / round-half-even / float->int / int->float
// are done with the 2^23 "magic number" adds, which are exact for the code range.
constexpr float kTwo23 = 8388608.0f;        // 2^23
constexpr float kMagic = 12582912.0f;       // 1.5 * 2^23: (c + kMagic) holds int c in its mantissa
constexpr int kMagicBits = 0x4B400000;

// Correctly rounded a / sf for many numerators and one denominator: y = RN(1/sf) once,
// then q0 = RN(a*y), r = a - q0*sf (exact, fma), q = RN(q0 + r*y).  With y correctly
// rounded and q0 within one ulp this is the IEEE quotient (Markstein); sf is an fp16 value,
// so its significand is never all ones, the one case the argument excludes.  sf == 0 (the
// fp16 scale underflowed) takes the plain IEEE divide so that inf / NaN come out as on the
// host.
struct Divider {
  float sf, y;
  __device__ __forceinline__ explicit Divider(float s) {
    sf = s;
    y = __frcp_rn(s);
  }
  __device__ __forceinline__ float operator()(float a) const {
    if (__builtin_expect(sf == 0.0f, 0)) return __fdiv_rn(a, sf);
    const float q0 = __fmul_rn(a, y);
    const float r = __fmaf_rn(-q0, sf, a);
    return __fmaf_rn(r, y, q0);
  }
};

// Quantizes one value given n = |x| / sf and its uniform draw. Returns the signed code;
// *cf receives the same code as a float (never -0), which is what dequantization
// multiplies by the scale.
template <int BITS, bool SR>
__device__ __forceinline__ int quant_core(float x, float n, float u, float* cf) {
  float mag;
  if constexpr (SR) {
    const float lo = __fsub_rn(__fadd_rd(n, kTwo23), kTwo23);  // floor(n) for 0 <= n < 2^23
    const float p = __fsub_rn(n, lo);                          // in [0, 1) for finite n
    mag = u < p ? __fadd_rn(lo, 1.0f) : lo;
  } else {
    mag = __fsub_rn(__fadd_rn(n, kTwo23), kTwo23);             // round half to even
  }
  float s = mag;
  if constexpr (BITS != 1)
    s = __uint_as_float(__float_as_uint(mag) | (__float_as_uint(x) & 0x80000000u));
  float c = fminf(fmaxf(s, (float)Range<BITS>::qmin), (float)Range<BITS>::qmax);
  c = (s != s) ? 0.0f : c;  // NaN (0/0 when the fp16 scale underflows) converts to 0
  const float t = __fadd_rn(c, kMagic);
  *cf = __fsub_rn(t, kMagic);
  return __float_as_int(t) - kMagicBits;
}

template <int BITS, bool SR>
__device__ __forceinline__ int quant1(float x, float sf, uint32_t key, uint32_t idx, float* cf) {
  const float n = __fdiv_rn(fabsf(x), sf);
  float u = 0.0f;
  if constexpr (SR) u = sr_uniform(key, idx);
  return quant_core<BITS, SR>(x, n, u, cf);
}

template <int BITS, bool SR>
__device__ __forceinline__ int quant1(float x, float sf, uint32_t key, uint32_t idx) {
  float unused;
  return quant1<BITS, SR>(x, sf, key, idx, &unused);
}

// Quantize + dequantize a group of 8 starting at index idx0: q gets the codes, d the
// dequantized values (code * sf).  The two rare cases (underflowed scale, odd first index)
// are decided once per group, so the per-element code is branch-free.
template <int BITS, bool SR>
__device__ __forceinline__ void quant8_dq(const float (&x)[GROUP], float sf, uint32_t key,
                                          uint32_t idx0, int (&q)[GROUP], float (&d)[GROUP]) {
  float n[GROUP];
  if (__builtin_expect(sf == 0.0f, 0)) {
#pragma unroll
    for (int i = 0; i < GROUP; ++i) n[i] = __fdiv_rn(fabsf(x[i]), sf);
  } else {
    const float y = __frcp_rn(sf);  // see Divider: correctly rounded quotients
#pragma unroll
    for (int i = 0; i < GROUP; ++i) {
      const float a = fabsf(x[i]);
      const float q0 = __fmul_rn(a, y);
      n[i] = __fmaf_rn(__fmaf_rn(-q0, sf, a), y, q0);
    }
  }
  float u[GROUP];
#pragma unroll
  for (int i = 0; i < GROUP; ++i) u[i] = 0.0f;
  if constexpr (SR) {
    if ((idx0 & 1u) == 0u) {  // the usual case: two elements share one hash
#pragma unroll
      for (int i = 0; i < GROUP; i += 2) {
        const uint32_t h = sr_hash(key, (idx0 + i) >> 1);
        u[i] = sr_u16(h & 0xFFFFu);
        u[i + 1] = sr_u16(h >> 16);
      }
    } else {
#pragma unroll
      for (int i = 0; i < GROUP; ++i) u[i] = sr_uniform(key, idx0 + i);
    }
  }
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    float cf;
    q[i] = quant_core<BITS, SR>(x[i], n[i], u[i], &cf);
    d[i] = __fmul_rn(cf, sf);
  }
}

template <int BITS, bool SR>
__device__ __forceinline__ void quant8(const float (&x)[GROUP], float sf, uint32_t key,
                                       uint32_t idx0, int (&q)[GROUP]) {
  float d[GROUP];
  quant8_dq<BITS, SR>(x, sf, key, idx0, q, d);
}

__device__ __forceinline__ void dequant8(const int (&q)[GROUP], float sf, float (&y)[GROUP]) {
#pragma unroll
  for (int i = 0; i < GROUP; ++i) y[i] = __fmul_rn((float)q[i], sf);
}

// ---------------------------------------------------------------------------
// register packing of one 8-element group: BITS bytes, first element lowest
// ---------------------------------------------------------------------------
template <int BITS> struct Packed8 {
  static constexpr int WORDS = (BITS + 3) / 4;  // 32-bit words, last may be partial
  uint32_t w[WORDS];
};

template <int BITS>
__device__ __forceinline__ Packed8<BITS> pack8(const int (&q)[GROUP]) {
  Packed8<BITS> out;
#pragma unroll
  for (int i = 0; i < Packed8<BITS>::WORDS; ++i) out.w[i] = 0u;
  constexpr uint32_t mask = BITS >= 32 ? 0xffffffffu : ((1u << BITS) - 1u);
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    const uint32_t code = (uint32_t)(q[i] - Range<BITS>::qmin) & mask;
    const int bit = i * BITS;
    out.w[bit >> 5] |= code << (bit & 31);
    if ((bit & 31) + BITS > 32) out.w[(bit >> 5) + 1] |= code >> (32 - (bit & 31));
  }
  return out;
}

// ---------------------------------------------------------------------------
// Lean quantize + pack of one group for the common case: finite absmax, finite non-zero fp16
// scale, whole-word codes (1, 2, 4, 8 bit).  Same codes as quant8_dq + pack8, fewer
// instructions per element (the kernels that call it are bound by instruction issue):
//   * no NaN rule and no underflow branch per element: those cases are decided once per group
//     (lean_group_ok) and take the general path;
//   * nearest rounding works on the SIGNED quotient (round-half-even is symmetric), so there is
//     no |x| and no sign transfer;
//   * the clamped code c is turned into its stored form by ONE add, t = c + (1.5 * 2^23 - qmin):
//     the float's bit pattern is 0x4B400000 + (c - qmin);
//   * the bit pattern is multiplied into its place with an integer multiply-add; the constant
//     that the 0x4B400000 parts add up to (mod 2^32) is subtracted once per word.
// d (if wanted) receives code * sf with the code as a float that is never -0.
// ---------------------------------------------------------------------------
template <int BITS> struct LeanOk {
  static constexpr bool value = BITS == 1 || BITS == 2 || BITS == 4 || BITS == 8;
};

__device__ __forceinline__ bool lean_group_ok(float absmax, float sf) {
  // false for NaN / inf absmax, for a scale that underflowed to 0 and for one that
  // overflowed fp16 (inf)
  return absmax < 3.0e38f && sf > 0.0f && sf <= 65504.0f;
}

template <int BITS, bool SR, bool WANT_D>
__device__ __forceinline__ Packed8<BITS> quant8_pack_lean(const float (&x)[GROUP], float sf,
                                                          uint32_t key, uint32_t idx0,
                                                          float (&d)[GROUP]) {
  static_assert(LeanOk<BITS>::value, "lean path: whole-word codes only");
  constexpr float lo = (float)Range<BITS>::qmin, hi = (float)Range<BITS>::qmax;
  constexpr float magic = kMagic - (float)Range<BITS>::qmin;  // exact: small integer offset
  constexpr uint32_t magic_bits = 0x4B400000u;                // bits of `magic` + (c - qmin)
  constexpr int PER_WORD = BITS == 8 ? 4 : 8;
  const float y = __frcp_rn(sf);
  float u[GROUP];
  if constexpr (SR) {
    if ((idx0 & 1u) == 0u) {  // the usual case: two elements share one hash
#pragma unroll
      for (int i = 0; i < GROUP; i += 2) {
        const uint32_t h = sr_hash(key, (idx0 + i) >> 1);
        u[i] = sr_u16(h & 0xFFFFu);
        u[i + 1] = sr_u16(h >> 16);
      }
    } else {
#pragma unroll
      for (int i = 0; i < GROUP; ++i) u[i] = sr_uniform(key, idx0 + i);
    }
  }
  Packed8<BITS> out;
#pragma unroll
  for (int k = 0; k < Packed8<BITS>::WORDS; ++k) out.w[k] = 0u;
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    float s;
    if constexpr (SR) {
      const float a = fabsf(x[i]);
      const float q0 = __fmul_rn(a, y);
      const float n = __fmaf_rn(__fmaf_rn(-q0, sf, a), y, q0);   // IEEE a / sf (see Divider)
      const float fl = __fsub_rn(__fadd_rd(n, kTwo23), kTwo23);  // floor(n)
      const float frac = __fsub_rn(n, fl);
      const float mag = u[i] < frac ? __fadd_rn(fl, 1.0f) : fl;
      s = BITS == 1 ? mag
                    : __uint_as_float(__float_as_uint(mag) | (__float_as_uint(x[i]) & 0x80000000u));
    } else {
      const float a = BITS == 1 ? fabsf(x[i]) : x[i];
      const float q0 = __fmul_rn(a, y);
      s = __fmaf_rn(__fmaf_rn(-q0, sf, a), y, q0);               // signed IEEE quotient
    }
    const float c = fminf(fmaxf(s, lo), hi);   // integer bounds: clamping commutes with rounding
    const float t = __fadd_rn(c, magic);       // nearest: rounds half to even here
    const int bit = (i % PER_WORD) * BITS;
    out.w[i / PER_WORD] = __float_as_uint(t) * (1u << bit) + out.w[i / PER_WORD];
    if constexpr (WANT_D) d[i] = __fmul_rn(__fsub_rn(t, magic), sf);
  }
  // what the magic_bits parts added up to, modulo 2^32
  uint32_t garbage = 0u;
#pragma unroll
  for (int i = 0; i < PER_WORD; ++i) garbage += magic_bits << (i * BITS);
#pragma unroll
  for (int k = 0; k < Packed8<BITS>::WORDS; ++k) out.w[k] -= garbage;
  return out;
}

// Quantize (+ dequantize) + pack one group: the lean path when it applies, else the general one.
template <int BITS, bool SR, bool WANT_D>
__device__ __forceinline__ Packed8<BITS> quant8_packed(const float (&x)[GROUP], float absmax,
                                                       float sf, uint32_t key, uint32_t idx0,
                                                       float (&d)[GROUP]) {
  if constexpr (LeanOk<BITS>::value) {
    if (__builtin_expect(lean_group_ok(absmax, sf), 1))
      return quant8_pack_lean<BITS, SR, WANT_D>(x, sf, key, idx0, d);
  }
  int q[GROUP];
  quant8_dq<BITS, SR>(x, sf, key, idx0, q, d);
  return pack8<BITS>(q);
}

template <int BITS>
__device__ __forceinline__ void unpack8(const Packed8<BITS>& in, int (&q)[GROUP]) {
  constexpr uint32_t mask = (1u << BITS) - 1u;
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    const int bit = i * BITS;
    uint32_t code = in.w[bit >> 5] >> (bit & 31);
    if ((bit & 31) + BITS > 32) code |= in.w[(bit >> 5) + 1] << (32 - (bit & 31));
    code &= mask;
    if constexpr (BITS == 16) {
      q[i] = (int)(int16_t)(uint16_t)(code + (uint32_t)Range<16>::qmin);  // int16 wrap
    } else {
      q[i] = (int)code + Range<BITS>::qmin;
    }
  }
}

// Unpack straight to float code values (code + qmin) without an int-to-float conversion:
// OR the code into the mantissa of 2^23 and subtract 2^23 - qmin.
template <int BITS>
__device__ __forceinline__ void unpack8f(const Packed8<BITS>& in, float (&v)[GROUP]) {
  constexpr uint32_t mask = (1u << BITS) - 1u;
  constexpr float bias = 8388608.0f - (float)Range<BITS>::qmin;
#pragma unroll
  for (int i = 0; i < GROUP; ++i) {
    const int bit = i * BITS;
    uint32_t code = in.w[bit >> 5] >> (bit & 31);
    if ((bit & 31) + BITS > 32) code |= in.w[(bit >> 5) + 1] << (32 - (bit & 31));
    code &= mask;
    v[i] = __fsub_rn(__uint_as_float(0x4B000000u | code), bias);
  }
}

// Store / load a full group at byte offset group_index * BITS. The widest naturally
// aligned access is used: 1, 2, 4, 8 bytes, 3 x 4 bytes (12-bit), 16 bytes.
template <int BITS>
__device__ __forceinline__ void store_group(uint8_t* base, long long group_index,
                                            const Packed8<BITS>& p) {
  uint8_t* dst = base + group_index * BITS;
  if constexpr (BITS == 1) {
    *dst = (uint8_t)p.w[0];
  } else if constexpr (BITS == 2) {
    *reinterpret_cast<uint16_t*>(dst) = (uint16_t)p.w[0];
  } else if constexpr (BITS == 4) {
    *reinterpret_cast<uint32_t*>(dst) = p.w[0];
  } else if constexpr (BITS == 8) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(p.w[0], p.w[1]);
  } else if constexpr (BITS == 12) {
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    d[0] = p.w[0]; d[1] = p.w[1]; d[2] = p.w[2];
  } else {
    *reinterpret_cast<uint4*>(dst) = make_uint4(p.w[0], p.w[1], p.w[2], p.w[3]);
  }
}

template <int BITS>
__device__ __forceinline__ Packed8<BITS> load_group(const uint8_t* base, long long group_index) {
  Packed8<BITS> p;
  const uint8_t* src = base + group_index * BITS;
  if constexpr (BITS == 1) {
    p.w[0] = *src;
  } else if constexpr (BITS == 2) {
    p.w[0] = *reinterpret_cast<const uint16_t*>(src);
  } else if constexpr (BITS == 4) {
    p.w[0] = *reinterpret_cast<const uint32_t*>(src);
  } else if constexpr (BITS == 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    p.w[0] = v.x; p.w[1] = v.y;
  } else if constexpr (BITS == 12) {
    const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
    p.w[0] = s[0]; p.w[1] = s[1]; p.w[2] = s[2];
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    p.w[0] = v.x; p.w[1] = v.y; p.w[2] = v.z; p.w[3] = v.w;
  }
  return p;
}

// Byte-wise tail variants: only the first `nbytes` bytes of the group exist.
template <int BITS>
__device__ __forceinline__ void store_group_bytes(uint8_t* base, long long group_index,
                                                  const Packed8<BITS>& p, int nbytes) {
  uint8_t* dst = base + group_index * BITS;
  for (int i = 0; i < nbytes; ++i) dst[i] = (uint8_t)(p.w[i >> 2] >> ((i & 3) * 8));
}

template <int BITS>
__device__ __forceinline__ Packed8<BITS> load_group_bytes(const uint8_t* base,
                                                          long long group_index, int nbytes) {
  Packed8<BITS> p;
#pragma unroll
  for (int i = 0; i < Packed8<BITS>::WORDS; ++i) p.w[i] = 0u;
  const uint8_t* src = base + group_index * BITS;
  for (int i = 0; i < nbytes; ++i) p.w[i >> 2] |= (uint32_t)src[i] << ((i & 3) * 8);
  return p;
}

// wire bytes of `n` codes
__host__ __device__ inline long long packed_nbytes(long long n, int bits) {
  if (bits == 12) return 3 * ((n + 1) / 2);
  if (bits == 16) return 2 * n;
  return (n * bits + 7) / 8;
}

}  // namespace bcom
