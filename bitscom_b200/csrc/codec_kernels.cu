// Standalone codec kernels (sm_100a): blockwise quantize+pack, unpack+dequantize,
// per-tensor quantize / dequantize with a device-side absmax, and pack / unpack of
// int16 codes for 1/2/4/8/12/16 bits.  They cover the surface of the reference's
// `_lowbit_cuda` extension (cpp/src/lowbit_cuda_kernels.cu:29-250 and the bindings in
// cpp/src/lowbit_cuda_bindings.cpp:38-87) plus bf16 input, 12/16-bit packing and a
// seedable stochastic-rounding stream.  The device functions come from codec.cuh and
// are the same ones the fused collective kernels inline.
//
// Exported with C linkage; every entry point takes raw device pointers and a stream,
// launches asynchronously and returns a cudaError_t as int.
#include <cuda_runtime.h>

#include "codec.cuh"

namespace bcom {

enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

constexpr int kThreads = 256;

static inline int grid_for(long long work_items, int per_cta, int max_ctas) {
  long long g = (work_items + per_cta - 1) / per_cta;
  if (g < 1) g = 1;
  if (g > max_ctas) g = max_ctas;
  return (int)g;
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// ---------------------------------------------------------------------------
// fast path: 8 elements per thread, block = 8*T elements inside one warp
// ---------------------------------------------------------------------------
// Quantize, pack and store one group whose values are already in registers.
template <typename T, int BITS, bool SR>
__device__ __forceinline__ void quantize_group(const float (&v)[GROUP], long long g,
                                               long long groups, long long n,
                                               int lanes_per_block, uint32_t key,
                                               uint32_t idx_offset, uint8_t* __restrict__ packed,
                                               __half* __restrict__ scales) {
  const long long base = g * GROUP;
  const bool full = base + GROUP <= n;
  const float m = block_absmax(absmax8(v), lanes_per_block);
  const __half sh = scale_from_absmax<BITS>(m);
  const float sf = __half2float(sh);
  if (g >= groups) return;
  if ((g & (lanes_per_block - 1)) == 0) scales[g / lanes_per_block] = sh;
  if (full) {
    float unused[GROUP];
    store_group<BITS>(packed, g, quant8_packed<BITS, SR, false>(
        v, m, sf, key, idx_offset + (uint32_t)base, unused));
    return;
  }
  int q[GROUP];
  quant8<BITS, SR>(v, sf, key, idx_offset + (uint32_t)base, q);
  // positions past the end carry code 0, like the host packer's padding
#pragma unroll
  for (int i = 0; i < GROUP; ++i)
    if (base + i >= n) q[i] = Range<BITS>::qmin;
  store_group_bytes<BITS>(packed, g, pack8<BITS>(q), (int)packed_nbytes(n - base, BITS));
}

// Two groups per thread and iteration (a stride apart, so that both stay coalesced): the loads
// of both are in flight before the first shuffle.  With one group per iteration the kernel ran
// at the same speed for fp32 and bf16 inputs, i.e. it waited on its one outstanding load.
template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kThreads)
blockwise_quantize_pack_fast(const T* __restrict__ x, long long n, int lanes_per_block,
                             uint32_t key, uint32_t idx_offset,
                             uint8_t* __restrict__ packed, __half* __restrict__ scales) {
  const long long groups = (n + GROUP - 1) / GROUP;
  const long long groups_padded = (groups + 31) & ~31LL;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; g0 < groups_padded;
       g0 += 2 * stride) {
    const long long g1 = g0 + stride;
    const bool two = g1 < groups_padded;  // warp-uniform: stride and the padding are multiples of 32
    float v0[GROUP], v1[GROUP];
    if (g0 * GROUP + GROUP <= n) load8_vec(x + g0 * GROUP, v0);
    else load8_guard(x, g0 * GROUP, n, v0);
    if (two) {
      if (g1 * GROUP + GROUP <= n) load8_vec(x + g1 * GROUP, v1);
      else load8_guard(x, g1 * GROUP, n, v1);
    }
    quantize_group<T, BITS, SR>(v0, g0, groups, n, lanes_per_block, key, idx_offset, packed,
                                scales);
    if (two)
      quantize_group<T, BITS, SR>(v1, g1, groups, n, lanes_per_block, key, idx_offset, packed,
                                  scales);
  }
}

template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
blockwise_unpack_dequantize_fast(const uint8_t* __restrict__ packed,
                                 const __half* __restrict__ scales, long long n,
                                 int lanes_per_block, T* __restrict__ out) {
  const long long groups = (n + GROUP - 1) / GROUP;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const long long base = g * GROUP;
    const bool full = base + GROUP <= n;
    const Packed8<BITS> p = full ? load_group<BITS>(packed, g)
                                 : load_group_bytes<BITS>(packed, g,
                                                          (int)packed_nbytes(n - base, BITS));
    const float sf = __half2float(scales[g / lanes_per_block]);
    float y[GROUP];
    unpack8f<BITS>(p, y);
#pragma unroll
    for (int i = 0; i < GROUP; ++i) y[i] = __fmul_rn(y[i], sf);
    if (full) {
      store8_vec(out + base, y);
    } else {
      store8_guard(out, base, n, y);
    }
  }
}

// ---------------------------------------------------------------------------
// generic path: any block size whose packed form is byte aligned, any alignment.
// One warp per quantization block; a lane owns "units" of UNIT elements that pack
// into UBYTES whole bytes.
// ---------------------------------------------------------------------------
template <int BITS> struct Unit {
  static constexpr int elems = BITS <= 8 ? 8 / BITS : (BITS == 12 ? 2 : 1);
  static constexpr int bytes = BITS <= 8 ? 1 : (BITS == 12 ? 3 : 2);
};

template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kThreads)
blockwise_quantize_pack_generic(const T* __restrict__ x, long long n, int block,
                                uint32_t key, uint32_t idx_offset,
                                uint8_t* __restrict__ packed, __half* __restrict__ scales) {
  constexpr int UE = Unit<BITS>::elems;
  constexpr int UB = Unit<BITS>::bytes;
  constexpr uint32_t mask = (1u << BITS) - 1u;
  const int lane = threadIdx.x & 31;
  const long long nblocks = (n + block - 1) / block;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long b = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < nblocks;
       b += warps) {
    const long long start = b * block;
    const long long stop = min(start + (long long)block, n);
    float m = 0.0f;
    for (long long i = start + lane; i < stop; i += 32)
      m = max_nan(m, fabsf(Elem<T>::to_f(x[i])));
    m = block_absmax(m, 32);
    const __half sh = scale_from_absmax<BITS>(m);
    const float sf = __half2float(sh);
    if (lane == 0) scales[b] = sh;
    const long long units = (stop - start + UE - 1) / UE;
    for (long long u = lane; u < units; u += 32) {
      uint32_t bits = 0u;
#pragma unroll
      for (int e = 0; e < UE; ++e) {
        const long long i = start + u * UE + e;
        int q = Range<BITS>::qmin;  // tail padding is code 0
        if (i < stop)
          q = quant1<BITS, SR>(Elem<T>::to_f(x[i]), sf, key, idx_offset + (uint32_t)i);
        bits |= ((uint32_t)(q - Range<BITS>::qmin) & mask) << (e * BITS);
      }
      uint8_t* dst = packed + (start / UE) * UB + u * UB;
      const long long limit = packed_nbytes(n, BITS);
#pragma unroll
      for (int k = 0; k < UB; ++k)
        if ((dst - packed) + k < limit) dst[k] = (uint8_t)(bits >> (8 * k));
    }
  }
}

template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads)
blockwise_unpack_dequantize_generic(const uint8_t* __restrict__ packed,
                                    const __half* __restrict__ scales, long long n, int block,
                                    T* __restrict__ out) {
  constexpr int UE = Unit<BITS>::elems;
  constexpr int UB = Unit<BITS>::bytes;
  constexpr uint32_t mask = (1u << BITS) - 1u;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long u = i / UE;
    const int e = (int)(i - u * UE);
    uint32_t bits = 0u;
#pragma unroll
    for (int k = 0; k < UB; ++k) bits |= (uint32_t)packed[u * UB + k] << (8 * k);
    const uint32_t code = (bits >> (e * BITS)) & mask;
    int q;
    if constexpr (BITS == 16) {
      q = (int)(int16_t)(uint16_t)(code + 0x8000u);
    } else {
      q = (int)code + Range<BITS>::qmin;
    }
    out[i] = Elem<T>::from_f(__fmul_rn((float)q, __half2float(scales[i / block])));
  }
}

// ---------------------------------------------------------------------------
// per-tensor quantizer: absmax on the device (no host round trip), then codes
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const T* __restrict__ x, long long n, unsigned int* __restrict__ absmax_bits) {
  float m = 0.0f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // whole 8-element groups as one vector access when the tensor is aligned for it
  const uintptr_t mask = sizeof(T) == 4 ? 31 : 15;
  const long long groups = (reinterpret_cast<uintptr_t>(x) & mask) == 0 ? n / GROUP : 0;
  for (long long g = tid; g < groups; g += stride) {
    float v[GROUP];
    load8_vec(x + g * GROUP, v);
    m = max_nan(m, absmax8(v));
  }
  for (long long i = groups * GROUP + tid; i < n; i += stride)
    m = max_nan(m, fabsf(Elem<T>::to_f(x[i])));
  m = block_absmax(m, 32);
  __shared__ float part[kThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.0f;
    m = block_absmax(m, 32);
    // non-negative floats order like their bit patterns
    if (threadIdx.x == 0) atomicMax(absmax_bits, __float_as_uint(m));
  }
}

template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kThreads)
quantize_per_tensor_kernel(const T* __restrict__ x, long long n,
                           const unsigned int* __restrict__ absmax_bits, uint32_t key,
                           uint32_t idx_offset, int16_t* __restrict__ q,
                           float* __restrict__ scale_out) {
  const float peak = __uint_as_float(*absmax_bits);
  const float scale = peak != 0.0f ? __fdiv_rn(peak, (float)Range<BITS>::qmax) : 1.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  auto code = [&](float xv, long long i) -> int16_t {
    const float r = __fdiv_rn(xv, scale);
    float v;
    if constexpr (SR) {
      const float lo = floorf(r);
      const float p = fminf(fmaxf(__fsub_rn(r, lo), 0.0f), 1.0f);
      v = sr_uniform(key, idx_offset + (uint32_t)i) < p ? __fadd_rn(lo, 1.0f) : lo;
    } else {
      v = rintf(r);
    }
    const float c = fminf(fmaxf(v, (float)Range<BITS>::qmin), (float)Range<BITS>::qmax);
    return (v != v) ? (int16_t)0 : (int16_t)(int)c;
  };
  // whole 8-element groups: one vector load, one 16-byte store of the codes
  const uintptr_t mask = sizeof(T) == 4 ? 31 : 15;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & mask) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  const long long groups = vec ? n / GROUP : 0;
  for (long long g = tid; g < groups; g += stride) {
    float v[GROUP];
    load8_vec(x + g * GROUP, v);
    uint4 raw;
    int16_t* h = reinterpret_cast<int16_t*>(&raw);
#pragma unroll
    for (int i = 0; i < GROUP; ++i) h[i] = code(v[i], g * GROUP + i);
    *reinterpret_cast<uint4*>(q + g * GROUP) = raw;
  }
  for (long long i = groups * GROUP + tid; i < n; i += stride)
    q[i] = code(Elem<T>::to_f(x[i]), i);
}

__global__ void __launch_bounds__(kThreads)
dequantize_per_tensor_kernel(const int16_t* __restrict__ q, long long n, float scale,
                             float* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 31) == 0;
  const long long groups = vec ? n / GROUP : 0;
  for (long long g = tid; g < groups; g += stride) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q + g * GROUP));
    const int16_t* h = reinterpret_cast<const int16_t*>(&raw);
    float y[GROUP];
#pragma unroll
    for (int i = 0; i < GROUP; ++i) y[i] = __fmul_rn((float)h[i], scale);
    store8_vec(out + g * GROUP, y);
  }
  for (long long i = groups * GROUP + tid; i < n; i += stride)
    out[i] = __fmul_rn((float)q[i], scale);
}

// ---------------------------------------------------------------------------
// pack / unpack of int16 codes; a thread owns one 8-element group
// ---------------------------------------------------------------------------
template <int BITS>
__global__ void __launch_bounds__(kThreads)
pack_kernel(const int16_t* __restrict__ q, long long n, uint8_t* __restrict__ packed) {
  const bool vec16 = (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  const long long groups = (n + GROUP - 1) / GROUP;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const long long base = g * GROUP;
    int v[GROUP];
    if (base + GROUP <= n && vec16) {   // eight codes as one 16-byte load
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q + base));
      const int16_t* h = reinterpret_cast<const int16_t*>(&raw);
#pragma unroll
      for (int i = 0; i < GROUP; ++i) v[i] = (int)h[i];
    } else {
#pragma unroll
      for (int i = 0; i < GROUP; ++i) v[i] = base + i < n ? (int)q[base + i] : Range<BITS>::qmin;
    }
    const Packed8<BITS> p = pack8<BITS>(v);
    if (base + GROUP <= n) {
      store_group<BITS>(packed, g, p);
    } else {
      store_group_bytes<BITS>(packed, g, p, (int)packed_nbytes(n - base, BITS));
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(kThreads)
unpack_kernel(const uint8_t* __restrict__ packed, long long n, int16_t* __restrict__ q) {
  const bool vec16 = (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  const long long groups = (n + GROUP - 1) / GROUP;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const long long base = g * GROUP;
    const bool full = base + GROUP <= n;
    const Packed8<BITS> p = full ? load_group<BITS>(packed, g)
                                 : load_group_bytes<BITS>(packed, g,
                                                          (int)packed_nbytes(n - base, BITS));
    int v[GROUP];
    unpack8<BITS>(p, v);
    if (full && vec16) {   // eight codes as one 16-byte store
      uint4 raw;
      int16_t* h = reinterpret_cast<int16_t*>(&raw);
#pragma unroll
      for (int i = 0; i < GROUP; ++i) h[i] = (int16_t)v[i];
      *reinterpret_cast<uint4*>(q + base) = raw;
    } else {
#pragma unroll
      for (int i = 0; i < GROUP; ++i)
        if (base + i < n) q[base + i] = (int16_t)v[i];
    }
  }
}

// ---------------------------------------------------------------------------
// dispatch helpers
// ---------------------------------------------------------------------------
#define BCOM_DISPATCH_BITS(bits, ...)                                  \
  switch (bits) {                                                      \
    case 1:  { constexpr int BITS = 1;  __VA_ARGS__; break; }          \
    case 2:  { constexpr int BITS = 2;  __VA_ARGS__; break; }          \
    case 4:  { constexpr int BITS = 4;  __VA_ARGS__; break; }          \
    case 8:  { constexpr int BITS = 8;  __VA_ARGS__; break; }          \
    case 12: { constexpr int BITS = 12; __VA_ARGS__; break; }          \
    case 16: { constexpr int BITS = 16; __VA_ARGS__; break; }          \
    default: return (int)cudaErrorInvalidValue;                        \
  }

#define BCOM_DISPATCH_DTYPE(dtype, ...)                                           \
  switch (dtype) {                                                                \
    case kF32:  { using T = float;         __VA_ARGS__; break; }                  \
    case kF16:  { using T = __half;        __VA_ARGS__; break; }                  \
    case kBF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }                  \
    default: return (int)cudaErrorInvalidValue;                                   \
  }

static inline bool fast_block(int block) {
  if (block % GROUP) return false;
  const int t = block / GROUP;
  return t >= 1 && t <= 32 && (t & (t - 1)) == 0;
}

}  // namespace bcom

using namespace bcom;

extern "C" {

// 1 if (bits, block) can run on the 8-per-thread fast path for 16-byte aligned data.
int bcom_codec_fast_block(int block) { return fast_block(block) ? 1 : 0; }

// 1 if the generic kernels can handle (bits, block): blocks must start on a byte.
int bcom_codec_generic_ok(int bits, int block) {
  switch (bits) {
    case 1: case 2: case 4: case 8: return block % (8 / bits) == 0;
    case 12: return block % 2 == 0;
    case 16: return 1;
    default: return 0;
  }
}

int bcom_blockwise_quantize_pack(const void* x, int dtype, long long n, int bits, int block,
                                 int stochastic, unsigned int key, unsigned int idx_offset,
                                 void* packed, void* scales, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  // 8-element groups move as one access: 32 bytes for fp32, 16 bytes for fp16 / bf16
  const uintptr_t in_mask = dtype == kF32 ? 31 : 15;
  const bool aligned = ((uintptr_t)x & in_mask) == 0 && ((uintptr_t)packed & 15) == 0;
  if (fast_block(block) && aligned) {
    const long long groups = (n + GROUP - 1) / GROUP;
    const int grid = grid_for(groups, kThreads, sm_count() * 8);
    BCOM_DISPATCH_DTYPE(dtype, BCOM_DISPATCH_BITS(bits, {
      if (stochastic)
        blockwise_quantize_pack_fast<T, BITS, true><<<grid, kThreads, 0, st>>>(
            (const T*)x, n, block / GROUP, key, idx_offset, (uint8_t*)packed, (__half*)scales);
      else
        blockwise_quantize_pack_fast<T, BITS, false><<<grid, kThreads, 0, st>>>(
            (const T*)x, n, block / GROUP, key, idx_offset, (uint8_t*)packed, (__half*)scales);
    }))
    return (int)cudaGetLastError();
  }
  if (!bcom_codec_generic_ok(bits, block)) return (int)cudaErrorNotSupported;
  const long long nblocks = (n + block - 1) / block;
  const int grid = grid_for(nblocks, kThreads / 32, sm_count() * 8);
  BCOM_DISPATCH_DTYPE(dtype, BCOM_DISPATCH_BITS(bits, {
    if (stochastic)
      blockwise_quantize_pack_generic<T, BITS, true><<<grid, kThreads, 0, st>>>(
          (const T*)x, n, block, key, idx_offset, (uint8_t*)packed, (__half*)scales);
    else
      blockwise_quantize_pack_generic<T, BITS, false><<<grid, kThreads, 0, st>>>(
          (const T*)x, n, block, key, idx_offset, (uint8_t*)packed, (__half*)scales);
  }))
  return (int)cudaGetLastError();
}

int bcom_blockwise_unpack_dequantize(const void* packed, const void* scales, int bits,
                                     long long n, int block, void* out, int dtype,
                                     void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const uintptr_t out_mask = dtype == kF32 ? 31 : 15;
  const bool aligned = ((uintptr_t)out & out_mask) == 0 && ((uintptr_t)packed & 15) == 0;
  if (fast_block(block) && aligned) {
    const long long groups = (n + GROUP - 1) / GROUP;
    const int grid = grid_for(groups, kThreads, sm_count() * 8);
    BCOM_DISPATCH_DTYPE(dtype, BCOM_DISPATCH_BITS(bits, {
      blockwise_unpack_dequantize_fast<T, BITS><<<grid, kThreads, 0, st>>>(
          (const uint8_t*)packed, (const __half*)scales, n, block / GROUP, (T*)out);
    }))
    return (int)cudaGetLastError();
  }
  if (!bcom_codec_generic_ok(bits, block)) return (int)cudaErrorNotSupported;
  const int grid = grid_for(n, kThreads, sm_count() * 8);
  BCOM_DISPATCH_DTYPE(dtype, BCOM_DISPATCH_BITS(bits, {
    blockwise_unpack_dequantize_generic<T, BITS><<<grid, kThreads, 0, st>>>(
        (const uint8_t*)packed, (const __half*)scales, n, block, (T*)out);
  }))
  return (int)cudaGetLastError();
}

// absmax_bits: one uint32 of device scratch (the float bits of the running max).
int bcom_quantize_per_tensor(const void* x, int dtype, long long n, int bits, int stochastic,
                             unsigned int key, unsigned int idx_offset, void* absmax_bits,
                             void* q, void* scale_out, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t err = cudaMemsetAsync(absmax_bits, 0, sizeof(unsigned int), st);
  if (err != cudaSuccess) return (int)err;
  const int grid = grid_for(n > 0 ? n : 1, kThreads * 8, sm_count() * 8);
  BCOM_DISPATCH_DTYPE(dtype, {
    if (n > 0)
      absmax_kernel<T><<<grid, kThreads, 0, st>>>((const T*)x, n, (unsigned int*)absmax_bits);
  })
  const int qgrid = grid_for(n > 0 ? n : 1, kThreads * 4, sm_count() * 8);
  BCOM_DISPATCH_DTYPE(dtype, BCOM_DISPATCH_BITS(bits, {
    if (stochastic)
      quantize_per_tensor_kernel<T, BITS, true><<<qgrid, kThreads, 0, st>>>(
          (const T*)x, n, (const unsigned int*)absmax_bits, key, idx_offset, (int16_t*)q,
          (float*)scale_out);
    else
      quantize_per_tensor_kernel<T, BITS, false><<<qgrid, kThreads, 0, st>>>(
          (const T*)x, n, (const unsigned int*)absmax_bits, key, idx_offset, (int16_t*)q,
          (float*)scale_out);
  }))
  return (int)cudaGetLastError();
}

int bcom_dequantize_per_tensor(const void* q, long long n, float scale, void* out,
                               void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n, kThreads * 4, sm_count() * 8);
  dequantize_per_tensor_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
      (const int16_t*)q, n, scale, (float*)out);
  return (int)cudaGetLastError();
}

int bcom_pack(const void* q, long long n, int bits, void* packed, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((n + GROUP - 1) / GROUP, kThreads, sm_count() * 8);
  BCOM_DISPATCH_BITS(bits, {
    pack_kernel<BITS><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        (const int16_t*)q, n, (uint8_t*)packed);
  })
  return (int)cudaGetLastError();
}

int bcom_unpack(const void* packed, long long n, int bits, void* q, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for((n + GROUP - 1) / GROUP, kThreads, sm_count() * 8);
  BCOM_DISPATCH_BITS(bits, {
    unpack_kernel<BITS><<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)packed, n, (int16_t*)q);
  })
  return (int)cudaGetLastError();
}

}  // extern "C"
