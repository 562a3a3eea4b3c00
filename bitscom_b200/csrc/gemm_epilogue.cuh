// Epilogue of the tcgen05 GEMM kernels: one warp moves its 32 accumulator rows (TMEM lanes)
// of a BN-column tile from tensor memory to global memory, as bf16 or fp32, overwriting or
// accumulating.  Shared by the one-CTA kernel (gemm_tcgen05.cu) and the CTA-pair kernel
// (gemm_tcgen05_2cta.cu); thread t of the warp owns row `row` = first row of the warp + t.
#pragma once

#include "tc_common.cuh"

namespace gemm {

// taddr: TMEM address of the warp's first lane at the tile's first column.
// C row `row`, columns [n0, n0 + BN) are written where row < M and column < N (N % 8 == 0).
// R (bf16 [M, N] with leading dimension ldr, or null): added to the product before the bf16
// result is rounded; only read by the bf16, non-accumulating form (a linear layer whose output
// joins a residual stream: C = R + A x B in one pass instead of a GEMM and an add kernel).
template <int BN, bool OUT_F32, bool ACCUM>
__device__ __forceinline__ void store_accumulator_rows(uint32_t taddr, void* C, long long ldc,
                                                       int row, int n0, int M, int N,
                                                       const void* R = nullptr,
                                                       long long ldr = 0) {
  if constexpr (OUT_F32 && ACCUM) {
    // Accumulating fp32 epilogue (weight gradients): the old values of chunk c+1 are
    // requested before chunk c is finished, so their latency hides behind the TMEM
    // load, the adds and the stores of the current chunk.
    float* crow = reinterpret_cast<float*>(C) + (long long)row * ldc + n0;
    const bool row_ok = row < M;
    float4 old[8], nxt[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      old[v] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row_ok && n0 + v * 4 < N) old[v] = *reinterpret_cast<const float4*>(crow + v * 4);
    }
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(taddr + c * 32, r);
      const int col0 = n0 + c * 32;
      if (c + 1 < BN / 32) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          nxt[v] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (row_ok && col0 + 32 + v * 4 < N)
            nxt[v] = *reinterpret_cast<const float4*>(crow + (c + 1) * 32 + v * 4);
        }
      }
      tc::tmem_wait_ld();
      if (row_ok) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          if (col0 + v * 4 < N) {
            float4 o = old[v];
            o.x += __uint_as_float(r[4 * v]);
            o.y += __uint_as_float(r[4 * v + 1]);
            o.z += __uint_as_float(r[4 * v + 2]);
            o.w += __uint_as_float(r[4 * v + 3]);
            *reinterpret_cast<float4*>(crow + c * 32 + v * 4) = o;
          }
        }
      }
#pragma unroll
      for (int v = 0; v < 8; ++v) old[v] = nxt[v];
    }
  } else {
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(taddr + c * 32, r);
      const int col0 = n0 + c * 32;
      uint4 res[4];
      if constexpr (!OUT_F32 && !ACCUM) {
        // the residual row segment is requested before the wait on the TMEM load
        if (R != nullptr && row < M) {
          const __nv_bfloat16* rrow =
              reinterpret_cast<const __nv_bfloat16*>(R) + (long long)row * ldr + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v)
            if (col0 + v * 8 < N) res[v] = *reinterpret_cast<const uint4*>(rrow + v * 8);
        }
      }
      tc::tmem_wait_ld();
      if (row < M && col0 < N) {
        if constexpr (OUT_F32) {
          float* dst = reinterpret_cast<float*>(C) + (long long)row * ldc + col0;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            if (col0 + v * 4 < N) {
              float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                     __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              if constexpr (ACCUM) {
                const float4 old = *reinterpret_cast<const float4*>(dst + v * 4);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(dst + v * 4) = o;
            }
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row * ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < N) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * v + i]);
              if constexpr (ACCUM) {
                const uint4 old = *reinterpret_cast<const uint4*>(dst + v * 8);
                const __nv_bfloat16* oh = reinterpret_cast<const __nv_bfloat16*>(&old);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] += __bfloat162float(oh[i]);
              } else if (R != nullptr) {
                const __nv_bfloat16* rh = reinterpret_cast<const __nv_bfloat16*>(&res[v]);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] += __bfloat162float(rh[i]);
              }
              uint4 o;
              __nv_bfloat162* oh2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i) oh2[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
              *reinterpret_cast<uint4*>(dst + v * 8) = o;
            }
          }
        }
      }
    }
  }
}

}  // namespace gemm
