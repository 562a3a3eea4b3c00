// Causal flash attention, forward and backward, on tcgen05 tensor cores (sm_100a),
// head_dim 128 (Llama) or 64 (GPT-2), operating directly on the fused projection
// qkv[tokens, 3 * heads * head_dim] (bf16, RoPE already applied where the model has it)
// through TMA tensor maps: no q/k/v copies.  The kernels are templates on the head dim; a
// [rows x head_dim] tile is head_dim / 64 chunks of 64 columns (one 128-byte swizzle row).
//
// TMEM gives every thread one accumulator ROW (thread t <-> TMEM lane t), so row maxima,
// row sums and the softmax need no cross-thread reduction at all.
//
// forward   one CTA per (batch, head, 128 query rows), 2 CTAs per SM.
//           per 64-key block:  S = Q K^T (tcgen05.mma, smem x smem -> TMEM)
//                              rows of S -> registers (tcgen05.ld), online softmax,
//                              P (bf16) -> 128B-swizzled smem
//                              O_blk = P V (V consumed MN-major straight from its row-major
//                              tile), rows of O_blk -> registers, O = O * alpha + O_blk
//           the next K / V tile is requested the moment the MMA that read the previous one
//           has completed, so TMA runs under the softmax.
// backward  one CTA per (batch, head, 128 keys), looping over the 128-row query blocks at
//           or below the diagonal; everything is kept transposed (rows = keys):
//             S^T = K Q^T, dP^T = V dO^T                       -> TMEM
//             P^T = exp2(S^T * c - lse), dS^T = P^T o (dP^T - D) * scale   -> smem (bf16)
//             dV += P^T dO, dK += dS^T Q   (accumulate in TMEM over all query blocks)
//             dQ  = dS K                    -> TMEM -> fp32 atomics into a dQ buffer
//           One smem tile serves as K-major operand of one product and MN-major operand of
//           another (same bytes, different descriptor), so each of Q, K, V, dO is loaded once.
//
// The library baseline is torch SDPA / flash_attn; the reference trainer takes attention
// from its external model package.  All mbarrier waits are bounded (status word + drain).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "tc_common.cuh"

namespace attn {

constexpr int BQ = 128;           // query rows per CTA (forward) / per iteration (backward)
constexpr int BKF = 64;           // keys per iteration, forward
constexpr int BKB = 128;          // keys per CTA, backward
constexpr int kThreads = 128;      // forward
constexpr int kBwdThreads = 256;   // backward: two warps share each TMEM lane quarter
constexpr unsigned long long kBudgetNs = 2000000000ull;
constexpr float kLog2e = 1.4426950408889634f;

__device__ unsigned int g_status[4];

__device__ __forceinline__ void record_fail(unsigned int code) {
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = threadIdx.x;
  }
}

// byte offset of the 16-byte unit `c8` (0..7) of row `r` inside a 128B-swizzled tile whose
// rows are 128 bytes; `rows` rows form one 64-column chunk
__device__ __forceinline__ uint32_t swz(int r, int c8) {
  return (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// UMMA descriptors for the two ways a [rows x (64 * chunks)-col] tile is consumed.
// K-major: MN = rows, K = columns. Chunk c (64 columns) starts at c * rows * 128.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int rows, int kstep) {
  const int chunk = kstep >> 2;  // 4 k-steps of 16 elements per 64-column chunk
  return tc::make_smem_desc_sw128(base + chunk * rows * 128 + (kstep & 3) * 32, 16, 1024);
}
// MN-major: MN = columns, K = rows. k-step advances 16 rows; chunks are `rows * 128` apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int rows, int kstep) {
  return tc::make_smem_desc_sw128(base + kstep * 16 * 128, rows * 128, 1024);
}

struct FwdParams {
  __nv_bfloat16* out;   // [tokens, heads * HD]
  float* lse2;          // [batch, heads, seq], log2 domain
  int batch, seq, heads;
  float scale_log2;     // softmax scale * log2(e)
};

struct FwdShared {
  uint64_t bar_q, bar_k, bar_v, bar_s, bar_o;
  uint32_t tmem_base;
  volatile int abort;
};

constexpr int FWD_P_BYTES = BQ * BKF * 2;   // 16 KiB
template <int HD> struct Fwd {
  static constexpr int Q_BYTES = BQ * HD * 2;    // 32 KiB at head_dim 128
  static constexpr int K_BYTES = BKF * HD * 2;   // 16 KiB at head_dim 128
  static constexpr int SMEM = Q_BYTES + 2 * K_BYTES + FWD_P_BYTES + 1024 + 128;
  static constexpr int TMEM_COLS = HD == 128 ? 256 : 128;  // S (64) + O (HD), power of two
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tm_q,    // box {64, 128}
                     const __grid_constant__ CUtensorMap tm_kv,   // box {64, 64}
                     const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int FWD_Q_BYTES = Fwd<HD>::Q_BYTES, FWD_K_BYTES = Fwd<HD>::K_BYTES;
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + FWD_Q_BYTES;
  uint8_t* sV = sK + FWD_K_BYTES;
  uint8_t* sP = sV + FWD_K_BYTES;
  FwdShared* sh = reinterpret_cast<FwdShared*>(sP + FWD_P_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qblocks = p.seq / BQ;
  // heavy (late) query blocks first
  const int qb = qblocks - 1 - (int)(blockIdx.x % qblocks);
  const int bh = blockIdx.x / qblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int H = p.heads * HD;
  const int row0 = b * p.seq + qb * BQ;          // first token row of this query block
  const int q_col = h * HD, k_col = H + h * HD, v_col = 2 * H + h * HD;
  const int nblocks = (qb * BQ + BQ) / BKF;      // causal: keys 0 .. q0 + 127

  if (tid == 0) {
    tc::mbar_init(&sh->bar_q, 1);
    tc::mbar_init(&sh->bar_k, 1);
    tc::mbar_init(&sh->bar_v, 1);
    tc::mbar_init(&sh->bar_s, 1);
    tc::mbar_init(&sh->bar_o, 1);
    sh->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&sh->tmem_base, Fwd<HD>::TMEM_COLS);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;
  const uint32_t tS = tmem, tO = tmem + 64;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;

  auto load_k = [&](int j) {
    tc::mbar_expect_tx(&sh->bar_k, FWD_K_BYTES);
#pragma unroll
    for (int c = 0; c < HD / 64; ++c)
      tc::tma_load_2d(sK + c * BKF * 128, &tm_kv, &sh->bar_k, k_col + 64 * c,
                      b * p.seq + j * BKF);
  };
  auto load_v = [&](int j) {
    tc::mbar_expect_tx(&sh->bar_v, FWD_K_BYTES);
#pragma unroll
    for (int c = 0; c < HD / 64; ++c)
      tc::tma_load_2d(sV + c * BKF * 128, &tm_kv, &sh->bar_v, v_col + 64 * c,
                      b * p.seq + j * BKF);
  };

  if (tid == 0) {
    tc::mbar_expect_tx(&sh->bar_q, FWD_Q_BYTES);
#pragma unroll
    for (int c = 0; c < HD / 64; ++c)
      tc::tma_load_2d(sQ + c * BQ * 128, &tm_q, &sh->bar_q, q_col + 64 * c, row0);
    load_k(0);
    load_v(0);
  }

  constexpr uint32_t idesc_s = tc::make_idesc_bf16(BQ, BKF, false, false);
  constexpr uint32_t idesc_o = tc::make_idesc_bf16(BQ, HD, false, true);
  const uint32_t aQ = tc::smem_u32(sQ), aK = tc::smem_u32(sK), aV = tc::smem_u32(sV),
                 aP = tc::smem_u32(sP);

  float o[HD];
#pragma unroll
  for (int i = 0; i < HD; ++i) o[i] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;
  const int q_idx = qb * BQ + tid;  // position of this thread's query inside the sequence

  if (!tc::mbar_wait(&sh->bar_q, 0, kBudgetNs)) { sh->abort = 1; record_fail(1); }

  for (int j = 0; j < nblocks; ++j) {
    const uint32_t par = (uint32_t)j & 1u;
    // ---- S = Q K^T ----
    if (tid == 0) {
      if (!tc::mbar_wait(&sh->bar_k, par, kBudgetNs)) { sh->abort = 1; record_fail(2); }
      tc::tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        tc::umma_bf16(tS, desc_kmajor(aQ, BQ, ks), desc_kmajor(aK, BKF, ks), idesc_s, ks != 0);
      tc::umma_commit(&sh->bar_s);
    }
    if (!tc::mbar_wait(&sh->bar_s, par, kBudgetNs)) { sh->abort = 1; record_fail(3); }
    tc::tc_fence_after_sync();
    if (tid == 0 && j + 1 < nblocks) load_k(j + 1);  // K tile is free again

    // ---- online softmax on this thread's row ----
    float s[BKF];
    {
      uint32_t r[32];
      tc::tmem_ld_32x32(tS + lane_addr, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]) * p.scale_log2;
      tc::tmem_ld_32x32(tS + lane_addr + 32, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(r[i]) * p.scale_log2;
    }
    const int k0 = j * BKF;
    if (k0 + BKF - 1 > qb * BQ) {  // block touches the diagonal
#pragma unroll
      for (int i = 0; i < BKF; ++i)
        if (k0 + i > q_idx) s[i] = -INFINITY;
    }
    float m_blk = m_run;
#pragma unroll
    for (int i = 0; i < BKF; ++i) m_blk = fmaxf(m_blk, s[i]);
    const float alpha = exp2f(m_run - m_blk);  // first block: exp2(-inf) = 0
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < BKF; ++i) {
      s[i] = exp2f(s[i] - m_blk);
      sum += s[i];
    }
    l_run = l_run * alpha + sum;
    m_run = m_blk;
#pragma unroll
    for (int c8 = 0; c8 < BKF / 8; ++c8) {
      uint4 v;
      v.x = pack_bf16(s[c8 * 8 + 0], s[c8 * 8 + 1]);
      v.y = pack_bf16(s[c8 * 8 + 2], s[c8 * 8 + 3]);
      v.z = pack_bf16(s[c8 * 8 + 4], s[c8 * 8 + 5]);
      v.w = pack_bf16(s[c8 * 8 + 6], s[c8 * 8 + 7]);
      *reinterpret_cast<uint4*>(sP + swz(tid, c8)) = v;
    }
    tc::fence_proxy_async();       // generic-proxy smem writes -> visible to the MMA
    tc::tc_fence_before_sync();
    __syncthreads();
    if (sh->abort) break;

    // ---- O_blk = P V ----
    if (tid == 0) {
      if (!tc::mbar_wait(&sh->bar_v, par, kBudgetNs)) { sh->abort = 1; record_fail(4); }
      tc::tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < BKF / 16; ++ks)
        tc::umma_bf16(tO, desc_kmajor(aP, BQ, ks), desc_mnmajor(aV, BKF, ks), idesc_o, ks != 0);
      tc::umma_commit(&sh->bar_o);
    }
    if (!tc::mbar_wait(&sh->bar_o, par, kBudgetNs)) { sh->abort = 1; record_fail(5); }
    tc::tc_fence_after_sync();
    if (tid == 0 && j + 1 < nblocks) load_v(j + 1);  // V tile is free again
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(tO + lane_addr + c * 32, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(r[i]);
    }
    tc::tc_fence_before_sync();
  }

  // ---- epilogue ----
  if (!sh->abort) {
    const float inv = 1.0f / l_run;
    __nv_bfloat16* dst = p.out + (size_t)(row0 + tid) * H + q_col;
#pragma unroll
    for (int c8 = 0; c8 < HD / 8; ++c8) {
      uint4 v;
      v.x = pack_bf16(o[c8 * 8 + 0] * inv, o[c8 * 8 + 1] * inv);
      v.y = pack_bf16(o[c8 * 8 + 2] * inv, o[c8 * 8 + 3] * inv);
      v.z = pack_bf16(o[c8 * 8 + 4] * inv, o[c8 * 8 + 5] * inv);
      v.w = pack_bf16(o[c8 * 8 + 6] * inv, o[c8 * 8 + 7] * inv);
      reinterpret_cast<uint4*>(dst)[c8] = v;
    }
    p.lse2[((size_t)b * p.heads + h) * p.seq + q_idx] = m_run + log2f(l_run);
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem, Fwd<HD>::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// forward, software-pipelined variant
// ---------------------------------------------------------------------------
// Same tiles and math as attention_fwd_kernel, but the tensor pipe and the softmax no
// longer take turns:
//   * warp 4 is the issuer (one thread drives TMA and tcgen05.mma), warps 0-3 do the softmax
//     (thread t <-> query row t <-> TMEM lane t) and never wait for a copy;
//   * S is double-buffered in TMEM, so S_{j+1} = Q K_{j+1}^T is computed while the softmax of
//     block j runs; K and V are double-buffered in shared memory and fetched two blocks ahead;
//   * O stays in TMEM and P V accumulates into it (no per-block read-back); a warp rescales
//     its 32 rows of O (tcgen05.ld / st) only in blocks where one of them raised its running
//     maximum, which after the first few blocks of a row is rare.
// Order on the tensor pipe: QK_0, QK_1, PV_0, QK_2, PV_1, QK_3, ...
// mbarriers: bar_k[b] / bar_v[b] copy of block j landed (b = j & 1, phase j >> 1);
// bar_s[b] S_j ready; bar_p (128 arrivals) P_j written, S_j consumed, O rescaled;
// bar_o PV_j done (phase j).  No barrier can complete twice between two waits of the same
// waiter: QK_{j+2} and PV_j are issued only after bar_p of block j.
constexpr int kPipeThreads = 160;

struct PipeShared {
  uint64_t bar_q, bar_k[2], bar_v[2], bar_s[2], bar_p, bar_o;
  uint32_t tmem_base;
  volatile int abort;
};

template <int HD> struct FwdPipe {
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int K_BYTES = BKF * HD * 2;
  static constexpr int DATA = Q_BYTES + 4 * K_BYTES + FWD_P_BYTES;  // 112 KiB at head_dim 128
  // no slack for manual alignment (two CTAs of 112 KiB + 1 KiB reserved each just fit one
  // SM): the kernel checks that the dynamic window is 1024-byte aligned and gives up if not
  static constexpr int SMEM = DATA + 128;
  static constexpr int TMEM_COLS = 256;  // S0 (64) + S1 (64) + O (HD)
};

// 2^x as one MUFU instruction (arguments here are <= 0; tiny results flush to zero)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// every lane waits; the verdict is made uniform so that the warp stays converged for the
// warp-collective tcgen05.ld / st that follow
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity) {
  const bool ok = tc::mbar_wait(bar, parity, kBudgetNs);
  return __all_sync(0xffffffffu, ok);
}

template <int HD>
__global__ void __launch_bounds__(kPipeThreads, 2)
attention_fwd_pipelined_kernel(const __grid_constant__ CUtensorMap tm_q,    // box {64, 128}
                               const __grid_constant__ CUtensorMap tm_kv,   // box {64, 64}
                               const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int Q_BYTES = FwdPipe<HD>::Q_BYTES, K_BYTES = FwdPipe<HD>::K_BYTES;
  uint8_t* sQ = smem;
  uint8_t* sK0 = sQ + Q_BYTES;
  uint8_t* sV0 = sK0 + 2 * K_BYTES;
  uint8_t* sP = sV0 + 2 * K_BYTES;
  PipeShared* sh = reinterpret_cast<PipeShared*>(sP + FWD_P_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((tc::smem_u32(smem) & 1023u) != 0u) {  // same answer in every thread of the CTA
    if (tid == 0) record_fail(20);
    return;
  }
  const int qblocks = p.seq / BQ;
  const int qb = qblocks - 1 - (int)(blockIdx.x % qblocks);  // heavy query blocks first
  const int bh = blockIdx.x / qblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int H = p.heads * HD;
  const int row0 = b * p.seq + qb * BQ;
  const int q_col = h * HD, k_col = H + h * HD, v_col = 2 * H + h * HD;
  const int n = (qb * BQ + BQ) / BKF;  // causal: keys 0 .. q0 + 127

  if (tid == 0) {
    tc::mbar_init(&sh->bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sh->bar_k[i], 1);
      tc::mbar_init(&sh->bar_v[i], 1);
      tc::mbar_init(&sh->bar_s[i], 1);
    }
    tc::mbar_init(&sh->bar_p, 128);
    tc::mbar_init(&sh->bar_o, 1);
    sh->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == 4) tc::tmem_alloc(&sh->tmem_base, FwdPipe<HD>::TMEM_COLS);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;
  const uint32_t tO = tmem + 128;

  if (warp == 4) {
    // ------------------------------- issuer -------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::make_idesc_bf16(BQ, BKF, false, false);
      constexpr uint32_t idesc_o = tc::make_idesc_bf16(BQ, HD, false, true);
      const uint32_t aQ = tc::smem_u32(sQ), aK0 = tc::smem_u32(sK0), aV0 = tc::smem_u32(sV0),
                     aP = tc::smem_u32(sP);
      bool ok = true;
      auto wait = [&](uint64_t* bar, uint32_t parity, unsigned code) {
        if (ok && !tc::mbar_wait(bar, parity, kBudgetNs)) {
          ok = false;
          sh->abort = 1;
          record_fail(code);
        }
      };
      auto load_k = [&](int j) {
        uint64_t* bar = &sh->bar_k[j & 1];
        tc::mbar_expect_tx(bar, K_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tc::tma_load_2d(sK0 + (j & 1) * K_BYTES + c * BKF * 128, &tm_kv, bar, k_col + 64 * c,
                          b * p.seq + j * BKF);
      };
      auto load_v = [&](int j) {
        uint64_t* bar = &sh->bar_v[j & 1];
        tc::mbar_expect_tx(bar, K_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tc::tma_load_2d(sV0 + (j & 1) * K_BYTES + c * BKF * 128, &tm_kv, bar, v_col + 64 * c,
                          b * p.seq + j * BKF);
      };
      auto issue_qk = [&](int j) {
        const uint32_t aK = aK0 + (j & 1) * K_BYTES;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          tc::umma_bf16(tmem + (j & 1) * 64, desc_kmajor(aQ, BQ, ks), desc_kmajor(aK, BKF, ks),
                        idesc_s, ks != 0);
        tc::umma_commit(&sh->bar_s[j & 1]);
      };
      auto issue_pv = [&](int j) {
        const uint32_t aV = aV0 + (j & 1) * K_BYTES;
#pragma unroll
        for (int ks = 0; ks < BKF / 16; ++ks)
          tc::umma_bf16(tO, desc_kmajor(aP, BQ, ks), desc_mnmajor(aV, BKF, ks), idesc_o,
                        (j != 0) || (ks != 0));
        tc::umma_commit(&sh->bar_o);
      };

      tc::mbar_expect_tx(&sh->bar_q, Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c)
        tc::tma_load_2d(sQ + c * BQ * 128, &tm_q, &sh->bar_q, q_col + 64 * c, row0);
      load_k(0);
      load_v(0);
      if (n > 1) {
        load_k(1);
        load_v(1);
      }
      wait(&sh->bar_q, 0, 21);
      wait(&sh->bar_k[0], 0, 22);
      if (ok) {
        tc::tc_fence_after_sync();
        issue_qk(0);
      }
      if (n > 1) {
        wait(&sh->bar_k[1], 0, 22);
        if (ok) {
          tc::tc_fence_after_sync();
          issue_qk(1);
        }
      }
      for (int j = 0; j < n && ok; ++j) {
        const uint32_t par2 = (uint32_t)(j >> 1) & 1u;
        if (j + 2 < n) {  // K buffer j & 1 is free once QK_j has completed
          wait(&sh->bar_s[j & 1], par2, 23);
          if (ok) load_k(j + 2);
        }
        if (j >= 1 && j + 1 < n) {  // V buffer (j + 1) & 1 is free once PV_{j-1} has completed
          wait(&sh->bar_o, (uint32_t)(j - 1) & 1u, 24);
          if (ok) load_v(j + 1);
        }
        wait(&sh->bar_p, (uint32_t)j & 1u, 25);  // P_j written, S_j consumed, O rescaled
        wait(&sh->bar_v[j & 1], par2, 26);
        if (!ok) break;
        tc::tc_fence_after_sync();
        issue_pv(j);
        if (j + 2 < n) {
          wait(&sh->bar_k[j & 1], (uint32_t)((j + 2) >> 1) & 1u, 22);
          if (!ok) break;
          tc::tc_fence_after_sync();
          issue_qk(j + 2);
        }
      }
      // every MMA issued must have finished before TMEM is handed back
      if (ok && n > 0) wait(&sh->bar_o, (uint32_t)(n - 1) & 1u, 27);
    }
    __syncwarp();
  } else {
    // ------------------------------- softmax warps ------------------------------------
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    const int q_idx = qb * BQ + tid;  // position of this thread's query inside the sequence
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (!warp_wait(&sh->bar_s[j & 1], (uint32_t)(j >> 1) & 1u)) {
        ok = false;
        if (lane == 0) { sh->abort = 1; record_fail(28); }
        break;
      }
      tc::tc_fence_after_sync();
      const uint32_t tS = tmem + (j & 1) * 64;
      float s[BKF];  // raw scores (unscaled), then probabilities
      {
        uint32_t r[BKF];
        tc::tmem_ld_32x32(tS + lane_addr, reinterpret_cast<uint32_t(&)[32]>(r[0]));
        tc::tmem_ld_32x32(tS + lane_addr + 32, reinterpret_cast<uint32_t(&)[32]>(r[32]));
        tc::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < BKF; ++i) s[i] = __uint_as_float(r[i]);
      }
      const int k0 = j * BKF;
      if (k0 + BKF - 1 > qb * BQ) {  // block touches the diagonal
#pragma unroll
        for (int i = 0; i < BKF; ++i)
          if (k0 + i > q_idx) s[i] = -INFINITY;
      }
      // the softmax scale is positive, so the maximum can be taken on the raw scores; four
      // independent chains instead of one 64-deep one (this loop is latency bound)
      float mx[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
      for (int i = 4; i < BKF; i += 4) {
#pragma unroll
        for (int q = 0; q < 4; ++q) mx[q] = fmaxf(mx[q], s[i + q]);
      }
      const float m_blk =
          fmaxf(m_run, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2);
      const float alpha = ex2_fast(m_run - m_blk);  // first block: 2^(-inf) = 0
      float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < BKF; i += 4) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          s[i + q] = ex2_fast(fmaf(s[i + q], p.scale_log2, -m_blk));
          sm[q] += s[i + q];
        }
      }
      l_run = l_run * alpha + ((sm[0] + sm[1]) + (sm[2] + sm[3]));
      m_run = m_blk;
      if (j > 0) {
        // PV_{j-1} done: the P buffer may be overwritten and O is at rest
        if (!warp_wait(&sh->bar_o, (uint32_t)(j - 1) & 1u)) {
          ok = false;
          if (lane == 0) { sh->abort = 1; record_fail(29); }
          break;
        }
        tc::tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tc::tmem_ld_32x32(tO + lane_addr + c * 32, r);
            tc::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tc::tmem_st_32x32(tO + lane_addr + c * 32, r);
          }
          tc::tmem_wait_st();
        }
      }
#pragma unroll
      for (int c8 = 0; c8 < BKF / 8; ++c8) {
        uint4 v;
        v.x = pack_bf16(s[c8 * 8 + 0], s[c8 * 8 + 1]);
        v.y = pack_bf16(s[c8 * 8 + 2], s[c8 * 8 + 3]);
        v.z = pack_bf16(s[c8 * 8 + 4], s[c8 * 8 + 5]);
        v.w = pack_bf16(s[c8 * 8 + 6], s[c8 * 8 + 7]);
        *reinterpret_cast<uint4*>(sP + swz(tid, c8)) = v;
      }
      tc::fence_proxy_async();       // generic-proxy smem writes -> visible to the MMA
      tc::tc_fence_before_sync();    // orders the TMEM reads / writes above before the arrival
      tc::mbar_arrive(&sh->bar_p);
      if (__any_sync(0xffffffffu, sh->abort != 0)) {
        ok = false;
        break;
      }
    }
    // ---- epilogue: O / l -> out ----
    if (ok && n > 0 && warp_wait(&sh->bar_o, (uint32_t)(n - 1) & 1u)) {
      tc::tc_fence_after_sync();
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = p.out + (size_t)(row0 + tid) * H + q_col;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tO + lane_addr + c * 32, r);
        tc::tmem_wait_ld();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[u * 8 + 0]) * inv, __uint_as_float(r[u * 8 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[u * 8 + 2]) * inv, __uint_as_float(r[u * 8 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[u * 8 + 4]) * inv, __uint_as_float(r[u * 8 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[u * 8 + 6]) * inv, __uint_as_float(r[u * 8 + 7]) * inv);
          reinterpret_cast<uint4*>(dst + c * 32)[u] = v;
        }
      }
      p.lse2[((size_t)b * p.heads + h) * p.seq + q_idx] = m_run + log2f(l_run);
    } else if (ok && lane == 0) {
      sh->abort = 1;
      record_fail(30);
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem, FwdPipe<HD>::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
struct BwdParams {
  __nv_bfloat16* dqkv;   // [tokens, 3 * heads * HD]; K and V thirds written here
  float* dq_acc;         // [tokens, heads * HD] fp32, zero on entry
  const float* lse2;     // [batch, heads, seq]
  const float* delta;    // [batch, heads, seq]  rowsum(dO o O)
  int batch, seq, heads;
  float scale_log2;      // scale * log2(e)
  float scale;           // softmax scale
};

struct BwdShared {
  uint64_t bar_kv, bar_q, bar_1, bar_2;
  uint32_t tmem_base;
  volatile int abort;
  float lse[BQ];
  float delta[BQ];
};

constexpr int TILE_SQ = 128 * 128 * 2;  // P^T and dS^T: 128 keys x 128 queries, 32 KiB
template <int HD> struct Bwd {
  static constexpr int TILE = 128 * HD * 2;  // K, V, Q, dO: 128 rows x HD (32 KiB at 128)
  static constexpr int SMEM = 4 * TILE + 2 * TILE_SQ + 1024 + sizeof(BwdShared) + 64;
};

// TMA_DQ: how a dQ tile reaches the fp32 accumulator.  false: float4 atomics straight from
// registers.  true: the tile is staged in shared memory (in the P^T / dS^T buffers, which are
// idle at that point; 128-byte swizzled so that the row-per-thread stores do not collide)
// and added to global memory by TMA reductions of [128 rows x 32 floats] boxes, which the L2
// performs at full-line granularity while the next block's MMAs run.
template <int HD, bool TMA_DQ>
__global__ void __launch_bounds__(kBwdThreads, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv,   // box {64, 128} over qkv
                     const __grid_constant__ CUtensorMap tm_do,    // box {64, 128} over dO
                     const __grid_constant__ CUtensorMap tm_dq,    // fp32, box {32, 128} (TMA_DQ)
                     const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int TILE = Bwd<HD>::TILE;
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sPT = sDO + TILE;
  uint8_t* sDS = sPT + TILE_SQ;
  BwdShared* sh = reinterpret_cast<BwdShared*>(sDS + TILE_SQ);

  const int tid = threadIdx.x, warp = tid >> 5;
  // Warps w and w + 4 may read the same 32 TMEM lanes; they split the columns. `row` is the
  // key row (and later the query row of dQ) this thread owns, `half` its column half.
  const int row = ((warp & 3) << 5) | (tid & 31);
  const int half = warp >> 2;
  const int kblocks = p.seq / BKB;
  const int kb = (int)(blockIdx.x % kblocks);  // early key blocks (most work) first
  const int bh = blockIdx.x / kblocks;
  const int h = bh % p.heads, b = bh / p.heads;
  const int H = p.heads * HD;
  const int key0 = b * p.seq + kb * BKB;
  const int q_col = h * HD, k_col = H + h * HD, v_col = 2 * H + h * HD;
  const int nq = kblocks - kb;  // query blocks kb .. kblocks-1 (BQ == BKB)

  if (tid == 0) {
    tc::mbar_init(&sh->bar_kv, 1);
    tc::mbar_init(&sh->bar_q, 1);
    tc::mbar_init(&sh->bar_1, 1);
    tc::mbar_init(&sh->bar_2, 1);
    sh->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&sh->tmem_base, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem = sh->tmem_base;
  // S^T and dP^T: 128 columns each; dV and dK: HD columns each; dQ reuses S^T's columns
  const uint32_t tST = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 256 + HD,
                 tDQ = tmem;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

  auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col, int row) {
#pragma unroll
    for (int c = 0; c < HD / 64; ++c)
      tc::tma_load_2d(dst + c * 128 * 128, map, bar, col + 64 * c, row);
  };
  auto load_q = [&](int qi) {
    const int row = b * p.seq + (kb + qi) * BQ;
    tc::mbar_expect_tx(&sh->bar_q, 2 * TILE);
    load_tile(sQ, &tm_qkv, &sh->bar_q, q_col, row);
    load_tile(sDO, &tm_do, &sh->bar_q, q_col, row);
  };

  if (tid == 0) {
    tc::mbar_expect_tx(&sh->bar_kv, 2 * TILE);
    load_tile(sK, &tm_qkv, &sh->bar_kv, k_col, key0);
    load_tile(sV, &tm_qkv, &sh->bar_kv, v_col, key0);
    load_q(0);
  }

  constexpr uint32_t idesc_kk = tc::make_idesc_bf16(128, 128, false, false);  // both K-major
  constexpr uint32_t idesc_kn = tc::make_idesc_bf16(128, HD, false, true);    // B MN-major
  constexpr uint32_t idesc_nn = tc::make_idesc_bf16(128, HD, true, true);     // both MN-major
  const uint32_t aK = tc::smem_u32(sK), aV = tc::smem_u32(sV), aQ = tc::smem_u32(sQ),
                 aDO = tc::smem_u32(sDO), aPT = tc::smem_u32(sPT), aDS = tc::smem_u32(sDS);
  const int key_idx = kb * BKB + row;  // this thread's key position inside the sequence

  if (!tc::mbar_wait(&sh->bar_kv, 0, kBudgetNs)) { sh->abort = 1; record_fail(11); }

  for (int qi = 0; qi < nq; ++qi) {
    const uint32_t par = (uint32_t)qi & 1u;
    const int qpos0 = (kb + qi) * BQ;  // first query position of this block
    // row statistics of the 128 queries of this block
    {
      const size_t base = ((size_t)b * p.heads + h) * p.seq + qpos0;
      if (tid < BQ) {
        sh->lse[tid] = p.lse2[base + tid];
        sh->delta[tid] = p.delta[base + tid];
      }
    }
    // ---- S^T = K Q^T and dP^T = V dO^T ----
    if (tid == 0) {
      if (!tc::mbar_wait(&sh->bar_q, par, kBudgetNs)) { sh->abort = 1; record_fail(12); }
      tc::tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        tc::umma_bf16(tST, desc_kmajor(aK, 128, ks), desc_kmajor(aQ, 128, ks), idesc_kk, ks != 0);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        tc::umma_bf16(tDP, desc_kmajor(aV, 128, ks), desc_kmajor(aDO, 128, ks), idesc_kk,
                      ks != 0);
      tc::umma_commit(&sh->bar_1);
      // the previous block's dQ reductions must have read their staging tile (the P^T / dS^T
      // buffers) before anybody overwrites it below
      if constexpr (TMA_DQ) tc::bulk_wait_group_read0();
    }
    __syncthreads();  // lse / delta visible; staging tile free
    if (!tc::mbar_wait(&sh->bar_1, par, kBudgetNs)) { sh->abort = 1; record_fail(13); }
    tc::tc_fence_after_sync();

    // ---- P^T and dS^T for this thread's key row, 32 query columns at a time ----
    const bool diagonal = qi == 0;
#pragma unroll 1
    for (int c = half * (BQ / 64); c < (half + 1) * (BQ / 64); ++c) {
      uint32_t rs[32], rd[32];
      tc::tmem_ld_32x32(tST + lane_addr + c * 32, rs);
      tc::tmem_ld_32x32(tDP + lane_addr + c * 32, rd);
      tc::tmem_wait_ld();
      float pt[32], ds[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int qq = c * 32 + i;
        float pv = exp2f(__uint_as_float(rs[i]) * p.scale_log2 - sh->lse[qq]);
        if (diagonal && key_idx > qpos0 + qq) pv = 0.0f;
        pt[i] = pv;
        ds[i] = pv * (__uint_as_float(rd[i]) - sh->delta[qq]) * p.scale;
      }
      const int chunk = c >> 1;            // 64-column chunk of the tile
      const int c8_0 = (c & 1) * 4;        // first 16-byte unit inside the chunk
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v, w;
        v.x = pack_bf16(pt[u * 8 + 0], pt[u * 8 + 1]);
        v.y = pack_bf16(pt[u * 8 + 2], pt[u * 8 + 3]);
        v.z = pack_bf16(pt[u * 8 + 4], pt[u * 8 + 5]);
        v.w = pack_bf16(pt[u * 8 + 6], pt[u * 8 + 7]);
        w.x = pack_bf16(ds[u * 8 + 0], ds[u * 8 + 1]);
        w.y = pack_bf16(ds[u * 8 + 2], ds[u * 8 + 3]);
        w.z = pack_bf16(ds[u * 8 + 4], ds[u * 8 + 5]);
        w.w = pack_bf16(ds[u * 8 + 6], ds[u * 8 + 7]);
        const uint32_t off = chunk * 128 * 128 + swz(row, c8_0 + u);
        *reinterpret_cast<uint4*>(sPT + off) = v;
        *reinterpret_cast<uint4*>(sDS + off) = w;
      }
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    if (sh->abort) break;

    // ---- dV += P^T dO, dK += dS^T Q, dQ = dS K ----
    if (tid == 0) {
      tc::tc_fence_after_sync();
      const uint32_t acc = qi != 0;
#pragma unroll
      for (int ks = 0; ks < BQ / 16; ++ks)
        tc::umma_bf16(tDV, desc_kmajor(aPT, 128, ks), desc_mnmajor(aDO, 128, ks), idesc_kn,
                      acc | (ks != 0));
#pragma unroll
      for (int ks = 0; ks < BQ / 16; ++ks)
        tc::umma_bf16(tDK, desc_kmajor(aDS, 128, ks), desc_mnmajor(aQ, 128, ks), idesc_kn,
                      acc | (ks != 0));
#pragma unroll
      for (int ks = 0; ks < BKB / 16; ++ks)
        tc::umma_bf16(tDQ, desc_mnmajor(aDS, 128, ks), desc_mnmajor(aK, 128, ks), idesc_nn,
                      ks != 0);
      tc::umma_commit(&sh->bar_2);
    }
    if (!tc::mbar_wait(&sh->bar_2, par, kBudgetNs)) { sh->abort = 1; record_fail(14); }
    tc::tc_fence_after_sync();
    if (tid == 0 && qi + 1 < nq) load_q(qi + 1);  // Q and dO tiles are free again

    // ---- dQ rows (thread t <-> query row t) into the fp32 buffer ----
    if constexpr (TMA_DQ) {
      // sub-tile c holds columns [32c, 32c + 32) of the 128 rows: 128 bytes per row, swizzled
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tDQ + lane_addr + c * 32, r);
        tc::tmem_wait_ld();
        uint8_t* tile = sPT + c * (128 * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(tile + swz(row, u)) =
              make_uint4(r[u * 4], r[u * 4 + 1], r[u * 4 + 2], r[u * 4 + 3]);
      }
      tc::fence_proxy_async();  // generic-proxy stores -> visible to the TMA engine
    } else {
      float* dst = p.dq_acc + (size_t)(b * p.seq + qpos0 + row) * H + q_col;
#pragma unroll 1
      for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
        uint32_t r[32];
        tc::tmem_ld_32x32(tDQ + lane_addr + c * 32, r);
        tc::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          atomicAdd(reinterpret_cast<float4*>(dst + c * 32 + i),
                    make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])));
      }
    }
    tc::tc_fence_before_sync();
    __syncthreads();  // everybody has read dQ before the next S^T overwrites its columns
    if constexpr (TMA_DQ) {
      if (tid == 0 && !sh->abort) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c)
          tc::tma_reduce_add_2d(&tm_dq, sPT + c * (128 * 128), q_col + 32 * c,
                                b * p.seq + qpos0);
        tc::bulk_commit_group();
      }
    }
    if (sh->abort) break;
  }
  if constexpr (TMA_DQ) {
    if (tid == 0) tc::bulk_wait_group0();  // the reductions are performed before the CTA exits
  }

  // ---- dK, dV rows (thread t <-> key row t) ----
  if (!sh->abort) {
    tc::tc_fence_after_sync();
    __nv_bfloat16* dk = p.dqkv + (size_t)(key0 + row) * 3 * H + k_col;
    __nv_bfloat16* dv = p.dqkv + (size_t)(key0 + row) * 3 * H + v_col;
#pragma unroll 1
    for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); ++c) {
      uint32_t r[32];
      tc::tmem_ld_32x32(tDK + lane_addr + c * 32, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(r[u * 8 + 0]), __uint_as_float(r[u * 8 + 1]));
        v.y = pack_bf16(__uint_as_float(r[u * 8 + 2]), __uint_as_float(r[u * 8 + 3]));
        v.z = pack_bf16(__uint_as_float(r[u * 8 + 4]), __uint_as_float(r[u * 8 + 5]));
        v.w = pack_bf16(__uint_as_float(r[u * 8 + 6]), __uint_as_float(r[u * 8 + 7]));
        reinterpret_cast<uint4*>(dk + c * 32)[u] = v;
      }
      tc::tmem_ld_32x32(tDV + lane_addr + c * 32, r);
      tc::tmem_wait_ld();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(r[u * 8 + 0]), __uint_as_float(r[u * 8 + 1]));
        v.y = pack_bf16(__uint_as_float(r[u * 8 + 2]), __uint_as_float(r[u * 8 + 3]));
        v.z = pack_bf16(__uint_as_float(r[u * 8 + 4]), __uint_as_float(r[u * 8 + 5]));
        v.w = pack_bf16(__uint_as_float(r[u * 8 + 6]), __uint_as_float(r[u * 8 + 7]));
        reinterpret_cast<uint4*>(dv + c * 32)[u] = v;
      }
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem, 512);
  }
}

// delta[b, h, s] = sum_d dO * O   (one warp per (token, head), HD / 32 elements per lane)
template <int HD>
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                       float* __restrict__ delta, int batch, int seq, int heads) {
  const int lane = threadIdx.x & 31;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long total = (long long)batch * seq * heads;
  if (warp_id >= total) return;
  const int h = (int)(warp_id % heads);
  const long long tok = warp_id / heads;
  constexpr int PAIRS = HD / 64;  // bf16 pairs per lane
  const size_t off = (size_t)tok * heads * HD + (size_t)h * HD + lane * (2 * PAIRS);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(o + off);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(d_o + off);
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(g2[i]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int w = 16; w > 0; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
  if (lane == 0) {
    const int b = (int)(tok / seq), sp = (int)(tok % seq);
    delta[((size_t)b * heads + h) * seq + sp] = s;
  }
}

// dqkv[:, 0:H] = bf16(dq_acc); dq_acc is left zeroed for the next call.  A thread owns one
// float4 column (blockIdx.x, threadIdx.x) and walks the tokens four at a time with all four
// loads issued before the first store: one load in flight per thread, and a 64-bit division per
// element to find its row, made this pass take as long as a quarter of the backward kernel.
__global__ void __launch_bounds__(256)
attention_dq_finish_kernel(float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv,
                           long long tokens, int H) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= H / 4) return;
  const int c = col * 4;
  constexpr int U = 4;
  for (long long t0 = (long long)blockIdx.y * U; t0 < tokens; t0 += (long long)gridDim.y * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (t0 + u < tokens) v[u] = *reinterpret_cast<const float4*>(dq_acc + (t0 + u) * H + c);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (t0 + u < tokens) {
        *reinterpret_cast<float4*>(dq_acc + (t0 + u) * H + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        uint2 o;
        o.x = pack_bf16(v[u].x, v[u].y);
        o.y = pack_bf16(v[u].z, v[u].w);
        *reinterpret_cast<uint2*>(dqkv + (t0 + u) * 3 * H + c) = o;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
// dense 2-D bf16 matrix [rows, cols]
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols,
                    int box_cols, int box_rows) {
  return tc::make_tensor_map_2d(map, ptr, 2, rows, cols, cols, box_cols, box_rows);
}

// fp32 [rows, cols] map with 128-byte swizzle: boxes of 32 floats (one swizzle row) x box_rows
static int make_map_f32(CUtensorMap* map, const void* ptr, long long rows, long long cols,
                        int box_cols, int box_rows) {
  return tc::make_tensor_map_2d(map, ptr, 4, rows, cols, cols, box_cols, box_rows);
}

// ---- launchers, one instantiation per head dim ------------------------------------
template <int HD>
static int launch_fwd(const void* qkv, void* out, void* lse2, int batch, int seq, int heads,
                      float scale, cudaStream_t st) {
  const long long tokens = (long long)batch * seq;
  const int W = 3 * heads * HD;
  CUtensorMap tm_q, tm_kv;
  if (make_map(&tm_q, qkv, tokens, W, 64, BQ)) return 1003;
  if (make_map(&tm_kv, qkv, tokens, W, 64, BKF)) return 1004;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute((const void*)attention_fwd_kernel<HD>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd<HD>::SMEM);
  });
  if (attr_err != cudaSuccess) return 1005;
  FwdParams p;
  p.out = (__nv_bfloat16*)out;
  p.lse2 = (float*)lse2;
  p.batch = batch;
  p.seq = seq;
  p.heads = heads;
  p.scale_log2 = scale * kLog2e;
  const int grid = batch * heads * (seq / BQ);
  attention_fwd_kernel<HD><<<grid, kThreads, Fwd<HD>::SMEM, st>>>(tm_q, tm_kv, p);
  return (int)cudaGetLastError();
}

// 0: float4 atomics, 1: TMA reduce-add from shared memory
static int g_bwd_dq_variant = 1;
// 0: attention_fwd_kernel, 1: attention_fwd_pipelined_kernel
static int g_fwd_variant = 1;

template <int HD>
static int launch_fwd_pipelined(const void* qkv, void* out, void* lse2, int batch, int seq,
                                int heads, float scale, cudaStream_t st) {
  const long long tokens = (long long)batch * seq;
  const int W = 3 * heads * HD;
  CUtensorMap tm_q, tm_kv;
  if (make_map(&tm_q, qkv, tokens, W, 64, BQ)) return 1003;
  if (make_map(&tm_kv, qkv, tokens, W, 64, BKF)) return 1004;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute((const void*)attention_fwd_pipelined_kernel<HD>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    FwdPipe<HD>::SMEM);
    if (attr_err == cudaSuccess)  // two CTAs of 112 KiB need the largest shared-memory carve-out
      attr_err = cudaFuncSetAttribute((const void*)attention_fwd_pipelined_kernel<HD>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared);
  });
  if (attr_err != cudaSuccess) return 1005;
  FwdParams p;
  p.out = (__nv_bfloat16*)out;
  p.lse2 = (float*)lse2;
  p.batch = batch;
  p.seq = seq;
  p.heads = heads;
  p.scale_log2 = scale * kLog2e;
  const int grid = batch * heads * (seq / BQ);
  attention_fwd_pipelined_kernel<HD><<<grid, kPipeThreads, FwdPipe<HD>::SMEM, st>>>(tm_q, tm_kv, p);
  return (int)cudaGetLastError();
}

template <int HD, bool TMA_DQ>
static int launch_bwd_kernel(const CUtensorMap& tm_qkv, const CUtensorMap& tm_do,
                             const CUtensorMap& tm_dq, const BwdParams& p, int grid,
                             cudaStream_t st) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute((const void*)attention_bwd_kernel<HD, TMA_DQ>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd<HD>::SMEM);
  });
  if (attr_err != cudaSuccess) return 1005;
  attention_bwd_kernel<HD, TMA_DQ><<<grid, kBwdThreads, Bwd<HD>::SMEM, st>>>(
      tm_qkv, tm_do, tm_dq, p);
  return 0;
}

template <int HD>
static int launch_bwd(const void* qkv, const void* out, const void* d_out, const void* lse2,
                      void* dqkv, float* dq_acc, float* delta, int batch, int seq, int heads,
                      float scale, cudaStream_t st) {
  const long long tokens = (long long)batch * seq;
  const int H = heads * HD;
  CUtensorMap tm_qkv, tm_do, tm_dq;
  if (make_map(&tm_qkv, qkv, tokens, 3 * H, 64, 128)) return 1003;
  if (make_map(&tm_do, d_out, tokens, H, 64, 128)) return 1004;
  const bool tma_dq = g_bwd_dq_variant >= 1;
  if (tma_dq) {
    if (((uintptr_t)dq_acc & 15) || make_map_f32(&tm_dq, dq_acc, tokens, H, 32, 128)) return 1007;
  } else {
    tm_dq = tm_do;  // unused by the kernel
  }
  {
    const long long warps = tokens * heads;
    const int grid = (int)((warps * 32 + 255) / 256);
    attention_delta_kernel<HD><<<grid, 256, 0, st>>>((const __nv_bfloat16*)out,
                                                     (const __nv_bfloat16*)d_out, delta, batch,
                                                     seq, heads);
  }
  BwdParams p;
  p.dqkv = (__nv_bfloat16*)dqkv;
  p.dq_acc = dq_acc;
  p.lse2 = (const float*)lse2;
  p.delta = delta;
  p.batch = batch;
  p.seq = seq;
  p.heads = heads;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  const int grid = batch * heads * (seq / BKB);
  const int rc = tma_dq ? launch_bwd_kernel<HD, true>(tm_qkv, tm_do, tm_dq, p, grid, st)
                        : launch_bwd_kernel<HD, false>(tm_qkv, tm_do, tm_dq, p, grid, st);
  if (rc) return rc;
  {
    const int col_blocks = (H / 4 + 255) / 256;
    long long rows = (tokens + 3) / 4;
    const long long cap = (148 * 8 + col_blocks - 1) / col_blocks;
    if (rows > cap) rows = cap;
    attention_dq_finish_kernel<<<dim3(col_blocks, (unsigned)rows), 256, 0, st>>>(
        dq_acc, (__nv_bfloat16*)dqkv, tokens, H);
  }
  return (int)cudaGetLastError();
}

static bool shape_ok(int batch, int seq, int heads, int head_dim) {
  return (head_dim == 64 || head_dim == 128) && seq % BQ == 0 && batch > 0 && heads > 0;
}

}  // namespace attn

extern "C" {

// 0: dQ tiles are added to the fp32 accumulator with float4 atomics; 1: with TMA reductions
// from a shared-memory staging tile.  Returns the previous value.
int bcom_attention_set_bwd_dq_variant(int variant) {
  const int old = attn::g_bwd_dq_variant;
  if (variant >= 0 && variant <= 1) attn::g_bwd_dq_variant = variant;
  return old;
}

// qkv: [batch*seq, 3*heads*head_dim] bf16 (q | k | v, RoPE already applied); out: [batch*seq,
// heads*head_dim] bf16; lse2: [batch, heads, seq] fp32.  head_dim is 64 or 128 and seq a
// multiple of 128.
int bcom_attention_fwd(const void* qkv, void* out, void* lse2, int batch, int seq, int heads,
                       int head_dim, float scale, void* stream) {
  using namespace attn;
  if (!shape_ok(batch, seq, heads, head_dim)) return 1001;
  if (((uintptr_t)qkv & 15) || ((uintptr_t)out & 15)) return 1002;
  tc::bind_context_once();
  cudaStream_t st = (cudaStream_t)stream;
  if (g_fwd_variant == 1)
    return head_dim == 128
               ? launch_fwd_pipelined<128>(qkv, out, lse2, batch, seq, heads, scale, st)
               : launch_fwd_pipelined<64>(qkv, out, lse2, batch, seq, heads, scale, st);
  return head_dim == 128 ? launch_fwd<128>(qkv, out, lse2, batch, seq, heads, scale, st)
                         : launch_fwd<64>(qkv, out, lse2, batch, seq, heads, scale, st);
}

// 0 selects the forward kernel whose MMA and softmax take turns, 1 the software-pipelined one
// (issuer warp, double-buffered S in TMEM, O accumulated in TMEM).  Returns the previous value.
int bcom_attention_set_fwd_variant(int variant) {
  const int old = attn::g_fwd_variant;
  if (variant >= 0 && variant <= 1) attn::g_fwd_variant = variant;
  return old;
}

// d_out: [batch*seq, heads*head_dim]; dqkv (written): [batch*seq, 3*heads*head_dim];
// dq_acc: fp32 [batch*seq, heads*head_dim] scratch, must be zero on entry and is zero on exit;
// delta: fp32 [batch, heads, seq] scratch.
int bcom_attention_bwd(const void* qkv, const void* out, const void* d_out, const void* lse2,
                       void* dqkv, void* dq_acc, void* delta, int batch, int seq, int heads,
                       int head_dim, float scale, void* stream) {
  using namespace attn;
  if (!shape_ok(batch, seq, heads, head_dim)) return 1001;
  if (((uintptr_t)qkv & 15) || ((uintptr_t)d_out & 15) || ((uintptr_t)dqkv & 15)) return 1002;
  tc::bind_context_once();
  cudaStream_t st = (cudaStream_t)stream;
  return head_dim == 128
             ? launch_bwd<128>(qkv, out, d_out, lse2, dqkv, (float*)dq_acc, (float*)delta, batch,
                               seq, heads, scale, st)
             : launch_bwd<64>(qkv, out, d_out, lse2, dqkv, (float*)dq_acc, (float*)delta, batch,
                              seq, heads, scale, st);
}

int bcom_attention_status(unsigned int out[4], int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, attn::g_status, sizeof(unsigned int) * 4);
  if (err == cudaSuccess && clear) {
    unsigned int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(attn::g_status, zero, sizeof(zero));
  }
  return (int)err;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared in no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"

namespace attn {

// Scratch that ships inside the library image: [ dQ accumulator | row statistics ].
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[BCOM_NO_ALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices];
static std::mutex g_scratch_mu;

// Device address of the scratch array on the current device; looked up once per device.
static cudaError_t no_alloc_scratch_ptr(unsigned char** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
    if (err != cudaSuccess) return err;
    g_scratch_addr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return cudaSuccess;
}

}  // namespace attn

extern "C" {

unsigned long long bcom_no_alloc_scratch_bytes(void) { return BCOM_NO_ALLOC_SCRATCH_BYTES; }

int bcom_attention_bwd_no_alloc(const void* qkv, const void* out, const void* d_out,
                                const void* lse2, void* dqkv, int batch, int seq, int heads,
                                int head_dim, float scale, void* stream) {
  using namespace attn;
  if (head_dim != 128 || seq % BQ || batch <= 0 || heads <= 0) return 1001;
  if (((uintptr_t)qkv & 15) || ((uintptr_t)d_out & 15) || ((uintptr_t)dqkv & 15)) return 1002;
  const long long tokens = (long long)batch * seq;
  const int H = heads * 128;
  const unsigned long long dq_bytes = 4ull * (unsigned long long)tokens * (unsigned long long)H;
  const unsigned long long delta_bytes =
      (4ull * (unsigned long long)tokens * (unsigned long long)heads + 255ull) & ~255ull;
  if (dq_bytes + delta_bytes > BCOM_NO_ALLOC_SCRATCH_BYTES) {
    fprintf(stderr,
            "bitscom_b200: bcom_attention_bwd_no_alloc needs %llu bytes of scratch for "
            "batch=%d seq=%d heads=%d but the built-in array holds %u; use "
            "bcom_attention_bwd with caller-provided buffers\n",
            dq_bytes + delta_bytes, batch, seq, heads, BCOM_NO_ALLOC_SCRATCH_BYTES);
    return 1006;
  }
  unsigned char* scratch = nullptr;
  cudaError_t err = no_alloc_scratch_ptr(&scratch);  // also binds this thread's context
  if (err != cudaSuccess) return (int)err;
  (void)cudaGetLastError();
  cudaStream_t st = (cudaStream_t)stream;
  float* dq_acc = reinterpret_cast<float*>(scratch);
  float* delta = reinterpret_cast<float*>(scratch + dq_bytes);
  // the accumulator must start at zero; the array still holds the previous call's data
  err = cudaMemsetAsync(dq_acc, 0, dq_bytes, st);
  if (err != cudaSuccess) return (int)err;
  return launch_bwd<128>(qkv, out, d_out, lse2, dqkv, dq_acc, delta, batch, seq, heads, scale,
                         st);
}

}  // extern "C"
