// bf16 GEMM on the 5th-generation tensor cores (sm_100a): C[M,N] (+)= A x B with fp32
// accumulation in tensor memory.
//
//   * persistent grid, one CTA per SM, static round-robin over 128x256 output tiles
//     (grouped along M so that concurrently running CTAs share B tiles in L2);
//   * warp 0: TMA producer (cp.async.bulk.tensor 2-D tiles, 128-byte swizzle) into a
//     4-stage shared-memory ring (48 KiB per stage);
//   * warp 1: allocates 512 TMEM columns and issues tcgen05.mma (cta_group::1,
//     M=128, N=256, K=16 per instruction) from one elected thread; tcgen05.commit
//     releases ring stages and publishes finished accumulators;
//   * warps 2-5: epilogue. Two 256-column accumulators alternate, so the epilogue of
//     tile i (tcgen05.ld -> registers -> global) overlaps the main loop of tile i+1.
//
// Operand layouts.  Either operand may be K-major (reduction dimension contiguous) or
// MN-major (the other dimension contiguous); this covers forward (x W^T), data
// gradient (dy W) and weight gradient (dy^T x) of a linear layer without transposes:
//
//   K-major  X[rows=MN, cols=K]  one TMA box {64 k, BM|BN rows}; descriptor SBO = 1024
//   MN-major X[rows=K, cols=MN]  boxes {64 mn, 64 k} side by side, 8 KiB each;
//                                descriptor LBO = 8192 (next 64-wide MN chunk), SBO = 1024
//
// Every mbarrier wait is bounded; on expiry the kernel records a code, all roles drain,
// TMEM is released and the kernel returns.  torch.matmul / cuBLAS is the library
// baseline this replaces for the trainer's linear layers (the reference trainer's model
// code is plain nn.Linear, benchmarks/train_llama7b_dp_pp_lowbit.py:222-238).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "gemm_epilogue.cuh"
#include "gemm_schedule.cuh"
#include "tc_common.cuh"

namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one MN-major box: 64 mn x 64 k
constexpr int kThreads = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256;

enum Status : unsigned int {
  kOk = 0, kProducerTimeout = 1, kMmaTimeout = 2, kEpilogueTimeout = 3, kAccumTimeout = 4
};

__device__ unsigned int g_status[4];

struct Params {
  void* C;
  const void* R;  // optional bf16 residual added in the bf16 epilogue (see gemm_epilogue.cuh)
  long long ldc, ldr;
  int M, N, K;
  int tiles_m, tiles_n;
};

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

__device__ __forceinline__ void fail(Shared* sh, unsigned int code) {
  sh->abort = 1;
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = threadIdx.x;
  }
}

// One unit of work of a CTA: rows [m0, m0 + BM), columns [n0, n0 + BN) of C.
using gemm_sched::WorkItem;
__device__ __forceinline__ WorkItem work_item(const Params& p, int w) {
  return gemm_sched::work_item<BM, BN, GROUP_M>(p.tiles_m, p.tiles_n, w);
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&sh->acc_full[b], 1);
      tc::mbar_init(&sh->acc_empty[b], 4);
    }
    sh->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == 1) tc::tmem_alloc(&sh->tmem_base, TMEM_COLS);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < total_tiles && !sh->abort; t += gridDim.x) {
        const WorkItem wi = work_item(p, t);
        const int m0 = wi.m0, n0 = wi.n0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1u, kWaitBudgetNs)) {
            fail(sh, kProducerTimeout);
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          tc::mbar_expect_tx(&sh->full[stage], STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tc::tma_load_2d(sA + c * CHUNK_BYTES, &tmA, &sh->full[stage], m0 + c * 64, k0);
          } else {
            tc::tma_load_2d(sA, &tmA, &sh->full[stage], k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tc::tma_load_2d(sB + c * CHUNK_BYTES, &tmB, &sh->full[stage], n0 + c * 64, k0);
          } else {
            tc::tma_load_2d(sB, &tmB, &sh->full[stage], k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = tc::make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      for (int t = blockIdx.x; t < total_tiles && !sh->abort; t += gridDim.x, ++iter) {
        const int buf = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        if (!tc::mbar_wait(&sh->acc_empty[buf], acc_phase ^ 1u, kWaitBudgetNs)) {
          fail(sh, kAccumTimeout);
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&sh->full[stage], phase, kWaitBudgetNs)) {
            fail(sh, kMmaTimeout);
            ok = false;
            break;
          }
          tc::tc_fence_after_sync();
          const uint32_t a_addr = tc::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN
                ? tc::make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                : tc::make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN
                ? tc::make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), CHUNK_BYTES, 1024)
                : tc::make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc::umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc::umma_commit(&sh->empty[stage]);  // stage reusable once these MMAs are done
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc::umma_commit(&sh->acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue -----------------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter ..
    int iter = 0;
    for (int t = blockIdx.x; t < total_tiles && !sh->abort; t += gridDim.x, ++iter) {
      const WorkItem wi = work_item(p, t);
      const int buf = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      if (!tc::mbar_wait(&sh->acc_full[buf], acc_phase, kWaitBudgetNs)) {
        if (lane == 0) fail(sh, kEpilogueTimeout);
        break;
      }
      tc::tc_fence_after_sync();
      const int row = wi.m0 + quarter * 32 + lane;
      const int n0 = wi.n0;
      const uint32_t taddr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(quarter * 32) << 16);
      store_accumulator_rows<BN, OUT_F32, ACCUM>(taddr, p.C, p.ldc, row, n0, p.M, p.N, p.R,
                                                 p.ldr);
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&sh->acc_empty[buf]);
    }
  }

  // ------------------------------ teardown -------------------------------------
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// 2-D bf16 row-major matrix [rows, cols] with leading dimension ld (elements).
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols,
                    long long ld, int box_cols, int box_rows) {
  return tc::cached_tensor_map_2d(map, ptr, 2, rows, cols, ld, box_cols, box_rows);
}

typedef void (*Kernel)(const CUtensorMap, const CUtensorMap, const Params);

template <bool A_MN, bool B_MN>
static Kernel pick_out(bool out_f32, bool accum) {
  if (out_f32) return accum ? gemm_bf16_kernel<A_MN, B_MN, true, true>
                            : gemm_bf16_kernel<A_MN, B_MN, true, false>;
  return accum ? gemm_bf16_kernel<A_MN, B_MN, false, true>
               : gemm_bf16_kernel<A_MN, B_MN, false, false>;
}

static Kernel pick(bool a_mn, bool b_mn, bool out_f32, bool accum) {
  if (a_mn) return b_mn ? pick_out<true, true>(out_f32, accum)
                        : pick_out<true, false>(out_f32, accum);
  return b_mn ? pick_out<false, true>(out_f32, accum) : pick_out<false, false>(out_f32, accum);
}

}  // namespace gemm

extern "C" {

// C[M,N] (+)= op(A) x op(B), bf16 operands, fp32 accumulation.
//   a_mn_major = 0: A is [M, K] row-major (lda >= K); 1: A is stored [K, M] (lda >= M)
//   b_mn_major = 0: B is [N, K] row-major (ldb >= K); 1: B is stored [K, N] (ldb >= N)
//   out_fp32: C is fp32 instead of bf16; accumulate: add to the existing C
// Leading dimensions are in elements and must keep rows 16-byte aligned.
//   residual (optional, bf16 [M, N], leading dimension ldr): C = residual + A x B; only with a
//   bf16, non-accumulating C
int bcom_gemm_bf16_ex(const void* A, const void* B, void* C, const void* residual, int M, int N,
                      int K, long long lda, long long ldb, long long ldc, long long ldr,
                      int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int max_ctas,
                      void* stream) {
  using namespace gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // argument errors get codes of their own (1001..1005) so that they cannot be mistaken
  // for a CUDA error
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8)) || (N % 8)) return 1001;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15)) return 1002;
  if (residual && (out_fp32 || accumulate || (ldr % 8) || ((uintptr_t)residual & 15))) return 1001;
  (void)cudaGetLastError();  // do not inherit an error left behind by an earlier call
  CUtensorMap tmA, tmB;
  // the tensor-map encoder is a driver call: make sure this thread (it may be an autograd
  // worker) has the device's primary context bound
  tc::bind_context_once();
  Params p;
  p.C = C;
  p.R = residual;
  p.ldc = ldc;
  p.ldr = ldr;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles;
  if (grid > sms) grid = sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (a_mn_major ? make_map(&tmA, A, K, M, lda, 64, BK) : make_map(&tmA, A, M, K, lda, BK, BM))
    return 1003;
  if (b_mn_major ? make_map(&tmB, B, K, N, ldb, 64, BK)
                 : make_map(&tmB, B, N, K, ldb, BK, BN))
    return 1004;
  Kernel kernel = pick(a_mn_major != 0, b_mn_major != 0, out_fp32 != 0, accumulate != 0);
  if (!tc::ensure_dynamic_smem((const void*)kernel, SMEM_BYTES)) return 1005;
  kernel<<<grid, kThreads, SMEM_BYTES, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

int bcom_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                   long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_fp32,
                   int accumulate, int max_ctas, void* stream) {
  return bcom_gemm_bf16_ex(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, a_mn_major, b_mn_major,
                           out_fp32, accumulate, max_ctas, stream);
}

// Copies the 4-word status record {code, cta, thread, -}; clears it when `clear` != 0.
int bcom_gemm_status(unsigned int out[4], int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, gemm::g_status, sizeof(unsigned int) * 4);
  if (err == cudaSuccess && clear) {
    unsigned int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(gemm::g_status, zero, sizeof(zero));
  }
  return (int)err;
}

}  // extern "C"
