// bf16 GEMM on CTA pairs (sm_100a, tcgen05 cta_group::2): C[M,N] (+)= A x B with fp32
// accumulation in tensor memory.  Same interface and operand layouts as gemm_tcgen05.cu; what
// changes is the tile a tensor-core instruction works on:
//
//   * clusters of two CTAs on neighbouring SMs compute one 256x256 output tile.  CTA r of the
//     pair stages rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the
//     B tile (that is, columns of C) in its own shared memory: 32 KiB per pipeline stage
//     against 48 KiB for the same work per SM in the one-CTA kernel, so the ring is 6 stages
//     deep and every B element is read from L2 once per pair instead of once per CTA;
//   * one thread of the even CTA (the leader) issues tcgen05.mma.cta_group::2 with M = 256,
//     N = 256, K = 16: the tensor cores of both SMs run it, each on its own 128 rows of A and
//     on both halves of B, and each accumulates its 128 x 256 slice in its own tensor memory;
//   * two tcgen05.commit per event, one on each CTA's barrier (the peer's is addressed through
//     mapa), release a ring stage and publish a finished accumulator in both CTAs;
//   * TMA loads are per-CTA loads in the cta_group::2 form: each CTA loads its own half of the
//     operands into its own shared memory, and both halves complete on the LEADER's "stage
//     full" barrier (the leader expects the bytes of both), so the MMA issuer waits on one
//     barrier per stage; the epilogue warps of the odd CTA hand their accumulator buffer back
//     with a remote mbarrier arrive.  Every load is an ordinary load of one CTA.
//
// Every wait is bounded; on expiry the kernel records a code, all roles of both CTAs drain
// (each through its own bounded waits), tensor memory is released and the kernel returns.
// This is the CTA-pair variant of the library GEMM that torch.matmul / cuBLAS provides to the
// reference trainer's nn.Linear layers (benchmarks/train_llama7b_dp_pp_lowbit.py:222-238).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "gemm_epilogue.cuh"
#include "gemm_schedule.cuh"
#include "tc_common.cuh"

namespace gemm2 {

constexpr int BM = 256;      // rows of C per CTA pair
constexpr int BN = 256;      // columns of C per CTA pair (and per CTA: each holds all columns)
constexpr int BM_CTA = 128;  // rows of A staged (and of C produced) by one CTA
constexpr int BN_CTA = 128;  // rows of B staged by one CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM_CTA * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN_CTA * BK * 2;  // 16 KiB
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
// Optional per-pair cycle counters of the MMA issuer {waiting for operands, waiting for a free
// accumulator, whole loop, k-blocks}: written when a buffer has been registered
// (bcom_gemm2_set_profile), for finding out which hand-off a slow shape is waiting on.
__device__ unsigned long long* g_profile;

struct Params {
  void* C;
  const void* R;  // optional bf16 residual added in the bf16 epilogue
  long long ldc, ldr;
  int M, N, K;
  int tiles_m, tiles_n;
};

// Identical layout, at identical shared-memory offsets, in both CTAs of a pair: the MMA and the
// commit address the peer's operands and barriers by the leader's offsets.
struct Shared {
  uint64_t full[STAGES];       // leader only: both CTAs' TMA loads of the stage have landed
  uint64_t empty[STAGES];      // the pair's MMAs have read the stage (one commit per CTA)
  uint64_t acc_full[2];        // accumulator buffer complete (one commit per CTA)
  uint64_t acc_empty[2];       // leader only: all 8 epilogue warps of the pair drained it
  uint32_t tmem_base;
  volatile int abort;
};

// ---------------------------------------------------------------------------
// cluster / cta_group::2 primitives
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(tc::smem_u32(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// bounded wait on a local barrier whose arrivals come from the other CTA
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(tc::smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity,
                                                  unsigned long long budget_ns) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = tc::globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 255u) == 0u && tc::globaltimer_ns() - t0 > budget_ns) return false;
  }
  return true;
}

// One warp of EACH CTA of the pair executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_out, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   tc::smem_u32(smem_out)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
               : "memory");
}

// D[tmem of both CTAs] (+)= A[smem of both] * B[smem of both]; issued by ONE thread of the leader.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The barrier at shared::cluster address `bar` (this CTA's or the peer's) receives one arrival
// once all tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_to(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// Both CTAs of the pair: the barrier at this offset here, and the one at the same offset in the
// peer (`peer_bar` = map_to_cta(bar, 1)).
__device__ __forceinline__ void umma_commit_both(uint64_t* bar, uint32_t peer_bar) {
  umma_commit_to(tc::smem_u32(bar));
  umma_commit_to(peer_bar);
}
// 2-D tiled load of the CTA-pair form: the data lands in THIS CTA's shared memory, the bytes
// are counted on the barrier at shared::cluster address `bar`, which may be the peer's.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(tc::smem_u32(smem_dst)), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void fail(Shared* sh, unsigned int code) {
  sh->abort = 1;
  if (atomicCAS(&g_status[0], 0u, code) == 0u) {
    g_status[1] = blockIdx.x;
    g_status[2] = threadIdx.x;
  }
}

__device__ __forceinline__ void tile_coords(const Params& p, int t, int* tm, int* tn) {
  gemm_sched::tile_coords<GROUP_M>(p.tiles_m, p.tiles_n, t, tm, tn);
}

template <bool A_MN, bool B_MN, bool OUT_F32, bool ACCUM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared* sh = reinterpret_cast<Shared*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader, 1: its peer
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + BK - 1) / BK;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(&sh->full[s], 1);
      tc::mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&sh->acc_full[b], 1);
      tc::mbar_init(&sh->acc_empty[b], 8);
    }
    sh->abort = 0;
    tc::fence_mbar_init();
  }
  if (warp == 1) tmem_alloc_pair(&sh->tmem_base, TMEM_COLS);
  tc::tc_fence_before_sync();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals the other CTA
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) -------------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < total_tiles && !sh->abort; t += num_pairs) {
        int tm, tn;
        tile_coords(p, t, &tm, &tn);
        const int m0 = tm * BM + (int)rank * BM_CTA;  // this CTA's rows of A (and of C)
        const int n0 = tn * BN + (int)rank * BN_CTA;  // this CTA's rows of B
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1u, kWaitBudgetNs)) {
            fail(sh, kProducerTimeout);
            break;
          }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          // the leader's barrier counts the bytes of both CTAs; the odd CTA's bytes may land
          // before this expect (the count goes negative for a moment), which is fine: the
          // phase cannot complete before the leader's own arrival below
          if (leader) tc::mbar_expect_tx(&sh->full[stage], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(&sh->full[stage], 0);
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int c = 0; c < BM_CTA / 64; ++c)
              tma_load_2d_pair(sA + c * CHUNK_BYTES, &tmA, bar, m0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sA, &tmA, bar, k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int c = 0; c < BN_CTA / 64; ++c)
              tma_load_2d_pair(sB + c * CHUNK_BYTES, &tmB, bar, n0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sB, &tmB, bar, k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      // Producer tail: the stage-release arrivals come from the leader's commits and land in
      // this CTA's shared memory asynchronously; wait until the last fill of every stage has
      // been released, so that none of them can arrive after this CTA has left.
      for (int i = 0; i < STAGES && !sh->abort; ++i) {
        if (!tc::mbar_wait(&sh->empty[stage], phase ^ 1u, kWaitBudgetNs)) {
          fail(sh, kProducerTimeout);
          break;
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------ MMA issuer (leader) ----------------------
      constexpr uint32_t idesc = tc::make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      unsigned long long* const prof = g_profile;
      long long t_full = 0, t_acc = 0, n_kb = 0;
      const long long t_begin = prof ? clock64() : 0;
      for (int t = pair; t < total_tiles && !sh->abort; t += num_pairs, ++iter) {
        const int buf = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        long long c0 = prof ? clock64() : 0;
        if (!mbar_wait_cluster(&sh->acc_empty[buf], acc_phase ^ 1u, kWaitBudgetNs)) {
          fail(sh, kAccumTimeout);
          break;
        }
        if (prof) t_acc += clock64() - c0;
        tc::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (prof) c0 = clock64();
          // the odd CTA's bytes arrive from the other SM: cluster-scope acquire
          if (!mbar_wait_cluster(&sh->full[stage], phase, kWaitBudgetNs)) {
            fail(sh, kMmaTimeout);
            ok = false;
            break;
          }
          if (prof) { t_full += clock64() - c0; ++n_kb; }
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
            umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // both CTAs may refill the stage
          umma_commit_both(&sh->empty[stage], map_to_cta(&sh->empty[stage], 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_both(&sh->acc_full[buf], map_to_cta(&sh->acc_full[buf], 1));
      }
      if (prof) {
        prof[4 * pair + 0] = (unsigned long long)t_full;
        prof[4 * pair + 1] = (unsigned long long)t_acc;
        prof[4 * pair + 2] = (unsigned long long)(clock64() - t_begin);
        prof[4 * pair + 3] = (unsigned long long)n_kb;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) -------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter ..
    int iter = 0;
    for (int t = pair; t < total_tiles && !sh->abort; t += num_pairs, ++iter) {
      int tm, tn;
      tile_coords(p, t, &tm, &tn);
      const int buf = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      if (!tc::mbar_wait(&sh->acc_full[buf], acc_phase, kWaitBudgetNs)) {
        if (lane == 0) fail(sh, kEpilogueTimeout);
        break;
      }
      tc::tc_fence_after_sync();
      const int row = tm * BM + (int)rank * BM_CTA + quarter * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(quarter * 32) << 16);
      gemm::store_accumulator_rows<BN, OUT_F32, ACCUM>(taddr, p.C, p.ldc, row, n0, p.M, p.N, p.R,
                                                       p.ldr);
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (leader) tc::mbar_arrive(&sh->acc_empty[buf]);
        else mbar_arrive_cluster(map_to_cta(&sh->acc_empty[buf], 0));
      }
    }
  }

  // ------------------------------ teardown -------------------------------------
  // Nobody leaves, and no tensor memory is released, while the other CTA may still signal this
  // CTA's barriers or the leader's MMAs may still read this CTA's operands.
  tc::tc_fence_before_sync();
  __syncwarp();
  cluster_sync_all();
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
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
  if (out_f32) return accum ? gemm_bf16_pair_kernel<A_MN, B_MN, true, true>
                            : gemm_bf16_pair_kernel<A_MN, B_MN, true, false>;
  return accum ? gemm_bf16_pair_kernel<A_MN, B_MN, false, true>
               : gemm_bf16_pair_kernel<A_MN, B_MN, false, false>;
}

static Kernel pick(bool a_mn, bool b_mn, bool out_f32, bool accum) {
  if (a_mn) return b_mn ? pick_out<true, true>(out_f32, accum) : pick_out<true, false>(out_f32, accum);
  return b_mn ? pick_out<false, true>(out_f32, accum) : pick_out<false, false>(out_f32, accum);
}


// CTA pairs that can be resident at once (pairs live inside one GPC, so this can be fewer than
// half the SM count); asked once per kernel.
static int resident_pairs(const void* kernel) {
  struct Seen {
    const void* kernel;
    int pairs;
  };
  static std::mutex mu;
  static Seen seen[64];
  static int count = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < count; ++i)
    if (seen[i].kernel == kernel) return seen[i].pairs;
  int pairs = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  if (cudaOccupancyMaxActiveClusters(&pairs, kernel, &cfg) != cudaSuccess || pairs <= 0) {
    (void)cudaGetLastError();
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    pairs = sms / 2;
  }
  if (count < 64) seen[count++] = Seen{kernel, pairs};
  return pairs;
}

}  // namespace gemm2

extern "C" {


// Same contract as bcom_gemm_bf16 (gemm_tcgen05.cu); max_ctas counts CTAs (two per pair).
int bcom_gemm2_bf16_ex(const void* A, const void* B, void* C, const void* residual, int M, int N,
                       int K, long long lda, long long ldb, long long ldc, long long ldr,
                       int a_mn_major, int b_mn_major, int out_fp32, int accumulate,
                       int max_ctas, void* stream) {
  using namespace gemm2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8)) || (N % 8)) return 1001;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15)) return 1002;
  if (residual && (out_fp32 || accumulate || (ldr % 8) || ((uintptr_t)residual & 15))) return 1001;
  (void)cudaGetLastError();
  CUtensorMap tmA, tmB;
  tc::bind_context_once();
  if (a_mn_major ? make_map(&tmA, A, K, M, lda, 64, BK) : make_map(&tmA, A, M, K, lda, BK, BM_CTA))
    return 1003;
  if (b_mn_major ? make_map(&tmB, B, K, N, ldb, 64, BK) : make_map(&tmB, B, N, K, ldb, BK, BN_CTA))
    return 1004;
  Kernel kernel = pick(a_mn_major != 0, b_mn_major != 0, out_fp32 != 0, accumulate != 0);
  if (!tc::ensure_dynamic_smem((const void*)kernel, SMEM_BYTES)) return 1005;
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
  // persistent grid: as many pairs as can be resident at once (pairs live inside one GPC, so
  // this can be fewer than half the SM count), never more than there are tiles
  int pairs = resident_pairs((const void*)kernel);
  const int tiles = p.tiles_m * p.tiles_n;
  if (pairs > tiles) pairs = tiles;
  if (max_ctas >= 2 && pairs > max_ctas / 2) pairs = max_ctas / 2;
  if (pairs < 1) pairs = 1;
  kernel<<<2 * pairs, kThreads, SMEM_BYTES, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

int bcom_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn_major, int b_mn_major, int out_fp32,
                    int accumulate, int max_ctas, void* stream) {
  return bcom_gemm2_bf16_ex(A, B, C, nullptr, M, N, K, lda, ldb, ldc, 0, a_mn_major, b_mn_major,
                            out_fp32, accumulate, max_ctas, stream);
}

// Debugging aid: registers a device buffer of 4 x (number of CTA pairs) 64-bit words that the
// MMA issuer of every pair fills with {cycles waiting for operands, cycles waiting for a free
// accumulator, cycles in its loop, k-blocks issued}; NULL switches it off (the default).
int bcom_gemm2_set_profile(void* device_buffer) {
  unsigned long long* p = (unsigned long long*)device_buffer;
  return (int)cudaMemcpyToSymbol(gemm2::g_profile, &p, sizeof(p));
}

// Copies the 4-word status record {code, cta, thread, -}; clears it when `clear` != 0.
int bcom_gemm2_status(unsigned int out[4], int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, gemm2::g_status, sizeof(unsigned int) * 4);
  if (err == cudaSuccess && clear) {
    unsigned int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(gemm2::g_status, zero, sizeof(zero));
  }
  return (int)err;
}

}  // extern "C"
