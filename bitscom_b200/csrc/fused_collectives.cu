// Fused low-bit collectives for one NVSwitch domain (sm_100a): ONE kernel per bucket
// chunk does what the reference spreads over ~20 ATen kernels per shard, four NCCL
// send/recv groups and three host-synchronised phases
// (cpp/src/process_group_lowbit.cc:641-861 phase 1, :1106-1251 phase 2, :1253-1293
// restore; Python twin python/bitscom/api.py:703-875):
//
//   phase 1  [error-feedback add] -> block absmax -> fp16 scale -> nearest/stochastic
//            rounding -> bit-pack -> store the packed shard j and its scales straight
//            into rank j's receive slot over NVLink (peer stores); new residual
//   flag 1   last CTA of the rank publishes epoch to every peer (st.release.sys)
//   phase 2  wait for all sources; dequantize the W streams from LOCAL memory, fp32 sum
//            in ascending source order; [stage-2 residual add]; re-quantize; push the
//            packed reduced shard into every rank's gather slot
//   flag 2   publish; wait for all owners
//   phase 3  unpack + dequantize all W shards from local gather slots, cast, optional
//            post-scale, write the bucket
//
// reduce-scatter = phases 1-2 without the re-quantize (writes the fp32 sum to `out`);
// all-gather = phase 2 fed from `in` plus phase 3.  All three modes keep both flag
// handshakes, which is what makes back-to-back calls safe without a separate barrier.
//
// Small all-reduces (up to 16 Mi elements, 4- or 8-bit codes) take a second form of the same
// three phases, further down ("small buckets"): every packed word and every scale travels as
// an 8-byte {word, epoch} pair that the consumer polls, so the two flag handshakes, the fence
// and the arrival counters disappear and the launch is an ordinary one.  Same numerics.
//
// Synchronisation rules: the grid is launched cooperatively (all CTAs co-resident);
// arrival counters live in the rank's control page and are re-armed by the kernel
// itself; every wait is bounded by a wall-clock budget and, when it expires, the
// kernel records {code, phase, peer, rank, observed, expected} in a host-mapped status
// record and returns instead of trapping.
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

#include "codec.cuh"
#include "symm_internal.h"

namespace bcom {

#ifndef BCOM_COLL_THREADS
#define BCOM_COLL_THREADS 512
#endif
#ifndef BCOM_PHASE2_GROUPS
#define BCOM_PHASE2_GROUPS 1
#endif
constexpr int kCollThreads = BCOM_COLL_THREADS;

struct RankParams {
  unsigned char* peer[BCOM_MAX_WORLD];
  unsigned int* status;
  const void* in;
  void* out;
  float* res1;
  float* res2;
  long long n, S, c0, L;
  unsigned long long epoch;
  unsigned long long timeout_ns;
  size_t region_bytes;
  size_t slot_stride;   // bytes between two sources' slots inside a region
  size_t scale_off;     // offset of the fp16 scales inside a slot
  int rank, world;
  int lanes_per_block;  // block / 8 (a power of two)
  int lanes_log2;
  int mode;
  unsigned int key1, key2;
  float post_scale;
  unsigned char* mc;    // NVLink multicast mapping of the symmetric blocks, or null
  size_t ll_off;        // flag-in-data launches: offset of their slots inside a region
};

// ---------------------------------------------------------------------------
// memory-model helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// one store that NVSwitch replicates into every rank's copy of the multicast-mapped block
__device__ __forceinline__ void multimem_st_b32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_b64(void* mc_addr, uint32_t lo, uint32_t hi) {
  const unsigned long long v = ((unsigned long long)hi << 32) | lo;
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc_addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// phase time stamp of the rank's first CTA into the host-mapped record (six stores per launch)
__device__ __forceinline__ void stamp(unsigned int* status, int cta, int slot) {
  if (cta == 0 && threadIdx.x == 0)
    reinterpret_cast<volatile unsigned long long*>(status + BCOM_STATUS_TIMES)[slot] =
        global_timer_ns();
}

// L2-coherent loads for slots that peers wrote during this kernel
template <int BITS>
__device__ __forceinline__ Packed8<BITS> load_group_cg(const unsigned char* base, long long g) {
  Packed8<BITS> p;
  const unsigned char* src = base + g * BITS;
  if constexpr (BITS == 1) {
    p.w[0] = __ldcg(src);
  } else if constexpr (BITS == 2) {
    p.w[0] = __ldcg(reinterpret_cast<const unsigned short*>(src));
  } else if constexpr (BITS == 4) {
    p.w[0] = __ldcg(reinterpret_cast<const unsigned int*>(src));
  } else if constexpr (BITS == 8) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(src));
    p.w[0] = v.x; p.w[1] = v.y;
  } else {
    static_assert(BITS == 12, "fused kernel: 1, 2, 4, 8 or 12 bits");
    const unsigned int* s3 = reinterpret_cast<const unsigned int*>(src);  // 12-byte groups
    p.w[0] = __ldcg(s3); p.w[1] = __ldcg(s3 + 1); p.w[2] = __ldcg(s3 + 2);
  }
  return p;
}
__device__ __forceinline__ float load_scale_cg(const unsigned char* slot, size_t scale_off,
                                               long long block_index) {
  const unsigned short raw =
      __ldcg(reinterpret_cast<const unsigned short*>(slot + scale_off) + block_index);
  return __half2float(__ushort_as_half(raw));
}

// ---------------------------------------------------------------------------
// arrive / publish / wait
// ---------------------------------------------------------------------------
// Every CTA of the rank calls this once its stores of the phase are issued.  The last
// one to arrive re-arms the other phase's counter and publishes `epoch` in slot `rank`
// of the flag array at `flag_off` on every peer.
__device__ __forceinline__ void arrive_and_publish(const RankParams& p, int ncta,
                                                   int arrive_off, int rearm_off, int flag_off) {
  __threadfence_system();  // this thread's peer stores are performed
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    unsigned int* ctr = reinterpret_cast<unsigned int*>(p.peer[p.rank] + arrive_off);
    const unsigned int seen = atomicAdd(ctr, 1u);
    is_last = (seen + 1u == (unsigned int)ncta);
    if (is_last) {
      *reinterpret_cast<volatile unsigned int*>(p.peer[p.rank] + rearm_off) = 0u;
      __threadfence_system();
    }
  }
  __syncthreads();
  if (is_last && threadIdx.x < p.world) {
    unsigned long long* flag =
        reinterpret_cast<unsigned long long*>(p.peer[threadIdx.x] + flag_off) + p.rank;
    st_release_sys(flag, p.epoch);
  }
}

// Waits until all `world` flags at `flag_off` of this rank's control page reach the
// epoch.  Returns false after recording a timeout.
__device__ __forceinline__ bool wait_flags(const RankParams& p, int flag_off, unsigned int code) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const unsigned long long* flag =
        reinterpret_cast<const unsigned long long*>(p.peer[p.rank] + flag_off) + threadIdx.x;
    unsigned long long seen = ld_acquire_sys(flag);
    if (seen < p.epoch) {
      const unsigned long long t0 = global_timer_ns();
      unsigned int spins = 0;
      while ((seen = ld_acquire_sys(flag)) < p.epoch) {
        if ((++spins & 63u) == 0u) {
          if (global_timer_ns() - t0 > p.timeout_ns) break;
          __nanosleep(64);
        }
      }
      if (seen < p.epoch) {
        failed = 1;
        if (atomicCAS(p.status, 0u, code) == 0u) {
          p.status[1] = code;
          p.status[2] = threadIdx.x;
          p.status[3] = (unsigned int)p.rank;
          p.status[4] = (unsigned int)seen;
          p.status[5] = (unsigned int)(seen >> 32);
          p.status[6] = (unsigned int)p.epoch;
          p.status[7] = (unsigned int)(p.epoch >> 32);
          __threadfence_system();
        }
      }
    }
  }
  __syncthreads();
  return failed == 0;
}

// ---------------------------------------------------------------------------
// typed tensor access with tail / alignment handling
// ---------------------------------------------------------------------------
template <typename T, bool ALIGNED>
__device__ __forceinline__ void load_vals(const T* base, long long idx, long long lim,
                                          float (&v)[GROUP]) {
  if (ALIGNED && lim >= GROUP) {
    load8_vec_coherent(base + idx, v);
  } else {
#pragma unroll
    for (int i = 0; i < GROUP; ++i) v[i] = (i < lim) ? Elem<T>::to_f(base[idx + i]) : 0.0f;
  }
}

template <typename T, bool ALIGNED>
__device__ __forceinline__ void store_vals(T* base, long long idx, long long lim,
                                           const float (&v)[GROUP]) {
  if (ALIGNED && lim >= GROUP) {
    store8_vec(base + idx, v);
  } else {
#pragma unroll
    for (int i = 0; i < GROUP; ++i)
      if (i < lim) base[idx + i] = Elem<T>::from_f(v[i]);
  }
}

template <typename T>
__device__ __forceinline__ float cast_roundtrip(float x, float post_scale) {
  // result = cast to T, then (optionally) one multiply carried out on the T value
  float y = Elem<T>::to_f(Elem<T>::from_f(x));
  if (post_scale != 1.0f) y = __fmul_rn(y, post_scale);
  return y;
}

// Quantize 8 values whose block absmax is shared by `lanes` adjacent lanes, push the
// packed group and the scale to `slot` on each listed destination.
template <int BITS>
__device__ __forceinline__ void push_group(unsigned char* slot, size_t scale_off, long long g,
                                           int lanes, int lanes_log2, const Packed8<BITS>& pk,
                                           __half sh) {
  store_group<BITS>(slot, g, pk);
  if ((g & (lanes - 1)) == 0)
    reinterpret_cast<__half*>(slot + scale_off)[g >> lanes_log2] = sh;
}

// ---------------------------------------------------------------------------
// the collective, as seen by one rank whose CTAs are numbered cta in [0, ncta)
// ---------------------------------------------------------------------------
// MC: the packed groups of the all-gather half go out as multimem stores through p.mc (built
// for 4- and 8-bit codes, whose groups are whole 32- / 64-bit words); scales stay on peer stores.
template <typename T, int BITS, bool SR, bool ALIGNED, bool MC = false>
__device__ void run_rank(const RankParams& p, int cta, int ncta) {
  const int tid = threadIdx.x;
  const long long nthreads = (long long)ncta * blockDim.x;
  const long long first = (long long)cta * blockDim.x + tid;
  const int W = p.world;
  const int lanes = p.lanes_per_block;
  const int llog = p.lanes_log2;
  const long long Gs = (p.L + GROUP - 1) / GROUP;  // groups in this shard chunk
  const long long Gp = (Gs + 31) & ~31LL;          // padded so warps never straddle shards
  const long long shard_end = p.c0 + p.L;
  unsigned char* const recv_region = p.peer[p.rank] + BCOM_CONTROL_BYTES;
  unsigned char* const gather_region = recv_region + p.region_bytes;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);

  stamp(p.status, cta, 0);
  // ---------------- phase 1: quantize every destination's shard and push it ----------
  if (p.mode != BCOM_MODE_ALL_GATHER) {
    const bool ef = p.res1 != nullptr;
    const int gs = (int)Gs, gp = (int)Gp, gfirst = (int)first, gstride = (int)nthreads;
    for (int k = 0; k < W; ++k) {
      const int j = (p.rank + k) % W;  // ranks start on different destinations
      unsigned char* slot = p.peer[j] + BCOM_CONTROL_BYTES + (size_t)p.rank * p.slot_stride;
      const long long base_idx = (long long)j * p.S + p.c0;   // first element of the chunk
      // real elements of this shard chunk: the rest of the chunk is zero padding
      long long valid_ll = min(shard_end - p.c0, p.n - base_idx);
      const int valid = (int)max(0LL, min(valid_ll, (long long)gs * GROUP));
      const T* src = in + base_idx;
      float* res = ef ? p.res1 + base_idx : nullptr;
      const uint32_t idx_lo = (uint32_t)base_idx;
      // Two groups per thread and iteration: the loads of both are issued before the first
      // is used, so a warp keeps twice the bytes in flight (the kernel waits on loads more
      // than on anything else).  gp is a multiple of 32 and a warp's first group is too, so
      // `second` is uniform over the warp and the shuffles below stay convergent.
      auto quantize_push = [&](int g, float (&v)[GROUP], const float (&r)[GROUP]) {
        const int e0 = g * GROUP;
        const bool live = g < gs;
        const int lim = live ? min(max(valid - e0, 0), GROUP) : 0;
        if (ef) {
#pragma unroll
          for (int i = 0; i < GROUP; ++i) v[i] = __fadd_rn(v[i], r[i]);
        }
        const float m = block_absmax(absmax8(v), lanes);
        const __half sh = scale_from_absmax<BITS>(m);
        const float sf = __half2float(sh);
        if (!live) return;
        Packed8<BITS> pk;
        float d[GROUP];
        if (ef) {
          pk = quant8_packed<BITS, SR, true>(v, m, sf, p.key1, idx_lo + (uint32_t)e0, d);
#pragma unroll
          for (int i = 0; i < GROUP; ++i) d[i] = __fsub_rn(v[i], d[i]);
          store_vals<float, ALIGNED>(res, e0, lim, d);
        } else {
          pk = quant8_packed<BITS, SR, false>(v, m, sf, p.key1, idx_lo + (uint32_t)e0, d);
        }
        push_group<BITS>(slot, p.scale_off, g, lanes, llog, pk, sh);
      };
      auto load_group_inputs = [&](int g, float (&v)[GROUP], float (&r)[GROUP]) {
        const int e0 = g * GROUP;
        const int lim = g < gs ? min(max(valid - e0, 0), GROUP) : 0;
        load_vals<T, ALIGNED>(src, e0, lim, v);
        if (ef) load_vals<float, ALIGNED>(res, e0, lim, r);
      };
      for (int g = gfirst; g < gp; g += 2 * gstride) {
        const int g2 = g + gstride;
        const bool second = g2 < gp;
        float v0[GROUP], r0[GROUP], v1[GROUP], r1[GROUP];
        load_group_inputs(g, v0, r0);
        if (second) load_group_inputs(g2, v1, r1);
        quantize_push(g, v0, r0);
        if (second) quantize_push(g2, v1, r1);
      }
    }
  }
  stamp(p.status, cta, 1);
  arrive_and_publish(p, ncta, BCOM_CTL_ARRIVE1, BCOM_CTL_ARRIVE2, BCOM_CTL_FLAG1);
  if (!wait_flags(p, BCOM_CTL_FLAG1, BCOM_TIMEOUT_PHASE1_FLAGS)) return;
  stamp(p.status, cta, 2);

  // ---------------- phase 2: reduce own shard, re-quantize, push to everybody ---------
  {
    const bool ef2 = p.res2 != nullptr && p.mode != BCOM_MODE_REDUCE_SCATTER;
    // Everything a group needs from memory is requested before anything is used: the first
    // eight sources' packed words and scales and the stage-2 residual (one latency instead of
    // two in a row).
    struct Inputs {
      Packed8<BITS> pk[8];
      float sc[8];
      float r[GROUP];
    };
    auto request = [&](long long g, Inputs& x) {
      const bool live = g < Gs;
      const long long off = p.c0 + g * GROUP;
      const long long lim = live ? min(shard_end - off, (long long)GROUP) : 0;
      if (p.mode == BCOM_MODE_ALL_GATHER) {
        load_vals<T, ALIGNED>(in, off, lim, x.r);       // the shard itself travels in r
      } else if (live) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (u < W) {
            const unsigned char* slot = recv_region + (size_t)u * p.slot_stride;
            x.pk[u] = load_group_cg<BITS>(slot, g);
            x.sc[u] = load_scale_cg(slot, p.scale_off, g >> llog);
          }
        }
      }
      if (ef2 && p.mode != BCOM_MODE_ALL_GATHER) load_vals<float, ALIGNED>(p.res2, off, lim, x.r);
    };
    auto reduce_push = [&](long long g, Inputs& x) {
      const bool live = g < Gs;
      const long long off = p.c0 + g * GROUP;
      const long long lim = live ? min(shard_end - off, (long long)GROUP) : 0;
      float acc[GROUP];
#pragma unroll
      for (int i = 0; i < GROUP; ++i) acc[i] = 0.0f;
      if (p.mode == BCOM_MODE_ALL_GATHER) {
#pragma unroll
        for (int i = 0; i < GROUP; ++i) acc[i] = x.r[i];
        if (ef2) {
          float r2[GROUP];
          load_vals<float, ALIGNED>(p.res2, off, lim, r2);
#pragma unroll
          for (int i = 0; i < GROUP; ++i) acc[i] = __fadd_rn(acc[i], r2[i]);
        }
      } else if (live) {
        // ascending source order: the order is part of the wire contract.  A code (at most 12
        // bits) times an fp16-valued scale (11 significant bits) is exact in fp32, so the fma
        // rounds once, exactly where add(acc, mul(code, scale)) of the host model rounds
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (u < W) {
            float c[GROUP];
            unpack8f<BITS>(x.pk[u], c);
#pragma unroll
            for (int i = 0; i < GROUP; ++i)
              acc[i] = __fmaf_rn(c[i], x.sc[u], acc[i]);  // exact product: see below
          }
        }
        for (int s0 = 8; s0 < W; s0 += 8) {     // worlds above eight: the rest, eight at a time
          Packed8<BITS> pk[8];
          float sc[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (s0 + u < W) {
              const unsigned char* slot = recv_region + (size_t)(s0 + u) * p.slot_stride;
              pk[u] = load_group_cg<BITS>(slot, g);
              sc[u] = load_scale_cg(slot, p.scale_off, g >> llog);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (s0 + u < W) {
              float c[GROUP];
              unpack8f<BITS>(pk[u], c);
#pragma unroll
              for (int i = 0; i < GROUP; ++i) acc[i] = __fmaf_rn(c[i], sc[u], acc[i]);
            }
          }
        }
      }
      if (p.mode == BCOM_MODE_REDUCE_SCATTER) {
        if (live) {
#pragma unroll
          for (int i = 0; i < GROUP; ++i) acc[i] = cast_roundtrip<T>(acc[i], p.post_scale);
          store_vals<T, ALIGNED>(out, off, lim, acc);
        }
        return;
      }
      if (ef2 && p.mode != BCOM_MODE_ALL_GATHER) {
#pragma unroll
        for (int i = 0; i < GROUP; ++i) acc[i] = __fadd_rn(acc[i], x.r[i]);
      }
      const float m = block_absmax(absmax8(acc), lanes);
      const __half sh = scale_from_absmax<BITS>(m);
      const float sf = __half2float(sh);
      if (!live) return;
      const uint32_t idx2 = (uint32_t)((long long)p.rank * p.S + off);
      Packed8<BITS> pk;
      float d[GROUP];
      if (ef2) {
        pk = quant8_packed<BITS, SR, true>(acc, m, sf, p.key2, idx2, d);
#pragma unroll
        for (int i = 0; i < GROUP; ++i) d[i] = __fsub_rn(acc[i], d[i]);
        store_vals<float, ALIGNED>(p.res2, off, lim, d);
      } else {
        pk = quant8_packed<BITS, SR, false>(acc, m, sf, p.key2, idx2, d);
      }
      if constexpr (MC) {
        static_assert(BITS == 4 || BITS == 8, "multimem path: whole-word groups only");
        const size_t slot_off = BCOM_CONTROL_BYTES + p.region_bytes + (size_t)p.rank * p.slot_stride;
        unsigned char* dst = p.mc + slot_off + (size_t)g * BITS;
        if constexpr (BITS == 4) multimem_st_b32(dst, pk.w[0]);
        else multimem_st_b64(dst, pk.w[0], pk.w[1]);
        if ((g & (lanes - 1)) == 0) {
          for (int k = 0; k < W; ++k) {
            const int t = (p.rank + k) % W;
            reinterpret_cast<__half*>(p.peer[t] + slot_off + p.scale_off)[g >> llog] = sh;
          }
        }
      } else {
        for (int k = 0; k < W; ++k) {
          const int t = (p.rank + k) % W;
          unsigned char* slot = p.peer[t] + BCOM_CONTROL_BYTES + p.region_bytes +
                                (size_t)p.rank * p.slot_stride;
          push_group<BITS>(slot, p.scale_off, g, lanes, llog, pk, sh);
        }
      }
    };
#if BCOM_PHASE2_GROUPS == 2
    // Gp is a multiple of 32 and so is a warp's first group: `second` is uniform over the warp
    for (long long g = first; g < Gp; g += 2 * nthreads) {
      const long long g2 = g + nthreads;
      const bool second = g2 < Gp;
      Inputs x0, x1;
      request(g, x0);
      if (second) request(g2, x1);
      reduce_push(g, x0);
      if (second) reduce_push(g2, x1);
    }
#else
    for (long long g = first; g < Gp; g += nthreads) {
      Inputs x;   // (two groups in flight do not fit 64 registers: they spill 600 bytes)
      request(g, x);
      reduce_push(g, x);
    }
#endif
  }
  stamp(p.status, cta, 3);
  arrive_and_publish(p, ncta, BCOM_CTL_ARRIVE2, BCOM_CTL_ARRIVE1, BCOM_CTL_FLAG2);
  if (!wait_flags(p, BCOM_CTL_FLAG2, BCOM_TIMEOUT_PHASE2_FLAGS)) return;
  stamp(p.status, cta, 4);
  if (p.mode == BCOM_MODE_REDUCE_SCATTER) {
    stamp(p.status, cta, 5);
    return;
  }

  // ---------------- phase 3: dequantize all shards into the bucket --------------------
  {
    const int gs = (int)Gs, gfirst = (int)first, gstride = (int)nthreads;
    for (int k = 0; k < W; ++k) {
      const int j = (p.rank + k) % W;
      const unsigned char* slot = gather_region + (size_t)j * p.slot_stride;
      const long long base_idx = (long long)j * p.S + p.c0;
      const long long valid_ll = min(shard_end - p.c0, p.n - base_idx);
      const int valid = (int)max(0LL, min(valid_ll, (long long)gs * GROUP));
      T* dst = out + base_idx;
      // four groups per thread and iteration, all loads first (see phase 1)
      constexpr int U = 4;
      for (int g0 = gfirst; g0 < gs; g0 += U * gstride) {
        Packed8<BITS> pk[U];
        float sf[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int g = g0 + u * gstride;
          if (g < gs) {
            pk[u] = load_group_cg<BITS>(slot, g);
            sf[u] = load_scale_cg(slot, p.scale_off, g >> llog);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int g = g0 + u * gstride;
          const int e0 = g * GROUP;
          const int lim = min(valid - e0, GROUP);
          if (g >= gs || lim <= 0) continue;
          float y[GROUP];
          unpack8f<BITS>(pk[u], y);
#pragma unroll
          for (int i = 0; i < GROUP; ++i)
            y[i] = cast_roundtrip<T>(__fmul_rn(y[i], sf[u]), p.post_scale);
          store_vals<T, ALIGNED>(dst, e0, lim, y);
        }
      }
    }
  }
  stamp(p.status, cta, 5);
}

// ---------------------------------------------------------------------------
// small buckets: the flags travel inside the data words
// ---------------------------------------------------------------------------
// Below a few megabytes the two flag handshakes of run_rank (fence, CTA arrivals, flag stores,
// polling: 13-19 us each on NVLink) cost more than the three phases together.  Here every
// 32-bit word of packed codes, and every fp16 scale, is stored as an 8-byte pair {word, epoch}
// with ONE store instruction; the consumer polls the pair it needs until its second half shows
// the epoch of this launch.  An 8-byte aligned store is performed as a whole, so a pair whose
// epoch matches carries this launch's data: no fence, no arrival counter, no flag array, and a
// thread starts on a group as soon as THAT group has arrived instead of when all of them have.
// The slots live in the tail of the two data regions (RankParams::ll_off), which no other
// kernel writes and which starts out as zeros; epochs are never zero and never repeat.
// Reuse of a slot by the next launch needs no barrier either: a rank enters launch k + 1 only
// after its phase 3 of launch k has seen every peer's reduced shard, which a peer produces
// only after it has read all it needed from its receive slots; and a rank's phase-2 stores of
// launch k + 1 wait for every peer's phase-1 words of launch k + 1, which a peer sends after
// its own phase 3 of launch k.
// The grid is NOT cooperative: no CTA waits for a CTA of its own rank.  It must still be
// resident as a whole (a CTA that has not started cannot have sent the phase-1 words a peer's
// resident CTAs are waiting for), so the host caps it at what an empty GPU holds.
__device__ __forceinline__ void st_pair(void* addr, uint32_t word, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(addr), "r"(word), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const void* addr) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(addr)
               : "memory");
  return v;
}

// Waits for `words` pairs starting at `addr`; false when the time budget ran out.
template <int WORDS>
__device__ __forceinline__ bool poll_pairs(const unsigned char* addr, uint32_t epoch,
                                           unsigned long long timeout_ns, uint32_t (&w)[WORDS]) {
#pragma unroll
  for (int k = 0; k < WORDS; ++k) {
    uint2 v = ld_pair(addr + 8 * k);
    if (v.y != epoch) {
      const unsigned long long t0 = global_timer_ns();
      unsigned int spins = 0;
      while ((v = ld_pair(addr + 8 * k)).y != epoch) {
        if ((++spins & 255u) == 0u && global_timer_ns() - t0 > timeout_ns) return false;
      }
    }
    w[k] = v.x;
  }
  return true;
}

__device__ __forceinline__ void record_ll_timeout(const RankParams& p, unsigned int code,
                                                  int peer) {
  if (atomicCAS(p.status, 0u, code) == 0u) {
    p.status[1] = code;
    p.status[2] = (unsigned int)peer;
    p.status[3] = (unsigned int)p.rank;
    p.status[4] = 0u;
    p.status[5] = 0u;
    p.status[6] = (unsigned int)p.epoch;
    p.status[7] = (unsigned int)(p.epoch >> 32);
    __threadfence_system();
  }
}

// All-reduce of one rank, whole shard in one launch (p.c0 == 0, p.L == p.S), aligned tensors.
template <typename T, int BITS, bool SR>
__device__ void run_rank_ll(const RankParams& p, int cta, int ncta) {
  static_assert(BITS == 4 || BITS == 8, "flag-in-data path: whole-word groups");
  constexpr int WORDS = BITS / 4;       // 32-bit words of packed codes per group
  constexpr int GBYTES = 8 * WORDS;     // bytes of one group's pairs
  const int tid = threadIdx.x;
  const int W = p.world;
  const int lanes = p.lanes_per_block, llog = p.lanes_log2;
  const int gs = (int)((p.L + GROUP - 1) / GROUP);
  const int gp = (gs + 31) & ~31;
  const int gfirst = cta * blockDim.x + tid, gstride = ncta * blockDim.x;
  const uint32_t epoch = (uint32_t)p.epoch == 0u ? 0x80000000u : (uint32_t)p.epoch;
  const size_t ll_base = BCOM_CONTROL_BYTES + p.ll_off;
  const unsigned char* recv = p.peer[p.rank] + ll_base;
  const unsigned char* gather = recv + p.region_bytes;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);
  const bool ef = p.res1 != nullptr, ef2 = p.res2 != nullptr;
  stamp(p.status, cta, 0);

  // ---- phase 1: quantize every destination's shard, send pairs ----
  for (int k = 0; k < W; ++k) {
    const int j = (p.rank + k) % W;
    unsigned char* slot = p.peer[j] + ll_base + (size_t)p.rank * p.slot_stride;
    const long long base_idx = (long long)j * p.S;
    const int valid = (int)max(0LL, min(p.L, p.n - base_idx));
    const T* src = in + base_idx;
    float* res = ef ? p.res1 + base_idx : nullptr;
    for (int g = gfirst; g < gp; g += gstride) {
      const int e0 = g * GROUP;
      const bool live = g < gs;
      const int lim = live ? min(max(valid - e0, 0), GROUP) : 0;
      float v[GROUP], d[GROUP];
      load_vals<T, true>(src, e0, lim, v);
      if (ef) {
        load_vals<float, true>(res, e0, lim, d);
#pragma unroll
        for (int i = 0; i < GROUP; ++i) v[i] = __fadd_rn(v[i], d[i]);
      }
      const float m = block_absmax(absmax8(v), lanes);
      const __half sh = scale_from_absmax<BITS>(m);
      const float sf = __half2float(sh);
      if (!live) continue;
      Packed8<BITS> pk;
      const uint32_t idx = (uint32_t)base_idx + (uint32_t)e0;
      if (ef) {
        pk = quant8_packed<BITS, SR, true>(v, m, sf, p.key1, idx, d);
#pragma unroll
        for (int i = 0; i < GROUP; ++i) d[i] = __fsub_rn(v[i], d[i]);
        store_vals<float, true>(res, e0, lim, d);
      } else {
        pk = quant8_packed<BITS, SR, false>(v, m, sf, p.key1, idx, d);
      }
#pragma unroll
      for (int q = 0; q < WORDS; ++q) st_pair(slot + (size_t)g * GBYTES + 8 * q, pk.w[q], epoch);
      if ((g & (lanes - 1)) == 0)
        st_pair(slot + p.scale_off + (size_t)(g >> llog) * 8, (uint32_t)__half_as_ushort(sh), epoch);
    }
  }
  stamp(p.status, cta, 1);
  stamp(p.status, cta, 2);

  // ---- phase 2: own shard: wait for each group's W sources, reduce, re-quantize, send ----
  for (int g = gfirst; g < gp; g += gstride) {
    const bool live = g < gs;
    const long long off = (long long)g * GROUP;
    const long long lim = live ? min(p.L - off, (long long)GROUP) : 0;
    float acc[GROUP], d[GROUP];
#pragma unroll
    for (int i = 0; i < GROUP; ++i) acc[i] = 0.0f;
    if (ef2) load_vals<float, true>(p.res2, off, lim, d);
    bool ok = true;
    int late = 0;
    if (live) {
      for (int s = 0; s < W && ok; ++s) {   // ascending source order: part of the wire contract
        const unsigned char* slot = recv + (size_t)s * p.slot_stride;
        uint32_t w[WORDS], sw[1];
        ok = poll_pairs<WORDS>(slot + (size_t)g * GBYTES, epoch, p.timeout_ns, w) &&
             poll_pairs<1>(slot + p.scale_off + (size_t)(g >> llog) * 8, epoch, p.timeout_ns, sw);
        late = s;
        Packed8<BITS> pk;
#pragma unroll
        for (int q = 0; q < WORDS; ++q) pk.w[q] = w[q];
        const float sc = __half2float(__ushort_as_half((unsigned short)sw[0]));
        float c[GROUP];
        unpack8f<BITS>(pk, c);
#pragma unroll
        for (int i = 0; i < GROUP; ++i) acc[i] = __fmaf_rn(c[i], sc, acc[i]);  // exact product
      }
    }
    if (__any_sync(0xffffffffu, !ok)) {   // the whole warp leaves together
      if (!ok) record_ll_timeout(p, BCOM_TIMEOUT_PHASE1_FLAGS, late);
      return;
    }
    if (ef2) {
#pragma unroll
      for (int i = 0; i < GROUP; ++i) acc[i] = __fadd_rn(acc[i], d[i]);
    }
    const float m = block_absmax(absmax8(acc), lanes);
    const __half sh = scale_from_absmax<BITS>(m);
    const float sf = __half2float(sh);
    if (!live) continue;
    const uint32_t idx2 = (uint32_t)((long long)p.rank * p.S + off);
    Packed8<BITS> pk;
    if (ef2) {
      pk = quant8_packed<BITS, SR, true>(acc, m, sf, p.key2, idx2, d);
#pragma unroll
      for (int i = 0; i < GROUP; ++i) d[i] = __fsub_rn(acc[i], d[i]);
      store_vals<float, true>(p.res2, off, lim, d);
    } else {
      pk = quant8_packed<BITS, SR, false>(acc, m, sf, p.key2, idx2, d);
    }
    for (int k = 0; k < W; ++k) {
      const int t = (p.rank + k) % W;
      unsigned char* slot = p.peer[t] + ll_base + p.region_bytes + (size_t)p.rank * p.slot_stride;
#pragma unroll
      for (int q = 0; q < WORDS; ++q) st_pair(slot + (size_t)g * GBYTES + 8 * q, pk.w[q], epoch);
      if ((g & (lanes - 1)) == 0)
        st_pair(slot + p.scale_off + (size_t)(g >> llog) * 8, (uint32_t)__half_as_ushort(sh), epoch);
    }
  }
  stamp(p.status, cta, 3);
  stamp(p.status, cta, 4);

  // ---- phase 3: every shard as it arrives: dequantize into the bucket ----
  for (int k = 0; k < W; ++k) {
    const int j = (p.rank + k) % W;
    const unsigned char* slot = gather + (size_t)j * p.slot_stride;
    const long long base_idx = (long long)j * p.S;
    const int valid = (int)max(0LL, min(p.L, p.n - base_idx));
    T* dst = out + base_idx;
    for (int g = gfirst; g < gs; g += gstride) {
      const int e0 = g * GROUP;
      const int lim = min(valid - e0, GROUP);
      uint32_t w[WORDS], sw[1];
      bool ok = true;
      if (lim > 0)
        ok = poll_pairs<WORDS>(slot + (size_t)g * GBYTES, epoch, p.timeout_ns, w) &&
             poll_pairs<1>(slot + p.scale_off + (size_t)(g >> llog) * 8, epoch, p.timeout_ns, sw);
      if (!ok) {   // nothing below needs the warp as a whole
        record_ll_timeout(p, BCOM_TIMEOUT_PHASE2_FLAGS, j);
        return;
      }
      if (lim <= 0) continue;
      Packed8<BITS> pk;
#pragma unroll
      for (int q = 0; q < WORDS; ++q) pk.w[q] = w[q];
      const float sf = __half2float(__ushort_as_half((unsigned short)sw[0]));
      float y[GROUP];
      unpack8f<BITS>(pk, y);
#pragma unroll
      for (int i = 0; i < GROUP; ++i) y[i] = cast_roundtrip<T>(__fmul_rn(y[i], sf), p.post_scale);
      store_vals<T, true>(dst, e0, lim, y);
    }
  }
  stamp(p.status, cta, 5);
}

template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kCollThreads, 2)
lowbit_collective_ll_kernel(const RankParams p) {
  run_rank_ll<T, BITS, SR>(p, blockIdx.x, gridDim.x);
}

template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kCollThreads, 2)
lowbit_collective_ll_emulated_kernel(const RankParams* all, int world) {
  const int per_rank = gridDim.x / world;
  const int r = blockIdx.x / per_rank;
  if (r >= world) return;
  __shared__ RankParams p;
  if (threadIdx.x == 0) p = all[r];
  __syncthreads();
  run_rank_ll<T, BITS, SR>(p, blockIdx.x - r * per_rank, per_rank);
}

template <typename T, int BITS, bool SR, bool ALIGNED>
__global__ void __launch_bounds__(kCollThreads, 2)
lowbit_collective_kernel(const RankParams p) {
  run_rank<T, BITS, SR, ALIGNED>(p, blockIdx.x, gridDim.x);
}

// the same kernel with the all-gather half on NVLink multicast stores (aligned buckets only)
template <typename T, int BITS, bool SR>
__global__ void __launch_bounds__(kCollThreads, 2)
lowbit_collective_mc_kernel(const RankParams p) {
  run_rank<T, BITS, SR, true, true>(p, blockIdx.x, gridDim.x);
}

// Same-device emulation of `world` ranks in ONE cooperative launch: CTA groups play the
// ranks, so the whole flag protocol runs (and can be tested) on a single GPU.
template <typename T, int BITS, bool SR, bool ALIGNED>
__global__ void __launch_bounds__(kCollThreads, 2)
lowbit_collective_emulated_kernel(const RankParams* all, int world) {
  const int per_rank = gridDim.x / world;
  const int r = blockIdx.x / per_rank;
  if (r >= world) return;
  __shared__ RankParams p;
  if (threadIdx.x == 0) p = all[r];
  __syncthreads();
  run_rank<T, BITS, SR, ALIGNED>(p, blockIdx.x - r * per_rank, per_rank);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef void (*RealKernel)(const RankParams);
typedef void (*EmuKernel)(const RankParams*, int);

template <typename T, int BITS>
static void pick(bool sr, bool aligned, RealKernel* real, EmuKernel* emu) {
  if (sr && aligned) {
    *real = lowbit_collective_kernel<T, BITS, true, true>;
    *emu = lowbit_collective_emulated_kernel<T, BITS, true, true>;
  } else if (sr) {
    *real = lowbit_collective_kernel<T, BITS, true, false>;
    *emu = lowbit_collective_emulated_kernel<T, BITS, true, false>;
  } else if (aligned) {
    *real = lowbit_collective_kernel<T, BITS, false, true>;
    *emu = lowbit_collective_emulated_kernel<T, BITS, false, true>;
  } else {
    *real = lowbit_collective_kernel<T, BITS, false, false>;
    *emu = lowbit_collective_emulated_kernel<T, BITS, false, false>;
  }
}

template <typename T>
static bool pick_bits(int bits, bool sr, bool aligned, RealKernel* real, EmuKernel* emu) {
  switch (bits) {
    case 1: pick<T, 1>(sr, aligned, real, emu); return true;
    case 2: pick<T, 2>(sr, aligned, real, emu); return true;
    case 4: pick<T, 4>(sr, aligned, real, emu); return true;
    case 8: pick<T, 8>(sr, aligned, real, emu); return true;
    case 12: pick<T, 12>(sr, aligned, real, emu); return true;
    default: return false;
  }
}

static bool pick_kernel(int dtype, int bits, bool sr, bool aligned, RealKernel* real,
                        EmuKernel* emu) {
  switch (dtype) {
    case 0: return pick_bits<float>(bits, sr, aligned, real, emu);
    case 1: return pick_bits<__half>(bits, sr, aligned, real, emu);
    case 2: return pick_bits<__nv_bfloat16>(bits, sr, aligned, real, emu);
    default: return false;
  }
}

template <typename T>
static bool pick_mc_bits(int bits, bool sr, RealKernel* real) {
  if (bits == 4) *real = sr ? lowbit_collective_mc_kernel<T, 4, true>
                            : lowbit_collective_mc_kernel<T, 4, false>;
  else if (bits == 8) *real = sr ? lowbit_collective_mc_kernel<T, 8, true>
                                 : lowbit_collective_mc_kernel<T, 8, false>;
  else return false;
  return true;
}

// multicast variant of the kernel for this setting, if there is one
static bool pick_mc_kernel(int dtype, int bits, bool sr, RealKernel* real) {
  switch (dtype) {
    case 0: return pick_mc_bits<float>(bits, sr, real);
    case 1: return pick_mc_bits<__half>(bits, sr, real);
    case 2: return pick_mc_bits<__nv_bfloat16>(bits, sr, real);
    default: return false;
  }
}

static bool block_ok(int block) {
  if (block % GROUP) return false;
  const int t = block / GROUP;
  return t >= 1 && t <= 32 && (t & (t - 1)) == 0;
}

static int elem_size(int dtype) { return dtype == 0 ? 4 : 2; }

struct SlotLayout {
  size_t scale_off;
  size_t stride;
};

// layout of one source's slot for a chunk of `L` elements
static SlotLayout slot_layout(long long L, int bits, int block) {
  const long long groups = ((L + GROUP - 1) / GROUP + 31) & ~31LL;
  SlotLayout s;
  s.scale_off = bcom_align_up((size_t)groups * bits, 256);
  const size_t scale_bytes = bcom_align_up((size_t)((L + block - 1) / block + 32) * 2, 256);
  s.stride = s.scale_off + scale_bytes;
  return s;
}

static long long max_chunk(size_t region_bytes, int world, int bits, int block) {
  // largest L (multiple of 256 elements) with world * stride(L) <= region_bytes
  const double per_elem = bits / 8.0 + 2.0 / block;
  long long L = (long long)((double)(region_bytes / world) / per_elem);
  L = L / 256 * 256;
  while (L > 0 && (size_t)world * slot_layout(L, bits, block).stride > region_bytes) L -= 256;
  return L;
}

// Vector path: shards start on 8-element boundaries and every tensor base is aligned to one
// 8-element group (32 bytes for fp32 tensors and the fp32 residuals, 16 bytes for 2-byte types).
static bool is_aligned(const BcomCollArgs& a) {
  const uintptr_t tmask = a.dtype == 0 ? 31 : 15;
  auto ok = [](const void* p, uintptr_t mask) { return ((uintptr_t)p & mask) == 0; };
  return a.S % GROUP == 0 && ok(a.in, tmask) && ok(a.out, tmask) && ok(a.res1, 31) &&
         ok(a.res2, 31);
}

static int validate(const BcomComm* c, const BcomCollArgs& a) {
  if (!c || a.n < 0 || a.S <= 0 || !block_ok(a.block)) return (int)cudaErrorInvalidValue;
  if (a.n > (long long)c->world * a.S) return (int)cudaErrorInvalidValue;
  if (a.mode < 0 || a.mode > 2) return (int)cudaErrorInvalidValue;
  for (int r = 0; r < c->world; ++r)  // a peer was unmapped (bcom_comm_close_peers) or never wired
    if (!c->peer[r]) return (int)cudaErrorInvalidResourceHandle;
  return 0;
}

static void fill_params(const BcomComm* c, const BcomCollArgs& a, long long c0, long long L,
                        unsigned long long epoch, RankParams* p) {
  for (int i = 0; i < BCOM_MAX_WORLD; ++i) p->peer[i] = i < c->world ? c->peer[i] : nullptr;
  p->status = c->status_dev;
  p->in = a.in;
  p->out = a.out;
  p->res1 = a.res1;
  p->res2 = a.res2;
  p->n = a.n;
  p->S = a.S;
  p->c0 = c0;
  p->L = L;
  p->epoch = epoch;
  p->timeout_ns = c->timeout_ns;
  p->region_bytes = c->region_bytes;
  const SlotLayout lay = slot_layout(L, a.bits, a.block);
  p->slot_stride = lay.stride;
  p->scale_off = lay.scale_off;
  p->rank = c->rank;
  p->world = c->world;
  p->lanes_per_block = a.block / GROUP;
  p->lanes_log2 = 0;
  while ((1 << p->lanes_log2) < p->lanes_per_block) ++p->lanes_log2;
  p->mode = a.mode;
  p->key1 = a.key1;
  p->key2 = a.key2;
  p->post_scale = a.post_scale;
  p->mc = c->mc;
  p->ll_off = 0;
}

static int ctas_for(const BcomComm* c, const BcomCollArgs& a, long long L, int resident_per_sm) {
  const long long groups = ((L + GROUP - 1) / GROUP + 31) & ~31LL;
  long long want = ((long long)c->world * groups + kCollThreads - 1) / kCollThreads;
  long long cap = (long long)c->sm_count * resident_per_sm;
  if (a.max_ctas > 0 && a.max_ctas < cap) cap = a.max_ctas;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

// resident CTAs per SM of a kernel, asked once per kernel
static cudaError_t resident_ctas(const void* kernel, int* out) {
  static std::mutex mu;
  static std::unordered_map<const void*, int> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(kernel);
  if (it != cache.end()) {
    *out = it->second;
    return cudaSuccess;
  }
  cudaError_t err =
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(out, kernel, kCollThreads, 0);
  if (err == cudaSuccess) cache[kernel] = *out;
  return err;
}


// ---- flag-in-data path: kernels, layout, when it applies ---------------------------------
typedef void (*LLEmuKernel)(const RankParams*, int);

template <typename T>
static bool pick_ll_bits(int bits, bool sr, RealKernel* real, LLEmuKernel* emu) {
  if (bits == 4) {
    *real = sr ? lowbit_collective_ll_kernel<T, 4, true> : lowbit_collective_ll_kernel<T, 4, false>;
    *emu = sr ? lowbit_collective_ll_emulated_kernel<T, 4, true>
              : lowbit_collective_ll_emulated_kernel<T, 4, false>;
  } else if (bits == 8) {
    *real = sr ? lowbit_collective_ll_kernel<T, 8, true> : lowbit_collective_ll_kernel<T, 8, false>;
    *emu = sr ? lowbit_collective_ll_emulated_kernel<T, 8, true>
              : lowbit_collective_ll_emulated_kernel<T, 8, false>;
  } else {
    return false;
  }
  return true;
}

static bool pick_ll_kernel(int dtype, int bits, bool sr, RealKernel* real, LLEmuKernel* emu) {
  switch (dtype) {
    case 0: return pick_ll_bits<float>(bits, sr, real, emu);
    case 1: return pick_ll_bits<__half>(bits, sr, real, emu);
    case 2: return pick_ll_bits<__nv_bfloat16>(bits, sr, real, emu);
    default: return false;
  }
}

// one source's slot: 8 bytes per 32-bit word of packed codes, then 8 bytes per block scale
static SlotLayout ll_slot_layout(long long L, int bits, int block) {
  const long long groups = ((L + GROUP - 1) / GROUP + 31) & ~31LL;
  SlotLayout s;
  s.scale_off = bcom_align_up((size_t)groups * 2 * bits, 256);
  s.stride = s.scale_off + bcom_align_up((size_t)((L + block - 1) / block + 32) * 8, 256);
  return s;
}

// all-reduce of an aligned tensor that is small enough for one flag-in-data launch
static bool ll_applies(const BcomComm* c, const BcomCollArgs& a) {
  if (a.mode != BCOM_MODE_ALL_REDUCE || (a.bits != 4 && a.bits != 8) || !is_aligned(a)) return false;
  if (c->ll_bytes == 0 || c->ll_max_payload <= 0) return false;
  // the limit counts four bytes per element whatever the dtype: what the form costs grows with
  // the number of codes, not with the width of the tensor (measured at 4 GPUs: it wins up to
  // 16 Mi elements, ties at 32 Mi, loses beyond)
  if (a.n * 4 > c->ll_max_payload) return false;
  return (size_t)c->world * ll_slot_layout(a.S, a.bits, a.block).stride <= c->ll_bytes;
}

static void fill_ll_params(const BcomComm* c, const BcomCollArgs& a, unsigned long long epoch,
                           RankParams* p) {
  fill_params(c, a, 0, a.S, epoch, p);
  const SlotLayout lay = ll_slot_layout(a.S, a.bits, a.block);
  p->slot_stride = lay.stride;
  p->scale_off = lay.scale_off;
  p->ll_off = c->region_bytes - c->ll_bytes;
}

}  // namespace bcom

using namespace bcom;

extern "C" {

int bcom_collective_supported(int dtype, int bits, int block) {
  RealKernel r;
  EmuKernel e;
  return (pick_kernel(dtype, bits, false, true, &r, &e) && block_ok(block)) ? 1 : 0;
}

long long bcom_comm_max_chunk(BcomComm* c, int bits, int block) {
  if (!c || !block_ok(block)) return 0;
  return max_chunk(c->region_bytes - c->ll_bytes, c->world, bits, block);
}

int bcom_collective(BcomComm* c, const BcomCollArgs* args, void* stream) {
  const BcomCollArgs& a = *args;
  if (int err = validate(c, a)) return err;
  RealKernel kernel;
  EmuKernel unused;
  if (ll_applies(c, a)) {
    LLEmuKernel unused_emu;
    if (!pick_ll_kernel(a.dtype, a.bits, a.stochastic != 0, &kernel, &unused_emu))
      return (int)cudaErrorNotSupported;
    int resident = 0;
    cudaError_t err = resident_ctas((const void*)kernel, &resident);
    if (err != cudaSuccess) return (int)err;
    if (resident < 1) return (int)cudaErrorLaunchOutOfResources;
    RankParams p;
    fill_ll_params(c, a, ++c->epoch, &p);
    // an ordinary launch: no CTA waits for a CTA of its own rank; the grid is capped at what an
    // empty GPU holds (ctas_for) because the peers wait for words of CTAs that must have started
    kernel<<<ctas_for(c, a, a.S, resident), kCollThreads, 0, (cudaStream_t)stream>>>(p);
    return (int)cudaGetLastError();
  }
  if (!pick_kernel(a.dtype, a.bits, a.stochastic != 0, is_aligned(a), &kernel, &unused))
    return (int)cudaErrorNotSupported;
  // with a multicast mapping, the modes that have an all-gather half use the multimem kernel
  if (c->mc != nullptr && is_aligned(a) && a.mode != BCOM_MODE_REDUCE_SCATTER) {
    RealKernel mc_kernel;
    if (pick_mc_kernel(a.dtype, a.bits, a.stochastic != 0, &mc_kernel)) kernel = mc_kernel;
  }
  int resident = 0;
  cudaError_t err = resident_ctas((const void*)kernel, &resident);
  if (err != cudaSuccess) return (int)err;
  if (resident < 1) return (int)cudaErrorLaunchOutOfResources;
  long long Lmax = max_chunk(c->region_bytes - c->ll_bytes, c->world, a.bits, a.block);
  if (Lmax <= 0) return (int)cudaErrorMemoryAllocation;
  Lmax = Lmax / a.block * a.block;  // chunks start on quantization-block boundaries
  if (Lmax <= 0) return (int)cudaErrorMemoryAllocation;
  for (long long c0 = 0; c0 < a.S; c0 += Lmax) {
    const long long L = a.S - c0 < Lmax ? a.S - c0 : Lmax;
    RankParams p;
    fill_params(c, a, c0, L, ++c->epoch, &p);
    void* kargs[] = {&p};
    err = cudaLaunchCooperativeKernel((const void*)kernel, dim3(ctas_for(c, a, L, resident)),
                                      dim3(kCollThreads), kargs, 0, (cudaStream_t)stream);
    if (err != cudaSuccess) return (int)err;
  }
  return 0;
}

int bcom_collective_emulated(BcomComm** comms, const BcomCollArgs* args, int world,
                             void* stream) {
  if (world < 1 || world > BCOM_MAX_WORLD) return (int)cudaErrorInvalidValue;
  for (int r = 0; r < world; ++r)
    if (int err = validate(comms[r], args[r])) return err;
  const BcomCollArgs& a0 = args[0];
  bool aligned = true;
  for (int r = 0; r < world; ++r) aligned = aligned && is_aligned(args[r]);
  RealKernel unused;
  EmuKernel kernel;
  bool ll = true;
  for (int r = 0; r < world; ++r) ll = ll && ll_applies(comms[r], args[r]);
  if (ll) {
    LLEmuKernel ll_kernel;
    if (!pick_ll_kernel(a0.dtype, a0.bits, a0.stochastic != 0, &unused, &ll_kernel))
      return (int)cudaErrorNotSupported;
    int resident = 0;
    cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
        &resident, (const void*)ll_kernel, kCollThreads, 0);
    if (err != cudaSuccess) return (int)err;
    if (resident < 1) return (int)cudaErrorLaunchOutOfResources;
    RankParams host[BCOM_MAX_WORLD];
    for (int r = 0; r < world; ++r) fill_ll_params(comms[r], args[r], ++comms[r]->epoch, &host[r]);
    RankParams* dev_params = nullptr;
    err = cudaMallocAsync((void**)&dev_params, sizeof(RankParams) * world, (cudaStream_t)stream);
    if (err != cudaSuccess) return (int)err;
    err = cudaMemcpyAsync(dev_params, host, sizeof(RankParams) * world, cudaMemcpyHostToDevice,
                          (cudaStream_t)stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize((cudaStream_t)stream);
    if (err == cudaSuccess) {
      int per_rank = ctas_for(comms[0], a0, a0.S, resident);
      const int cap = comms[0]->sm_count * resident / world;
      if (per_rank > cap) per_rank = cap;
      if (per_rank < 1) {
        err = cudaErrorLaunchOutOfResources;
      } else {
        int w = world;
        void* kargs[] = {&dev_params, &w};
        // all emulated ranks share this GPU: cooperative, so that every rank's CTAs are resident
        err = cudaLaunchCooperativeKernel((const void*)ll_kernel, dim3(per_rank * world),
                                          dim3(kCollThreads), kargs, 0, (cudaStream_t)stream);
      }
    }
    cudaFreeAsync(dev_params, (cudaStream_t)stream);
    return (int)err;
  }
  if (!pick_kernel(a0.dtype, a0.bits, a0.stochastic != 0, aligned, &unused, &kernel))
    return (int)cudaErrorNotSupported;
  int resident = 0;
  cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(
      &resident, (const void*)kernel, kCollThreads, 0);
  if (err != cudaSuccess) return (int)err;
  if (resident < 1) return (int)cudaErrorLaunchOutOfResources;
  BcomComm* c0comm = comms[0];
  long long Lmax = max_chunk(c0comm->region_bytes - c0comm->ll_bytes, world, a0.bits, a0.block);
  Lmax = Lmax / a0.block * a0.block;
  if (Lmax <= 0) return (int)cudaErrorMemoryAllocation;
  RankParams* dev_params = nullptr;
  err = cudaMallocAsync((void**)&dev_params, sizeof(RankParams) * world, (cudaStream_t)stream);
  if (err != cudaSuccess) return (int)err;
  for (long long c0 = 0; c0 < a0.S; c0 += Lmax) {
    const long long L = a0.S - c0 < Lmax ? a0.S - c0 : Lmax;
    RankParams host[BCOM_MAX_WORLD];
    for (int r = 0; r < world; ++r)
      fill_params(comms[r], args[r], c0, L, ++comms[r]->epoch, &host[r]);
    err = cudaMemcpyAsync(dev_params, host, sizeof(RankParams) * world, cudaMemcpyHostToDevice,
                          (cudaStream_t)stream);
    if (err != cudaSuccess) break;
    // host[] is on the stack: make sure the copy has consumed it
    err = cudaStreamSynchronize((cudaStream_t)stream);
    if (err != cudaSuccess) break;
    int per_rank = ctas_for(c0comm, a0, L, resident);
    const int cap = c0comm->sm_count * resident / world;
    if (per_rank > cap) per_rank = cap;
    if (per_rank < 1) { err = cudaErrorLaunchOutOfResources; break; }
    int w = world;
    void* kargs[] = {&dev_params, &w};
    err = cudaLaunchCooperativeKernel((const void*)kernel, dim3(per_rank * world),
                                      dim3(kCollThreads), kargs, 0, (cudaStream_t)stream);
    if (err != cudaSuccess) break;
  }
  cudaFreeAsync(dev_params, (cudaStream_t)stream);
  return (int)err;
}

}  // extern "C"
