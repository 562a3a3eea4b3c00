// Thin inline-PTX layer for Blackwell (sm_100a) tensor-core kernels: mbarriers with
// bounded waits, TMA tiled loads, TMEM allocation, tcgen05.mma / commit / ld, and the
// shared-memory / instruction descriptors they consume.
//
// Descriptor bit layouts (sm_100 "UMMA"):
//   shared-memory matrix descriptor (64 bit)
//     [ 0,14) start address >> 4        [16,30) leading-dim byte offset >> 4
//     [32,46) stride-dim byte offset >> 4   [46,48) version = 1
//     [49,52) base offset = 0           [61,64) swizzle: 0 none, 2 128B, 4 64B, 6 32B
//   instruction descriptor (32 bit), kind::f16
//     [4,6) D format (1 = f32)  [7,10) A format (0 f16, 1 bf16)  [10,13) B format
//     [15] A is MN-major  [16] B is MN-major  [17,23) N >> 3  [24,29) M >> 4
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <mutex>

namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `budget_ns` of wall clock and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          unsigned long long budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > budget_ns) return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// TMA: 2-D tiled load, global -> shared, completion on an mbarrier
// (coordinate 0 is the contiguous dimension; c0 * elem_size must be a multiple of 16)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// 2-D tiled reduction, shared -> global: global[tile] += shared[tile], element-wise, in the
// tensor map's data type.  Completion is tracked by bulk groups of the issuing thread.  The
// innermost coordinate times the element size must be a multiple of 16 bytes and no
// coordinate may be negative.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src,
                                                  int c0, int c1) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group"
      " [%0, {%2, %3}], [%1];"
      :
      : "l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// all committed groups of this thread have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// ... have completed entirely (their global writes are performed)
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------
// TMEM
// ---------------------------------------------------------------------------
// Executed by one full warp. Writes the base TMEM address to *smem_out.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_out, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_out)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp reads lane (base+t)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// the store twin: thread t of the warp writes 32 consecutive columns of lane (base+t)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// 128-byte swizzled operand tile; `lbo_bytes` / `sbo_bytes` as defined in the header
// comment (K-major: lbo unused (1), sbo = 1024; MN-major: lbo = bytes between 64-element
// MN chunks, sbo = 1024).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                        uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, bool a_mn_major,
                                                       bool b_mn_major) {
  return (1u << 4)                       // D = f32
         | (1u << 7) | (1u << 10)        // A, B = bf16
         | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// mbarrier arrives once all tcgen05 ops issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Host side.  cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link
// against libcuda); nullptr when the driver does not offer it.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

// Tensor map of a 2-D row-major matrix [rows, cols] of bf16 (elem_bytes 2) or fp32 (4)
// elements with leading dimension `ld` (elements), 128-byte swizzle, boxes of
// box_cols x box_rows elements, out-of-range elements read as zero.  Returns the driver's
// result code (0 = ok, -1 = entry point missing) and reports a failure on stderr.
inline int make_tensor_map_2d(CUtensorMap* map, const void* ptr, int elem_bytes, long long rows,
                              long long cols, long long ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const bool half = elem_bytes == 2;
  const CUresult r = fn(
      map, half ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B,
      half ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr,
            "bitscom_b200: cuTensorMapEncodeTiled failed (%d): ptr=%p elem=%d rows=%lld "
            "cols=%lld ld=%lld box=%dx%d\n",
            (int)r, ptr, elem_bytes, rows, cols, ld, box_cols, box_rows);
  return (int)r;
}

// Tensor maps are pure functions of (address, shape, leading dimension, box): a training step
// presents the same few hundred operands again and again (weights, and activations that the
// caching allocator hands back at the same addresses), so the encoded maps are kept in a small
// per-thread direct-mapped cache and the driver call is skipped on a hit.
struct TensorMapKey {
  const void* ptr;
  long long rows, cols, ld;
  int elem_bytes, box_cols, box_rows;
  bool operator==(const TensorMapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           elem_bytes == o.elem_bytes && box_cols == o.box_cols && box_rows == o.box_rows;
  }
};

inline int cached_tensor_map_2d(CUtensorMap* map, const void* ptr, int elem_bytes, long long rows,
                                long long cols, long long ld, int box_cols, int box_rows) {
  constexpr int kSlots = 1024;
  struct Slot {
    TensorMapKey key;
    CUtensorMap map;
    bool valid;
  };
  static thread_local Slot* slots = nullptr;
  if (!slots) slots = new Slot[kSlots]();
  const TensorMapKey key{ptr, rows, cols, ld, elem_bytes, box_cols, box_rows};
  unsigned long long h = (unsigned long long)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
  h ^= (unsigned long long)rows * 0xC2B2AE3D27D4EB4Full + (unsigned long long)cols * 0x165667B19E3779F9ull;
  h ^= (unsigned long long)ld * 0x27D4EB2F165667C5ull + (unsigned long long)(box_cols * 131 + box_rows);
  Slot& s = slots[(h >> 32) % kSlots];
  if (s.valid && s.key == key) {
    *map = s.map;
    return 0;
  }
  const int r = make_tensor_map_2d(map, ptr, elem_bytes, rows, cols, ld, box_cols, box_rows);
  if (r == 0) {
    s.key = key;
    s.map = *map;
    s.valid = true;
  }
  return r;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of on every
// launch.  Returns false if the attribute could not be set.
inline bool ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Seen {
    const void* kernel;
    int device;
  };
  static std::mutex mu;
  static Seen seen[256];
  static int count = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < count; ++i)
    if (seen[i].kernel == kernel && seen[i].device == dev) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
      cudaSuccess)
    return false;
  if (count < 256) seen[count++] = Seen{kernel, dev};
  return true;
}

// Driver calls such as the tensor-map encoder need the device's primary context
// bound to the calling thread, which an autograd worker thread may not have yet: a no-op
// runtime call binds it.  Done once per (thread, device), so that later calls issue nothing
// that stream capture would object to.
inline void bind_context_once() {
  static thread_local int bound_device = -1;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  if (dev != bound_device) {
    (void)cudaFree(nullptr);
    (void)cudaGetLastError();
    bound_device = dev;
  }
}


}  // namespace tc
