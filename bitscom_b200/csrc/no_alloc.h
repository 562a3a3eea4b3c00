// Allocation-free entry point.  It has no counterpart in the reference library.
//
// Who needs it: hosts that may not allocate device memory at the moment they call into
// this library — a serving or training runtime that hands the GPU's memory to one arena at
// start-up and forbids cudaMalloc afterwards, a plugin called from inside another
// framework's allocator lock, or C code without access to torch's caching allocator.  The
// ordinary attention backward entry point (bcom_attention_bwd) expects the caller to bring
// two scratch buffers; this variant brings its own, a fixed array that lives inside the
// library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of device scratch built into the library.  Every GPU that loads the library
// holds this much until the process exits.
#define BCOM_NO_ALLOC_SCRATCH_BYTES (36u << 20)

// Same computation and same outputs as bcom_attention_bwd (causal flash-attention
// backward, head_dim 128, seq % 128 == 0), but the fp32 dQ accumulator
// [batch*seq, heads*128] and the row-statistics buffer [batch, heads, seq] come from the
// built-in scratch array instead of from the caller.
//
//   * Limit: 4 * batch*seq * heads*128 + 4 * batch*heads*seq (rounded up to 256) bytes must
//     fit in BCOM_NO_ALLOC_SCRATCH_BYTES; larger problems are refused with return code
//     1006 and a message on stderr, nothing is launched.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any call.
//   * The first call on a device looks up the device address of the scratch array
//     (cudaGetSymbolAddress) with that device current; make that first call outside any
//     stream capture.
//   * The array is part of the library's device image.  With CUDA's default lazy module
//     loading the image (and with it the 36 MiB) is placed on a device when the first kernel
//     or symbol of this library is used there, which may be this entry point's own first
//     call.  A host that gives all device memory to an arena must therefore touch the library
//     BEFORE it does so (one warm-up call of any entry point of this library on that device,
//     or CUDA_MODULE_LOADING=EAGER in the environment); otherwise that first call can fail
//     with an out-of-memory error from the module load, although it allocates nothing itself.
//   * Return codes: 0; 1001-1006 for argument errors (1006: larger than the scratch); any
//     other value is the cudaError_t of the failing runtime call (for example 2,
//     cudaErrorMemoryAllocation, from the module load described above).
//   * All calls on a device share the one array, and it keeps whatever the previous call
//     left: the accumulator part is cleared on the stream at the start of every call.
//     Two calls whose kernels overlap on the GPU (different streams, no ordering) race
//     on the array and corrupt each other's gradients: order them.
//
// Returns 0 or an error code as bcom_attention_bwd does.
int bcom_attention_bwd_no_alloc(const void* qkv, const void* out, const void* d_out,
                                const void* lse2, void* dqkv, int batch, int seq, int heads,
                                int head_dim, float scale, void* stream);

// BCOM_NO_ALLOC_SCRATCH_BYTES, for callers that bind through dlsym.
unsigned long long bcom_no_alloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
