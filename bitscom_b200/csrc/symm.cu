// Host side of the symmetric-memory communicator: allocation, CUDA IPC mapping of the
// peers' blocks, status record, reset.  See symm.h for the layout and the protocol.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "symm_internal.h"

#define BCOM_TRY(expr)                         \
  do {                                         \
    cudaError_t e__ = (expr);                  \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)

// canary pattern in the unused tail of the control page and in the guard page behind the regions
static cudaError_t write_canaries(BcomComm* c) {
  cudaError_t err = cudaMemset(c->local + BCOM_CTL_CANARY, BCOM_CANARY_BYTE,
                               BCOM_CONTROL_BYTES - BCOM_CTL_CANARY);
  // the tail of both data regions only ever holds (data, epoch) words of the flag-in-data
  // path: it starts out as zeros, and epoch 0 is never used
  for (int region = 0; region < 2 && err == cudaSuccess; ++region)
    if (c->ll_bytes)
      err = cudaMemset(c->local + BCOM_CONTROL_BYTES + (region + 1) * c->region_bytes -
                           c->ll_bytes, 0, c->ll_bytes);
  if (err == cudaSuccess)
    err = cudaMemset(c->local + BCOM_CONTROL_BYTES + 2 * c->region_bytes, BCOM_CANARY_BYTE,
                     BCOM_GUARD_BYTES);
  return err;
}

extern "C" {

int bcom_comm_create(int rank, int world, size_t region_bytes, BcomComm** out) {
  if (!out || world < 1 || world > BCOM_MAX_WORLD || rank < 0 || rank >= world)
    return (int)cudaErrorInvalidValue;
  BcomComm* c = new (std::nothrow) BcomComm();
  if (!c) return (int)cudaErrorMemoryAllocation;
  std::memset(c, 0, sizeof(*c));
  c->rank = rank;
  c->world = world;
  c->region_bytes = bcom_align_up(region_bytes, 4096);
  c->total_bytes = BCOM_CONTROL_BYTES + 2 * c->region_bytes + BCOM_GUARD_BYTES;
  c->timeout_ns = 30ull * 1000ull * 1000ull * 1000ull;
  c->ll_bytes = c->region_bytes / 8 / 4096 * 4096;
  c->ll_max_payload = 64ll << 20;
  cudaError_t err = cudaGetDevice(&c->device);
  if (err == cudaSuccess)
    err = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device);
  if (err == cudaSuccess) err = cudaMalloc((void**)&c->local, c->total_bytes);
  if (err == cudaSuccess) err = cudaMemset(c->local, 0, BCOM_CONTROL_BYTES);
  if (err == cudaSuccess) err = write_canaries(c);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();  // peers may write as soon as they map us
  if (err == cudaSuccess)
    err = cudaHostAlloc((void**)&c->status_host, BCOM_STATUS_WORDS * sizeof(unsigned int),
                        cudaHostAllocMapped);
  if (err == cudaSuccess) {
    std::memset(c->status_host, 0, BCOM_STATUS_WORDS * sizeof(unsigned int));
    err = cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0);
  }
  if (err != cudaSuccess) {
    if (c->local) cudaFree(c->local);
    if (c->status_host) cudaFreeHost(c->status_host);
    delete c;
    return (int)err;
  }
  c->peer[rank] = c->local;
  c->owns_local = true;
  *out = c;
  return 0;
}

size_t bcom_comm_block_bytes(size_t region_bytes) {
  return BCOM_CONTROL_BYTES + 2 * bcom_align_up(region_bytes, 4096) + BCOM_GUARD_BYTES;
}

int bcom_comm_create_external(int rank, int world, size_t region_bytes, void* const* bases,
                              void* mc_base, BcomComm** out) {
  if (!out || !bases || world < 1 || world > BCOM_MAX_WORLD || rank < 0 || rank >= world)
    return (int)cudaErrorInvalidValue;
  for (int p = 0; p < world; ++p)
    if (!bases[p] || ((uintptr_t)bases[p] & 255)) return (int)cudaErrorInvalidValue;
  if ((uintptr_t)mc_base & 255) return (int)cudaErrorInvalidValue;
  BcomComm* c = new (std::nothrow) BcomComm();
  if (!c) return (int)cudaErrorMemoryAllocation;
  std::memset(c, 0, sizeof(*c));
  c->rank = rank;
  c->world = world;
  c->region_bytes = bcom_align_up(region_bytes, 4096);
  c->total_bytes = BCOM_CONTROL_BYTES + 2 * c->region_bytes + BCOM_GUARD_BYTES;
  c->timeout_ns = 30ull * 1000ull * 1000ull * 1000ull;
  c->ll_bytes = c->region_bytes / 8 / 4096 * 4096;
  c->ll_max_payload = 64ll << 20;
  c->local = (unsigned char*)bases[rank];
  c->mc = (unsigned char*)mc_base;
  c->owns_local = false;
  for (int p = 0; p < world; ++p) c->peer[p] = (unsigned char*)bases[p];
  cudaError_t err = cudaGetDevice(&c->device);
  if (err == cudaSuccess)
    err = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device);
  if (err == cudaSuccess) err = cudaMemset(c->local, 0, BCOM_CONTROL_BYTES);
  if (err == cudaSuccess) err = write_canaries(c);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err == cudaSuccess)
    err = cudaHostAlloc((void**)&c->status_host, BCOM_STATUS_WORDS * sizeof(unsigned int),
                        cudaHostAllocMapped);
  if (err == cudaSuccess) {
    std::memset(c->status_host, 0, BCOM_STATUS_WORDS * sizeof(unsigned int));
    err = cudaHostGetDevicePointer((void**)&c->status_dev, c->status_host, 0);
  }
  if (err != cudaSuccess) {
    if (c->status_host) cudaFreeHost(c->status_host);
    delete c;
    return (int)err;
  }
  *out = c;
  return 0;
}

void* bcom_comm_multicast_base(BcomComm* c) { return c ? c->mc : nullptr; }

int bcom_comm_close_peers(BcomComm* c) {
  if (!c) return 0;
  int before = -1;
  BCOM_TRY(cudaGetDevice(&before));
  if (before != c->device) BCOM_TRY(cudaSetDevice(c->device));
  cudaError_t err = cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank) continue;
    if (c->opened[p] && c->peer[p]) {
      const cudaError_t e = cudaIpcCloseMemHandle(c->peer[p]);
      if (err == cudaSuccess) err = e;
    }
    c->opened[p] = false;
    c->peer[p] = nullptr;  // bcom_collective refuses a communicator with an unmapped peer
  }
  if (before != c->device) (void)cudaSetDevice(before);
  return (int)err;
}

int bcom_comm_destroy(BcomComm* c) {
  if (!c) return 0;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (p != c->rank && c->opened[p] && c->peer[p]) cudaIpcCloseMemHandle(c->peer[p]);
  if (c->local && c->owns_local) cudaFree(c->local);
  if (c->status_host) cudaFreeHost(c->status_host);
  delete c;
  return 0;
}

int bcom_comm_check_canaries(BcomComm* c, long long* first_bad) {
  if (!c || !first_bad) return (int)cudaErrorInvalidValue;
  *first_bad = -1;
  int before = -1;
  BCOM_TRY(cudaGetDevice(&before));
  if (before != c->device) BCOM_TRY(cudaSetDevice(c->device));
  const size_t head = BCOM_CONTROL_BYTES - BCOM_CTL_CANARY;
  const size_t tail_off = BCOM_CONTROL_BYTES + 2 * c->region_bytes;
  std::vector<unsigned char> host(head + BCOM_GUARD_BYTES);
  cudaError_t err = cudaDeviceSynchronize();
  if (err == cudaSuccess)
    err = cudaMemcpy(host.data(), c->local + BCOM_CTL_CANARY, head, cudaMemcpyDeviceToHost);
  if (err == cudaSuccess)
    err = cudaMemcpy(host.data() + head, c->local + tail_off, BCOM_GUARD_BYTES,
                     cudaMemcpyDeviceToHost);
  if (before != c->device) (void)cudaSetDevice(before);
  if (err != cudaSuccess) return (int)err;
  for (size_t i = 0; i < host.size(); ++i) {
    if (host[i] != BCOM_CANARY_BYTE) {
      *first_bad = (long long)(i < head ? BCOM_CTL_CANARY + i : tail_off + (i - head));
      break;
    }
  }
  return 0;
}

int bcom_comm_ipc_handle(BcomComm* c, void* handle_out) {
  static_assert(sizeof(cudaIpcMemHandle_t) == BCOM_IPC_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  BCOM_TRY(cudaIpcGetMemHandle(&h, c->local));
  std::memcpy(handle_out, &h, sizeof(h));
  return 0;
}

int bcom_comm_open_peers(BcomComm* c, const void* handles) {
  const unsigned char* hs = (const unsigned char*)handles;
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, hs + (size_t)p * BCOM_IPC_HANDLE_BYTES, sizeof(h));
    void* base = nullptr;
    BCOM_TRY(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer[p] = (unsigned char*)base;
    c->opened[p] = true;
  }
  return 0;
}

int bcom_comm_set_peer(BcomComm* c, int peer, void* base) {
  if (peer < 0 || peer >= c->world) return (int)cudaErrorInvalidValue;
  c->peer[peer] = (unsigned char*)base;
  c->opened[peer] = false;
  return 0;
}

void* bcom_comm_local_base(BcomComm* c) { return c->local; }
size_t bcom_comm_region_bytes(BcomComm* c) { return c->region_bytes; }
unsigned long long bcom_comm_epoch(BcomComm* c) { return c->epoch; }

int bcom_comm_set_timeout_ms(BcomComm* c, double ms) {
  if (ms <= 0) return (int)cudaErrorInvalidValue;
  c->timeout_ns = (unsigned long long)(ms * 1.0e6);
  return 0;
}

int bcom_comm_set_ll_max_bytes(BcomComm* c, long long bytes) {
  if (bytes < 0) return (int)cudaErrorInvalidValue;
  c->ll_max_payload = bytes;
  return 0;
}

int bcom_comm_status(BcomComm* c, unsigned int out[8]) {
  for (int i = 0; i < 8; ++i) out[i] = ((volatile unsigned int*)c->status_host)[i];
  return 0;
}

// Device time stamps (ns, %globaltimer) the first CTA of the last kernel took at its phase
// boundaries: [0] entry, [1] phase-1 loop done, [2] all phase-1 flags seen, [3] phase-2 loop
// done, [4] all phase-2 flags seen, [5] phase-3 loop done.  Valid once that kernel has finished.
int bcom_comm_phase_times(BcomComm* c, unsigned long long out[6]) {
  const volatile unsigned long long* t =
      reinterpret_cast<const volatile unsigned long long*>(c->status_host + BCOM_STATUS_TIMES);
  for (int i = 0; i < 6; ++i) out[i] = t[i];
  return 0;
}

// Host address of the 8-word status record (pinned, written by the kernels): lets a caller
// poll status[0] without a library call.
void* bcom_comm_status_host(BcomComm* c) { return c->status_host; }

int bcom_comm_reset(BcomComm* c, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  BCOM_TRY(cudaStreamSynchronize(st));
  std::memset(c->status_host, 0, BCOM_STATUS_WORDS * sizeof(unsigned int));
  BCOM_TRY(cudaMemsetAsync(c->local + BCOM_CTL_ARRIVE1, 0, 16, st));
  BCOM_TRY(cudaStreamSynchronize(st));
  return 0;
}

}  // extern "C"
