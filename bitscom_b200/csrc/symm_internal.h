// Internal layout shared by symm.cu (host runtime) and fused_collectives.cu (kernels).
#pragma once

#include <cuda_runtime.h>

#include "symm.h"

struct BcomComm {
  int rank;
  int world;
  int device;
  size_t region_bytes;      // bytes of each of the two data regions
  size_t total_bytes;
  unsigned char* local;     // this rank's block
  unsigned char* mc;        // NVLink multicast mapping of the block (all ranks), or null
  bool owns_local;          // the block was allocated by bcom_comm_create (else: adopted)
  unsigned char* peer[BCOM_MAX_WORLD];
  bool opened[BCOM_MAX_WORLD];  // peer mapping came from cudaIpcOpenMemHandle
  unsigned int* status_host;    // pinned, mapped
  unsigned int* status_dev;
  unsigned long long epoch;     // collective launches so far (same on every rank)
  unsigned long long timeout_ns;
  int sm_count;
  size_t ll_bytes;              // tail of each data region kept for flag-in-data launches
  long long ll_max_payload;     // largest tensor (bytes) that takes that path; 0 = never
};

// control page layout (byte offsets inside the block)
#define BCOM_CTL_FLAG1 0      // u64[BCOM_MAX_WORLD]: peer p finished pushing phase-1 data
#define BCOM_CTL_FLAG2 128    // u64[BCOM_MAX_WORLD]: peer p finished pushing phase-2 data
#define BCOM_CTL_ARRIVE1 256  // u32: CTAs of this rank that finished phase 1
#define BCOM_CTL_ARRIVE2 264  // u32: CTAs of this rank that finished phase 2
#define BCOM_CTL_CANARY 512   // from here to the end of the page: canary bytes

static inline size_t bcom_align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
