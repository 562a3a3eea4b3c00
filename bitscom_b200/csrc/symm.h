// Symmetric-memory communicator and fused low-bit collectives: C API.
//
// One communicator per (process group, device).  Every rank allocates one block of
// device memory with the same layout
//
//     [ control 4 KiB | receive region | gather region | guard 4 KiB ]
//
// (the unused tail of the control page and the guard page hold a fixed byte pattern that no
// kernel may touch; bcom_comm_check_canaries verifies it, see below)
// and maps every peer's block (CUDA IPC between processes of one NVSwitch domain).
// The fused kernel pushes packed shards into the *destination's* regions with plain
// peer stores, so a consumer only ever reads its own HBM; cross-GPU ordering uses
// monotonically increasing 64-bit epoch flags in the control page
// (st.release.sys / ld.acquire.sys), never reset, and every wait is bounded.
//
// This replaces the reference's private NCCL communicator with grouped
// ncclSend/ncclRecv (cpp/src/process_group_lowbit.cc:543-575,776-835,1179-1239).
#pragma once

#include <stddef.h>
#include <stdint.h>

#define BCOM_MAX_WORLD 16
#define BCOM_CONTROL_BYTES 4096
#define BCOM_GUARD_BYTES 4096
#define BCOM_CANARY_BYTE 0xA5
#define BCOM_IPC_HANDLE_BYTES 64
// host-mapped status record: words 0-7 error record, words 8-19 six 64-bit phase time stamps
#define BCOM_STATUS_WORDS 32
#define BCOM_STATUS_TIMES 8

#ifdef __cplusplus
extern "C" {
#endif

typedef struct BcomComm BcomComm;

// kernel status codes (status[0]); 0 = ok
enum {
  BCOM_OK = 0,
  BCOM_TIMEOUT_PHASE1_FLAGS = 1,  // a peer never announced its packed shards
  BCOM_TIMEOUT_PHASE2_FLAGS = 2,  // a peer never announced its reduced shard
};

enum { BCOM_MODE_ALL_REDUCE = 0, BCOM_MODE_REDUCE_SCATTER = 1, BCOM_MODE_ALL_GATHER = 2 };

// One collective on one rank.  For all modes S is the shard length and the logical
// full tensor has n <= world * S elements:
//   all-reduce      in/out: [n]            res1: [world*S] or null   res2: [S] or null
//   reduce-scatter  in: [world*S] out: [S] res1: [world*S] or null
//   all-gather      in: [S] out: [world*S] res2: [S] or null
typedef struct {
  const void* in;
  void* out;
  float* res1;
  float* res2;
  long long n;
  long long S;
  int dtype;       // 0 fp32, 1 fp16, 2 bf16
  int bits;        // 1, 2, 4, 8, 12
  int block;       // 8 * power of two, <= 256
  int mode;        // BCOM_MODE_*
  int stochastic;  // 0 nearest, 1 stochastic rounding
  unsigned int key1;  // stage-1 random key
  unsigned int key2;  // stage-2 random key
  float post_scale;   // applied to the result after the cast to dtype
  int max_ctas;       // 0 = library default
  int reserved;
} BcomCollArgs;

int bcom_comm_create(int rank, int world, size_t region_bytes, BcomComm** out);
// Adopt blocks that somebody else allocated and mapped (for example torch symmetric memory):
// bases[p] is rank p's block as mapped into this process (bases[rank] the local one), each
// bcom_comm_block_bytes(region_bytes) long; mc_base is the NVLink multicast mapping of the
// same blocks (a store through it lands in every rank's block) or NULL.  The caller keeps
// ownership of the memory, and all ranks must pass a barrier between this call (which zeroes
// the local control page) and the first collective.  With a multicast mapping the 4- and
// 8-bit all-gather half sends each packed group with one multimem store instead of one store
// per peer.
int bcom_comm_create_external(int rank, int world, size_t region_bytes, void* const* bases,
                              void* mc_base, BcomComm** out);
size_t bcom_comm_block_bytes(size_t region_bytes);
void* bcom_comm_multicast_base(BcomComm* comm);
// Orderly teardown is two steps with a barrier among the ranks after each:
//   1. every rank waits for its own kernels (nobody stores into a peer any more) -> barrier ->
//      bcom_comm_close_peers (unmaps the peers' blocks; the communicator can no longer launch)
//   2. barrier (nobody maps this rank's block any more) -> bcom_comm_destroy (frees it).
// Freeing a block that a peer still has mapped is undefined; bcom_comm_destroy alone is for a
// rank whose peers are gone or have already unmapped it.
int bcom_comm_close_peers(BcomComm* comm);
int bcom_comm_destroy(BcomComm* comm);
// Debugging aid for tests: synchronises the device and checks the canary bytes around this
// rank's regions (control-page tail in front of the receive region, guard page behind the
// gather region).  A store that missed its slot, from this rank's kernels or from a peer's
// pushes, shows up here.  Returns 0 and *first_bad = -1 when intact; otherwise 0 with the
// byte offset (inside the block) of the first damaged byte; a CUDA error code on failure.
int bcom_comm_check_canaries(BcomComm* comm, long long* first_bad);
// 64-byte CUDA IPC handle of this rank's block
int bcom_comm_ipc_handle(BcomComm* comm, void* handle_out);
// handles: world * 64 bytes, in rank order (own entry ignored)
int bcom_comm_open_peers(BcomComm* comm, const void* handles);
// wire a peer by address (same-process emulation, or memory mapped by other means)
int bcom_comm_set_peer(BcomComm* comm, int peer, void* base);
void* bcom_comm_local_base(BcomComm* comm);
size_t bcom_comm_region_bytes(BcomComm* comm);
// largest shard chunk (elements) one launch can carry for this codec setting
long long bcom_comm_max_chunk(BcomComm* comm, int bits, int block);
// copies the 8-word status record; status[0] != 0 means the last kernels gave up
int bcom_comm_status(BcomComm* comm, unsigned int out[8]);
// time stamps (ns) of the phase boundaries of the last kernel's first CTA: entry, phase-1 loop
// done, phase-1 flags seen, phase-2 loop done, phase-2 flags seen, phase-3 loop done
int bcom_comm_phase_times(BcomComm* comm, unsigned long long out[6]);
// host address of that record (pinned memory the kernels write), for polling without a call
void* bcom_comm_status_host(BcomComm* comm);
// clears status, flags stay; zeroes the local arrival counters (after an error)
int bcom_comm_reset(BcomComm* comm, void* stream);
int bcom_comm_set_timeout_ms(BcomComm* comm, double ms);
// Largest all-reduce that runs as ONE pass with the flags inside the data words (see
// fused_collectives.cu, "small buckets"), in bytes counted at four per element whatever the
// dtype; 0 switches that path off.  Default 64 MiB = 16 Mi elements (the slots must also fit the
// tail of the regions that is kept for them: an eighth of each).
int bcom_comm_set_ll_max_bytes(BcomComm* comm, long long bytes);
unsigned long long bcom_comm_epoch(BcomComm* comm);

// Launch the fused kernel(s) for one collective on this rank (one launch per chunk).
int bcom_collective(BcomComm* comm, const BcomCollArgs* args, void* stream);
// All ranks of a same-device emulation in one cooperative launch per chunk.
int bcom_collective_emulated(BcomComm** comms, const BcomCollArgs* args, int world,
                             void* stream);
// 1 if (dtype, bits, block) is covered by the fused kernel
int bcom_collective_supported(int dtype, int bits, int block);

#ifdef __cplusplus
}
#endif
