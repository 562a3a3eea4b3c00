// Host model of the small-bucket form of the fused all-reduce (csrc/fused_collectives.cu:
// run_rank_ll): every word travels as an 8-byte pair {payload, epoch} written with ONE store,
// consumers poll the pair they need until its epoch is this launch's, and there is no fence,
// no arrival counter and no flag array.  Run by tests/test_ll_protocol_model.py.
//
// W ranks x C CTAs are threads, G groups per shard.  A pair is a relaxed 64-bit atomic: what
// the GPU guarantees for an aligned 8-byte store is that it is performed as a whole, nothing
// about its order against other stores, and relaxed atomics give exactly that.  The payload
// encodes (phase, epoch, source, destination, group), so a pair that is accepted with the
// wrong content is caught by value; a pair that was overwritten by a later launch before its
// consumer read it is caught because the consumer then never sees its epoch (bounded wait).
// Launches follow each other back to back with no barrier between ranks; only the CTAs of one
// rank are joined between two launches (stream order on one GPU).
//
// What the model checks is the claim that slots may be reused by the next launch without a
// barrier: a rank enters launch k + 1 only after its phase 3 of launch k has seen every peer's
// reduced shard, which a peer produces only after it has read what it needed from its receive
// slots; and phase-2 stores of launch k + 1 wait for every peer's phase-1 words of launch k + 1.
//
// -DBUG=1  phase 3 does not wait for the peers' pairs (a rank can run a launch ahead and
//          overwrite receive slots that a slow peer has not read)          (must be detected)
// -DBUG=2  every launch uses the same epoch (a stale pair is accepted)      (must be detected)
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <random>
#include <thread>
#include <vector>

#ifndef BUG
#define BUG 0
#endif

constexpr int W = 4;    // ranks
constexpr int C = 3;    // CTAs per rank
constexpr int G = 12;   // groups per shard
constexpr int K = 300;  // launches, back to back

struct Rank {
  std::atomic<uint64_t> recv[W][G];    // recv[source][group]: phase-1 pairs from `source`
  std::atomic<uint64_t> gather[W][G];  // gather[owner][group]: phase-2 pairs from `owner`
};
static Rank ranks[W];
static std::atomic<int> violations{0};

static uint32_t payload(int phase, uint32_t launch, int src, int dst, int g) {
  return ((((uint32_t)phase * 1024u + (launch & 1023u)) * 8u + (uint32_t)src) * 8u + (uint32_t)dst) * 16u +
         (uint32_t)g;
}
static uint64_t make_pair(uint32_t data, uint32_t epoch) { return ((uint64_t)epoch << 32) | data; }

static void fail(const char* what, int rank, int cta, uint32_t launch) {
  if (violations.fetch_add(1) == 0)
    std::fprintf(stderr, "protocol violation: %s (rank %d cta %d launch %u)\n", what, rank, cta, launch);
}

static void jitter(std::mt19937& rng) {
  const unsigned r = rng() & 63u;
  if (r == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() & 255u));
  else if (r < 8) std::this_thread::yield();
}

// polls one pair; false when the epoch never shows up
static bool poll(std::atomic<uint64_t>& slot, uint32_t epoch, uint32_t* data) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    const uint64_t v = slot.load(std::memory_order_relaxed);
    if ((uint32_t)(v >> 32) == epoch) {
      *data = (uint32_t)v;
      return true;
    }
    std::this_thread::yield();
    if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(5)) return false;
  }
}

static void cta_body(int r, int c, uint32_t launch, unsigned seed) {
  std::mt19937 rng(seed);
#if BUG == 2
  const uint32_t epoch = 1;
#else
  const uint32_t epoch = launch;
#endif
  // phase 1: this CTA's groups of every destination's shard
  for (int k = 0; k < W; ++k) {
    const int j = (r + k) % W;
    for (int g = c; g < G; g += C) {
      ranks[j].recv[r][g].store(make_pair(payload(1, launch, r, j, g), epoch), std::memory_order_relaxed);
      jitter(rng);
    }
  }
  // phase 2: this CTA's groups of the own shard: wait for every source, then send to everybody
  for (int g = c; g < G; g += C) {
    for (int s = 0; s < W; ++s) {
      uint32_t data;
      if (!poll(ranks[r].recv[s][g], epoch, &data))
        return fail("a phase-1 pair never arrived (overwritten before it was read?)", r, c, launch);
      if (data != payload(1, launch, s, r, g)) return fail("stale phase-1 pair accepted", r, c, launch);
    }
    jitter(rng);
    for (int k = 0; k < W; ++k) {
      const int t = (r + k) % W;
      ranks[t].gather[r][g].store(make_pair(payload(2, launch, r, t, g), epoch), std::memory_order_relaxed);
    }
  }
  // phase 3: this CTA's groups of every owner's reduced shard
#if BUG != 1
  for (int k = 0; k < W; ++k) {
    const int j = (r + k) % W;
    for (int g = c; g < G; g += C) {
      uint32_t data;
      if (!poll(ranks[r].gather[j][g], epoch, &data))
        return fail("a phase-2 pair never arrived", r, c, launch);
      if (data != payload(2, launch, j, r, g)) return fail("stale phase-2 pair accepted", r, c, launch);
      jitter(rng);
    }
  }
#endif
}

static void rank_body(int r) {
  for (uint32_t launch = 1; launch <= (uint32_t)K && violations.load() == 0; ++launch) {
    std::vector<std::thread> ctas;
    for (int c = 0; c < C; ++c)
      ctas.emplace_back(cta_body, r, c, launch, (unsigned)(launch * 977u + r * 31u + c));
    for (auto& t : ctas) t.join();  // stream order: the next launch starts after this one
#if BUG == 1
    // make the fast ranks fast and the last rank slow, so that running ahead shows quickly
    if (r == W - 1) std::this_thread::sleep_for(std::chrono::microseconds(300));
#endif
  }
}

int main() {
  for (auto& rk : ranks)
    for (int s = 0; s < W; ++s)
      for (int g = 0; g < G; ++g) {
        rk.recv[s][g].store(0);    // zeros at creation; epoch 0 is never used
        rk.gather[s][g].store(0);
      }
  std::vector<std::thread> threads;
  for (int r = 0; r < W; ++r) threads.emplace_back(rank_body, r);
  for (auto& t : threads) t.join();
  if (violations.load()) return 3;
  std::printf("ok: %d ranks x %d CTAs x %d groups x %d launches\n", W, C, G, K);
  return 0;
}
