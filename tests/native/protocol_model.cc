// Host model of the fused collective's synchronisation protocol (csrc/fused_collectives.cu:
// arrive_and_publish / wait_flags and the three phases around them), run by
// tests/test_protocol_model.py under ThreadSanitizer.
//
// W ranks x C CTAs are threads.  Per rank there is a control block (two arrays of epoch
// flags, two arrival counters) and two data regions (receive slots, gather slots), exactly
// the roles of the symmetric block.  The data regions are PLAIN memory, so ThreadSanitizer
// checks that every read of a slot is ordered after the peer's write by the flag protocol
// alone; the payload of every slot encodes (epoch, source, destination, cta), so a stale or
// early read is also caught by value.  Calls follow each other back to back without any
// barrier between ranks; only the CTAs of one rank are joined between two calls, which is
// what stream order gives the kernels of one GPU.
//
// The device code orders its stores with __threadfence_system() followed by a relaxed
// atomicAdd; the model uses acq_rel read-modify-writes instead (the sanitizer does not follow
// stand-alone fences), which is not stronger than what the fence gives.
//
// -DBUG=1  publish the epoch before re-arming the other counter   (must be detected)
// -DBUG=2  do not wait for the phase-2 flags before reading       (must be detected)
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#ifndef BUG
#define BUG 0
#endif

constexpr int W = 4;   // ranks
constexpr int C = 3;   // CTAs per rank
constexpr int K = 200; // collectives, back to back

struct Control {
  std::atomic<uint64_t> flag1[W], flag2[W];
  std::atomic<uint32_t> arrive1, arrive2;
};
struct Rank {
  Control ctl;
  uint64_t recv[W][C];    // recv[source][cta]: written by the source's CTAs in phase 1
  uint64_t gather[W][C];  // gather[source][cta]: written by the source's CTAs in phase 2
};

static Rank ranks[W];
static std::atomic<int> violations{0};

static uint64_t enc(int phase, uint64_t epoch, int src, int dst, int cta) {
  return (((epoch * 8 + phase) * 64 + src) * 64 + dst) * 64 + cta;
}

static void fail(const char* what, int rank, int cta, uint64_t epoch) {
  if (violations.fetch_add(1) == 0)
    std::fprintf(stderr, "protocol violation: %s (rank %d cta %d epoch %llu)\n", what, rank, cta,
                 (unsigned long long)epoch);
}

static void jitter(std::mt19937& rng) {
  const unsigned r = rng() & 63u;
  if (r == 0) std::this_thread::sleep_for(std::chrono::microseconds(rng() & 127u));
  else if (r < 8) std::this_thread::yield();
}

// returns false if the counter overflowed (an increment met a counter that was not re-armed)
static bool arrive_and_publish(int r, uint64_t epoch, bool phase1) {
  Control& ctl = ranks[r].ctl;
  std::atomic<uint32_t>& ctr = phase1 ? ctl.arrive1 : ctl.arrive2;
  std::atomic<uint32_t>& other = phase1 ? ctl.arrive2 : ctl.arrive1;
  const uint32_t seen = ctr.fetch_add(1, std::memory_order_acq_rel);
  if (seen >= (uint32_t)C) return false;
  if (seen + 1 == (uint32_t)C) {
#if BUG == 1
    for (int t = 0; t < W; ++t)
      (phase1 ? ranks[t].ctl.flag1 : ranks[t].ctl.flag2)[r].store(epoch, std::memory_order_release);
    std::this_thread::yield();
    other.store(0, std::memory_order_relaxed);
#else
    other.store(0, std::memory_order_relaxed);
    for (int t = 0; t < W; ++t)
      (phase1 ? ranks[t].ctl.flag1 : ranks[t].ctl.flag2)[r].store(epoch, std::memory_order_release);
#endif
  }
  return true;
}

static bool wait_flags(int r, uint64_t epoch, bool phase1) {
  const auto t0 = std::chrono::steady_clock::now();
  for (int s = 0; s < W; ++s) {
    std::atomic<uint64_t>& f = (phase1 ? ranks[r].ctl.flag1 : ranks[r].ctl.flag2)[s];
    while (f.load(std::memory_order_acquire) < epoch) {
      std::this_thread::yield();
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) return false;
    }
  }
  return true;
}

static void cta_body(int r, int c, uint64_t epoch, unsigned seed) {
  std::mt19937 rng(seed);
  // phase 1: push one value into every destination's receive slot
  for (int k = 0; k < W; ++k) {
    const int j = (r + k) % W;
    ranks[j].recv[r][c] = enc(1, epoch, r, j, c);
    jitter(rng);
  }
  if (!arrive_and_publish(r, epoch, true)) return fail("phase-1 counter not re-armed", r, c, epoch);
  if (!wait_flags(r, epoch, true)) return fail("phase-1 flags never arrived", r, c, epoch);
  // phase 2: read what every source sent to this rank, push the result to every gather slot
  for (int s = 0; s < W; ++s)
    for (int cc = 0; cc < C; ++cc)
      if (ranks[r].recv[s][cc] != enc(1, epoch, s, r, cc))
        return fail("stale or early receive slot", r, c, epoch);
  jitter(rng);
  for (int k = 0; k < W; ++k) {
    const int t = (r + k) % W;
    ranks[t].gather[r][c] = enc(2, epoch, r, t, c);
    jitter(rng);
  }
  if (!arrive_and_publish(r, epoch, false)) return fail("phase-2 counter not re-armed", r, c, epoch);
#if BUG != 2
  if (!wait_flags(r, epoch, false)) return fail("phase-2 flags never arrived", r, c, epoch);
#endif
  // phase 3: read every rank's contribution from the local gather slots
  for (int j = 0; j < W; ++j)
    for (int cc = 0; cc < C; ++cc)
      if (ranks[r].gather[j][cc] != enc(2, epoch, j, r, cc))
        return fail("stale or early gather slot", r, c, epoch);
}

static void rank_body(int r) {
  for (uint64_t epoch = 1; epoch <= (uint64_t)K && violations.load() == 0; ++epoch) {
    std::vector<std::thread> ctas;
    for (int c = 0; c < C; ++c)
      ctas.emplace_back(cta_body, r, c, epoch, (unsigned)(epoch * 977 + r * 31 + c));
    for (auto& t : ctas) t.join();  // stream order: the next kernel starts after this one
  }
}

int main() {
  for (auto& rk : ranks) {
    for (int i = 0; i < W; ++i) {
      rk.ctl.flag1[i].store(0);
      rk.ctl.flag2[i].store(0);
    }
    rk.ctl.arrive1.store(0);
    rk.ctl.arrive2.store(0);
  }
  std::vector<std::thread> threads;
  for (int r = 0; r < W; ++r) threads.emplace_back(rank_body, r);
  for (auto& t : threads) t.join();
  if (violations.load()) return 3;
  std::printf("ok: %d ranks x %d CTAs x %d collectives\n", W, C, K);
  return 0;
}
