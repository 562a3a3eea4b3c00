// Host model of the barrier protocol of the CTA-pair GEMM (csrc/gemm_tcgen05_2cta.cu), run by
// tests/test_gemm_pair_model.py.
//
// Threads: per CTA of the pair a TMA producer and four epilogue warps; the leader's MMA issuer;
// one tensor pipe that executes the issued MMAs and commits in order; one copy engine per CTA
// that completes loads after a random delay.  Both CTAs' loads of a stage complete on the
// LEADER's "stage full" barrier, which the leader's producer arms for the bytes of both (modelled
// as three arrivals: the arming and one per CTA's bytes).  mbarriers carry an arrival count and
// a phase, waits are parity waits, ring stages and accumulator buffers carry a tag (which
// k-block / which tile they hold) and a count of asynchronous readers.
//
//   -DBUG=1  the leader's barrier counts its own CTA's bytes only            (must be detected)
//   -DBUG=2  the accumulator hand-back barrier counts one CTA's warps only   (must be detected)
//   -DBUG=3  the stage-release commit reaches the leader only                (must be detected)
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <functional>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

#ifndef BUG
#define BUG 0
#endif

constexpr int STAGES = 6;

static std::atomic<int> violations{0};
static void fail(const char* what, long long id) {
  if (violations.fetch_add(1) == 0) std::fprintf(stderr, "violation: %s (%lld)\n", what, id);
}
// a wait that ran out: the protocol is stuck, the other threads would follow one by one
[[noreturn]] static void die(const char* what, long long id) {
  std::fprintf(stderr, "violation: timeout: %s (%lld)\n", what, id);
  std::fflush(stderr);
  std::_Exit(3);
}

struct MBar {
  std::mutex mu;
  std::condition_variable cv;
  int count = 1, pending = 1;
  unsigned long long phase = 0;
  void init(int c) { count = pending = c; }
  void arrive() {
    std::lock_guard<std::mutex> lk(mu);
    if (--pending == 0) {
      pending = count;
      ++phase;
      cv.notify_all();
    }
  }
  bool wait(unsigned parity) {
    std::unique_lock<std::mutex> lk(mu);
    return cv.wait_for(lk, std::chrono::seconds(3), [&] { return (phase & 1u) != parity; });
  }
};

struct Work {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void()>> q;
  bool stop = false;
  void push(std::function<void()> f) {
    std::lock_guard<std::mutex> lk(mu);
    q.push_back(std::move(f));
    cv.notify_one();
  }
  void run() {
    for (;;) {
      std::function<void()> f;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop || !q.empty(); });
        if (q.empty()) return;
        f = std::move(q.front());
        q.pop_front();
      }
      f();
    }
  }
  void finish() {
    std::lock_guard<std::mutex> lk(mu);
    stop = true;
    cv.notify_all();
  }
};

static void nap(std::mt19937& rng, int max_us) {
  const int us = (int)(rng() % (unsigned)(max_us + 1));
  if (us) std::this_thread::sleep_for(std::chrono::microseconds(us));
}

struct Pair {
  int tiles, num_kb;
  // per CTA
  MBar empty[2][STAGES], acc_full[2][2];
  // leader only
  MBar full[STAGES], acc_empty[2];
  std::atomic<long long> stage_tag[2][STAGES];  // global k-block index held by the stage
  std::atomic<int> stage_readers[STAGES];       // MMAs reading the stage (in both CTAs)
  std::atomic<long long> acc_tag[2];            // tile whose sum the buffer holds
  std::atomic<int> acc_kb[2];                   // k-blocks accumulated into the buffer
  std::atomic<int> acc_readers[2];              // epilogue warps (of both CTAs) draining it
  std::atomic<int> tiles_stored{0};
  std::atomic<int> tail_done[2];                // the CTA's producer has seen every release
  Work tensor, copy[2];

  Pair(int t, int k) : tiles(t), num_kb(k) {
    for (int c = 0; c < 2; ++c)
      for (int s = 0; s < STAGES; ++s) { empty[c][s].init(1); stage_tag[c][s] = -1; }
    for (int s = 0; s < STAGES; ++s) {
#if BUG == 1
      full[s].init(2);
#else
      full[s].init(3);
#endif
      stage_readers[s] = 0;
    }
    for (int b = 0; b < 2; ++b) {
      acc_full[0][b].init(1); acc_full[1][b].init(1);
#if BUG == 2
      acc_empty[b].init(4);
#else
      acc_empty[b].init(8);
#endif
      acc_tag[b] = -1; acc_kb[b] = 0; acc_readers[b] = 0;
    }
    tail_done[0] = tail_done[1] = 0;
  }

  void producer(int c) {
    std::mt19937 rng(100u + (unsigned)c);
    int stage = 0; unsigned phase = 0; long long id = 0;
    for (int t = 0; t < tiles; ++t)
      for (int kb = 0; kb < num_kb; ++kb, ++id) {
        if (!empty[c][stage].wait(phase ^ 1u)) die("producer: stage never released", id);
        const int s = stage; const long long my = id; const unsigned seed = (unsigned)(id * 2 + c);
        if (c == 0) full[s].arrive();  // the leader arms its barrier for the bytes of both CTAs
        copy[c].push([this, c, s, my, seed] {
          std::mt19937 r(seed);
          nap(r, c == 1 ? 240 : 120);  // the odd CTA's bytes travel further
          if (stage_readers[s] != 0) fail("stage overwritten while MMAs were reading it", my);
          stage_tag[c][s] = my;
#if BUG == 1
          if (c == 0)
#endif
          full[s].arrive();  // complete_tx on the LEADER's barrier, from either CTA
        });
        nap(rng, 10);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    // producer tail: every stage's last fill has been released before this CTA may leave
    for (int i = 0; i < STAGES; ++i) {
      if (!empty[c][stage].wait(phase ^ 1u)) die("producer tail: stage never released", id);
      if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
    tail_done[c] = 1;
  }

  void issuer() {
    std::mt19937 rng(7u);
    int stage = 0; unsigned phase = 0; long long id = 0;
    for (int t = 0; t < tiles; ++t) {
      const int buf = t & 1;
      const unsigned acc_phase = (unsigned)(t >> 1) & 1u;
      if (!acc_empty[buf].wait(acc_phase ^ 1u)) die("issuer: accumulator never handed back", t);
      for (int kb = 0; kb < num_kb; ++kb, ++id) {
        if (!full[stage].wait(phase)) die("issuer: stage never landed", id);
        const int s = stage; const long long my = id; const int first = kb == 0; const int tile = t;
        tensor.push([this, s, my, buf, first, tile] {  // the four MMAs of the k-block
          ++stage_readers[s];
          if (stage_tag[0][s] != my) fail("MMA read a leader stage that holds another k-block", my);
          if (stage_tag[1][s] != my) fail("MMA read a peer stage that holds another k-block", my);
          if (acc_readers[buf] != 0) fail("MMA wrote an accumulator that was being drained", my);
          std::this_thread::sleep_for(std::chrono::microseconds(8));
          if (stage_tag[0][s] != my || stage_tag[1][s] != my) fail("stage changed under the MMAs", my);
          if (first) { acc_kb[buf] = 0; acc_tag[buf] = tile; }
          acc_kb[buf].fetch_add(1);
          --stage_readers[s];
        });
        tensor.push([this, s] {  // commit -> empty[stage] in the CTAs of the mask
          if (tail_done[0] || tail_done[1]) fail("a stage release arrived after its CTA left", s);
          empty[0][s].arrive();
#if BUG != 3
          empty[1][s].arrive();
#endif
        });
        nap(rng, 5);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      tensor.push([this, buf] { acc_full[0][buf].arrive(); acc_full[1][buf].arrive(); });
    }
  }

  void epilogue(int c, int w) {
    std::mt19937 rng(900u + (unsigned)(c * 4 + w));
    for (int t = 0; t < tiles; ++t) {
      const int buf = t & 1;
      const unsigned acc_phase = (unsigned)(t >> 1) & 1u;
      if (!acc_full[c][buf].wait(acc_phase)) die("epilogue: accumulator never completed", t);
      ++acc_readers[buf];
      if (acc_tag[buf] != t) fail("epilogue drained an accumulator of another tile", t);
      if (acc_kb[buf] != num_kb) fail("epilogue drained an incomplete accumulator", t);
      nap(rng, 60);
      if (acc_tag[buf] != t || acc_kb[buf] != num_kb) fail("accumulator changed while it was drained", t);
      --acc_readers[buf];
      if (c == 0 && w == 0) tiles_stored.fetch_add(1);
      acc_empty[buf].arrive();  // local arrive in the leader, remote arrive from the odd CTA
    }
  }

  void run() {
    std::thread tp([this] { tensor.run(); }), c0([this] { copy[0].run(); }), c1([this] { copy[1].run(); });
    std::vector<std::thread> th;
    for (int c = 0; c < 2; ++c) {
      th.emplace_back([this, c] { producer(c); });
      for (int w = 0; w < 4; ++w) th.emplace_back([this, c, w] { epilogue(c, w); });
    }
    th.emplace_back([this] { issuer(); });
    for (auto& t : th) t.join();
    tensor.finish(); copy[0].finish(); copy[1].finish();
    tp.join(); c0.join(); c1.join();
    if (violations.load() == 0 && tiles_stored != tiles) fail("not every tile was stored", tiles);
  }
};

int main() {
  const int shapes[][2] = {{1, 1}, {1, 3}, {2, 6}, {3, 7}, {5, 13}, {8, 2}, {4, 64}};
  for (int rep = 0; rep < 4 && violations.load() == 0; ++rep)
    for (auto& s : shapes) {
      Pair p(s[0], s[1]);
      p.run();
      if (violations.load()) break;
    }
  if (violations.load()) return 3;
  std::printf("ok: cta pair\n");
  return 0;
}
