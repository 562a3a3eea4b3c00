// Host model of the barrier protocol of the attention backward kernel's query-block loop
// (csrc/attention_tcgen05.cu: attention_bwd_kernel with dQ accumulated by TMA reductions),
// run by tests/test_attention_pipeline_model.py.
//
// Threads: NT CTA threads (thread 0 is the one that issues MMAs and copies), one tensor pipe
// that executes the issued MMAs in order, one copy engine that completes TMA loads and
// reductions after a random delay.  mbarriers are phase counters with parity waits, the CTA
// barrier is a reusable barrier, and bulk-group waits count outstanding reductions, as in the
// kernel.  Every buffer carries a tag saying which query block its content belongs to and a
// count of asynchronous readers; a writer that finds a reader, or a reader that finds the
// wrong tag, is a violation.
//
//   -DEARLY=0 | 1   when the next Q / dO tiles are requested: after the whole second MMA
//                   group (bar_2), or as soon as dV and dK are done (bar_2a)
//   -DBUG=1  EARLY without the wait on bar_2a                                (must be detected)
//   -DBUG=2  no wait for the previous reductions to have read the staging tile (must be detected)
//   -DBUG=3  the reductions are issued without the CTA barrier after staging  (must be detected)
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

#ifndef EARLY
#define EARLY 0
#endif
#ifndef BUG
#define BUG 0
#endif

constexpr int NT = 4;  // CTA threads in the model

static std::atomic<int> violations{0};
static void fail(const char* what, int qi) {
  if (violations.fetch_add(1) == 0) std::fprintf(stderr, "violation: %s (block %d)\n", what, qi);
}

// a failed wait: the other threads would block on the CTA barrier for ever, so stop here
[[noreturn]] static void die(const char* what, int qi) {
  std::fprintf(stderr, "violation: %s (block %d)\n", what, qi);
  std::fflush(stderr);
  std::_Exit(3);
}

struct MBar {
  std::mutex mu;
  std::condition_variable cv;
  unsigned long long phase = 0;
  void arrive() {
    std::lock_guard<std::mutex> lk(mu);
    ++phase;
    cv.notify_all();
  }
  bool wait(unsigned parity) {
    std::unique_lock<std::mutex> lk(mu);
    return cv.wait_for(lk, std::chrono::seconds(5), [&] { return (phase & 1u) != parity; });
  }
};

struct CtaBarrier {
  std::mutex mu;
  std::condition_variable cv;
  int waiting = 0;
  unsigned long long gen = 0;
  void sync() {
    std::unique_lock<std::mutex> lk(mu);
    const unsigned long long g = gen;
    if (++waiting == NT) {
      waiting = 0;
      ++gen;
      cv.notify_all();
    } else {
      cv.wait(lk, [&] { return gen != g; });
    }
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

struct Kernel {
  int nq;
  MBar bar_q, bar_1, bar_2, bar_2a;
  CtaBarrier cta;
  Work tensor, copy;
  std::atomic<int> q_tag{-1}, q_readers{0};      // the Q / dO tiles
  std::atomic<int> q_pending{0};                 // issued MMAs that read Q / dO, not yet complete
  std::atomic<int> st_tag{-1};                   // S^T / dP^T accumulators
  std::atomic<int> dq_tag{-1}, dq_readers{0};    // dQ accumulator
  std::atomic<int> kv_acc{0};                    // query blocks accumulated into dK / dV
  // P^T / dS^T tiles and the dQ staging tile share memory: slice t is written by thread t
  std::atomic<int> tile_tag[NT];                 // >= 0: P^T of block; <= -2: staging of -(tag+2)
  std::atomic<int> tile_readers{0};              // MMAs or reductions reading the tiles
  std::atomic<int> reductions_unread{0};         // committed reductions that have not read yet
  std::atomic<int> reduced{0};                   // query blocks added to global dQ

  explicit Kernel(int blocks) : nq(blocks) {
    for (auto& t : tile_tag) t = -1;
  }

  void load_q(int qi, unsigned seed) {
    // the copy may land at once, so every MMA that reads the tiles must be complete already
    if (q_pending != 0) fail("Q / dO requested while MMAs that read them were outstanding", qi);
    copy.push([this, qi, seed] {
      std::mt19937 rng(seed);
      nap(rng, 200);
      if (q_readers != 0) fail("Q / dO overwritten while an MMA was reading them", qi);
      q_tag = qi;
      bar_q.arrive();
    });
  }
  void issue_scores(int qi) {  // S^T = K Q^T, dP^T = V dO^T
    ++q_pending;
    tensor.push([this, qi] {
      ++q_readers;
      if (q_tag != qi) fail("scores read Q / dO of another block", qi);
      if (dq_readers != 0) fail("S^T written over dQ columns that are still being read", qi);
      std::this_thread::sleep_for(std::chrono::microseconds(15));
      if (q_tag != qi) fail("Q / dO changed under the score MMAs", qi);
      st_tag = qi;
      --q_readers; --q_pending;
      bar_1.arrive();
    });
  }
  void issue_dv_dk(int qi) {
    ++q_pending;
    tensor.push([this, qi] {
      ++q_readers; ++tile_readers;
      for (auto& t : tile_tag) if (t != qi) fail("dV / dK read a P^T slice of another block", qi);
      if (q_tag != qi) fail("dV / dK read Q / dO of another block", qi);
      std::this_thread::sleep_for(std::chrono::microseconds(25));
      if (q_tag != qi) fail("Q / dO changed under dV / dK", qi);
      kv_acc.fetch_add(1);
      --q_readers; --tile_readers; --q_pending;
#if EARLY
      bar_2a.arrive();
#endif
    });
  }
  void issue_dq(int qi) {
    tensor.push([this, qi] {
      ++tile_readers;
      for (auto& t : tile_tag) if (t != qi) fail("dQ read a dS^T slice of another block", qi);
      if (dq_readers != 0) fail("dQ accumulator overwritten while it was being drained", qi);
      std::this_thread::sleep_for(std::chrono::microseconds(40));
      for (auto& t : tile_tag) if (t != qi) fail("dS^T changed under the dQ MMAs", qi);
      dq_tag = qi;
      --tile_readers;
      bar_2.arrive();
    });
  }
  void issue_reduction(int qi, unsigned seed) {
    // the engine may read the tile at once
    for (auto& t : tile_tag)
      if (t != -(qi + 2)) fail("reduction issued before every staging slice was written", qi);
    ++reductions_unread;
    copy.push([this, qi, seed] {
      std::mt19937 rng(seed);
      nap(rng, 150);
      ++tile_readers;
      for (auto& t : tile_tag)
        if (t != -(qi + 2)) fail("reduction read a staging slice that is not this block's dQ", qi);
      nap(rng, 30);
      for (auto& t : tile_tag)
        if (t != -(qi + 2)) fail("staging tile changed under the reduction", qi);
      --tile_readers;
      --reductions_unread;
      reduced.fetch_add(1);
    });
  }
  bool wait_reductions_read() {
    for (int i = 0; i < 50000 && reductions_unread != 0; ++i)
      std::this_thread::sleep_for(std::chrono::microseconds(100));
    return reductions_unread == 0;
  }

  void thread(int t) {
    std::mt19937 rng(4242u + 17u * (unsigned)t + (unsigned)nq);
    if (t == 0) load_q(0, 1);
    for (int qi = 0; qi < nq; ++qi) {
      const unsigned par = (unsigned)qi & 1u;
      if (t == 0) {
        if (!bar_q.wait(par)) die("Q never landed", qi);
        issue_scores(qi);
#if BUG != 2
        if (!wait_reductions_read()) die("reductions never read their tile", qi);
#endif
      }
      cta.sync();
      if (!bar_1.wait(par)) die("scores never completed", qi);
      if (st_tag != qi) die("softmax read scores of another block", qi);
      nap(rng, 40);
      if (tile_readers != 0) fail("P^T written while the tiles were being read", qi);
      if (reductions_unread != 0) fail("P^T written over a staging tile not yet reduced", qi);
      tile_tag[t] = qi;
      cta.sync();
      if (t == 0) {
        issue_dv_dk(qi);
        issue_dq(qi);
#if EARLY
#if BUG != 1
        if (!bar_2a.wait(par)) die("dV / dK never completed", qi);
#endif
        if (qi + 1 < nq) load_q(qi + 1, 100u + (unsigned)qi);
#endif
      }
      if (!bar_2.wait(par)) die("dQ never completed", qi);
#if !EARLY
      if (t == 0 && qi + 1 < nq) load_q(qi + 1, 100u + (unsigned)qi);
#endif
      // drain dQ into the staging tile (which is the P^T / dS^T memory)
      ++dq_readers;
      if (dq_tag != qi) fail("drained a dQ accumulator of another block", qi);
      nap(rng, 30);
      if (tile_readers != 0) fail("staging written while the tiles were being read", qi);
      tile_tag[t] = -(qi + 2);
      --dq_readers;
#if BUG != 3
      cta.sync();
#endif
      if (t == 0) issue_reduction(qi, 300u + (unsigned)qi);
#if BUG == 3
      cta.sync();
#endif
    }
  }

  void run() {
    std::thread tp([this] { tensor.run(); }), cp([this] { copy.run(); });
    std::vector<std::thread> th;
    for (int t = 0; t < NT; ++t) th.emplace_back([this, t] { thread(t); });
    for (auto& t : th) t.join();
    tensor.finish();
    copy.finish();
    tp.join();
    cp.join();
    if (violations.load() == 0) {
      if (kv_acc != nq) fail("dK / dV accumulated the wrong number of blocks", nq);
      if (reduced != nq) fail("not every dQ block reached global memory", nq);
    }
  }
};

int main() {
  const int sizes[] = {1, 2, 3, 4, 7, 16, 32};
  for (int rep = 0; rep < 8 && violations.load() == 0; ++rep)
    for (int n : sizes) {
      Kernel k(n);
      k.run();
      if (violations.load()) break;
    }
  if (violations.load()) return 3;
  std::printf("ok: early=%d\n", EARLY);
  return 0;
}
