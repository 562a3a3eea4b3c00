// Host model of the barrier protocol of the software-pipelined attention forward kernels
// (csrc/attention_tcgen05.cu: attention_fwd_pipelined_kernel with 4 softmax warps,
// attention_fwd_pipelined8_kernel with 8), run by tests/test_attention_pipeline_model.py.
//
// Threads: one issuer, one tensor pipe that executes the issued MMAs in order, one copy
// engine that completes TMA loads after a random delay, and one thread per softmax warp.
// mbarriers are modelled with phase counters and parity waits exactly as the kernels use
// them.  Every buffer (K / V stages, the two S buffers, P, O, the row-maximum mailbox)
// carries a tag saying which key block its content belongs to; every consumer checks the tag
// it expects, so a missing wait shows up as a wrong tag and a wrong parity as a timeout.
//
//   -DSOFTMAX_WARPS=4 | 8     which kernel's protocol
//   -DBUG=1  the issuer does not wait for bar_p before issuing P V      (must be detected)
//   -DBUG=2  the softmax warps do not wait for bar_o before writing P   (must be detected)
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

#ifndef SOFTMAX_WARPS
#define SOFTMAX_WARPS 4
#endif
#ifndef BUG
#define BUG 0
#endif

static std::atomic<int> violations{0};
static void fail(const char* what, int j) {
  if (violations.fetch_add(1) == 0) std::fprintf(stderr, "violation: %s (block %d)\n", what, j);
}

struct MBar {
  std::mutex mu;
  std::condition_variable cv;
  int count = 1, pending = 1;
  unsigned long long phase = 0;  // completed phases
  void init(int c) { count = pending = c; phase = 0; }
  void arrive() {
    std::lock_guard<std::mutex> lk(mu);
    if (--pending == 0) {
      pending = count;
      ++phase;
      cv.notify_all();
    }
  }
  // mbarrier.try_wait.parity: true once the phase with this parity has completed, i.e. the
  // phase in progress has the other parity
  bool wait(unsigned parity) {
    std::unique_lock<std::mutex> lk(mu);
    return cv.wait_for(lk, std::chrono::seconds(5), [&] { return (phase & 1u) != parity; });
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
  int n;  // key blocks
  MBar bar_k[2], bar_v[2], bar_s[2], bar_p, bar_o, bar_x[4], bar_y[4];
  // content tags (-1 = nothing valid)
  std::atomic<int> k_tag[2], v_tag[2], s_tag[2], p_tag{-1};
  std::atomic<int> o_blocks{0};         // number of P V products accumulated into O
  std::atomic<int> o_busy{0};           // a P V product is writing O right now
  std::atomic<int> rowmax_tag[4];       // per quarter: block whose maximum is in the mailbox
  Work tensor, copy;

  explicit Kernel(int blocks) : n(blocks) {
    for (int i = 0; i < 2; ++i) {
      bar_k[i].init(1); bar_v[i].init(1); bar_s[i].init(1);
      k_tag[i] = v_tag[i] = s_tag[i] = -1;
    }
    bar_p.init(SOFTMAX_WARPS);
    bar_o.init(1);
    for (int i = 0; i < 4; ++i) { bar_x[i].init(2); bar_y[i].init(2); rowmax_tag[i] = -1; }
  }

  void load(bool is_k, int j, unsigned seed) {
    copy.push([this, is_k, j, seed] {
      std::mt19937 rng(seed);
      nap(rng, 300);
      (is_k ? k_tag : v_tag)[j & 1] = j;
      (is_k ? bar_k : bar_v)[j & 1].arrive();
    });
  }
  void issue_qk(int j) {
    tensor.push([this, j] {
      if (k_tag[j & 1] != j) fail("QK read a K stage that does not hold its block", j);
      s_tag[j & 1] = j;
      bar_s[j & 1].arrive();
    });
  }
  void issue_pv(int j) {
    tensor.push([this, j] {
      if (p_tag != j) fail("PV read a P tile that does not hold its block", j);
      if (v_tag[j & 1] != j) fail("PV read a V stage that does not hold its block", j);
      o_busy = 1;
      std::this_thread::sleep_for(std::chrono::microseconds(20));
      if (p_tag != j) fail("P was overwritten while PV was reading it", j);
      o_blocks.fetch_add(1);
      o_busy = 0;
      bar_o.arrive();
    });
  }

  void issuer() {
    std::mt19937 rng(12345u + (unsigned)n);
    auto wait = [&](MBar& b, unsigned par, const char* what, int j) {
      if (!b.wait(par)) { fail(what, j); return false; }
      return true;
    };
    load(true, 0, 1); load(false, 0, 2);
    if (n > 1) { load(true, 1, 3); load(false, 1, 4); }
    if (!wait(bar_k[0], 0, "K_0 never landed", 0)) return;
    issue_qk(0);
    if (n > 1) {
      if (!wait(bar_k[1], 0, "K_1 never landed", 1)) return;
      issue_qk(1);
    }
    for (int j = 0; j < n; ++j) {
      const unsigned par2 = (unsigned)(j >> 1) & 1u;
      nap(rng, 30);
      if (j + 2 < n) {
        if (!wait(bar_s[j & 1], par2, "issuer: S_j never completed", j)) return;
        load(true, j + 2, 100u + (unsigned)j);
      }
      if (j >= 1 && j + 1 < n) {
        if (!wait(bar_o, (unsigned)(j - 1) & 1u, "issuer: PV_{j-1} never completed", j)) return;
        load(false, j + 1, 200u + (unsigned)j);
      }
#if BUG != 1
      if (!wait(bar_p, (unsigned)j & 1u, "issuer: P_j never written", j)) return;
#endif
      if (!wait(bar_v[j & 1], par2, "issuer: V_j never landed", j)) return;
      issue_pv(j);
      if (j + 2 < n) {
        if (!wait(bar_k[j & 1], (unsigned)((j + 2) >> 1) & 1u, "issuer: K_{j+2} never landed", j))
          return;
        issue_qk(j + 2);
      }
    }
    wait(bar_o, (unsigned)(n - 1) & 1u, "issuer: last PV never completed", n - 1);
  }

  void softmax_warp(int w) {
    std::mt19937 rng(777u + (unsigned)w * 31u + (unsigned)n);
    const int quarter = w & 3;
    for (int j = 0; j < n; ++j) {
      if (!bar_s[j & 1].wait((unsigned)(j >> 1) & 1u)) return fail("softmax: S_j never ready", j);
      if (s_tag[j & 1] != j) return fail("softmax read an S buffer that holds another block", j);
      nap(rng, 40);
#if SOFTMAX_WARPS == 8
      if (j > 0 && !bar_y[quarter].wait((unsigned)(j - 1) & 1u))
        return fail("partner never read the previous maximum", j);
      rowmax_tag[quarter] = j;  // atomicMax into the mailbox
      bar_x[quarter].arrive();
      if (!bar_x[quarter].wait((unsigned)j & 1u)) return fail("partner never contributed", j);
      if (rowmax_tag[quarter] != j) return fail("row maximum of another block was read", j);
      bar_y[quarter].arrive();
#endif
      nap(rng, 60);
      if (j > 0) {
#if BUG != 2
        if (!bar_o.wait((unsigned)(j - 1) & 1u)) return fail("softmax: PV_{j-1} never done", j);
#endif
        if (o_busy) return fail("O rescaled while a PV product was writing it", j);
        if (o_blocks != j) return fail("O holds the wrong number of accumulated blocks", j);
      }
      p_tag = j;  // the softmax warps write their slices of P_j
      bar_p.arrive();
    }
    if (!bar_o.wait((unsigned)(n - 1) & 1u)) return fail("epilogue: last PV never done", n - 1);
    if (o_blocks != n) fail("epilogue read an incomplete O", n);
  }

  void run() {
    std::thread tp([this] { tensor.run(); }), cp([this] { copy.run(); });
    std::vector<std::thread> th;
    th.emplace_back([this] { issuer(); });
    for (int w = 0; w < SOFTMAX_WARPS; ++w) th.emplace_back([this, w] { softmax_warp(w); });
    for (auto& t : th) t.join();
    tensor.finish();
    copy.finish();
    tp.join();
    cp.join();
  }
};

int main() {
  const int sizes[] = {2, 3, 4, 5, 8, 16, 32};
  for (int rep = 0; rep < 6 && violations.load() == 0; ++rep)
    for (int n : sizes) {
      Kernel k(n);
      k.run();
      if (violations.load()) break;
    }
  if (violations.load()) return 3;
  std::printf("ok: %d softmax warps\n", SOFTMAX_WARPS);
  return 0;
}
