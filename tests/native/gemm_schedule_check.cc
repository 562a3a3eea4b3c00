// Host check of the GEMM tile scheduler (csrc/gemm_schedule.cuh), built by
// tests/test_gemm_schedule.py with g++: for many (M, N) the tiles of the one-CTA kernel
// (128 x 256) and of the CTA-pair kernel (256 x 256) must cover every element of C exactly
// once, whatever the grouping along M does at the edges.
#include <cstdio>
#include <vector>

#define __host__
#define __device__
#include "gemm_schedule.cuh"

template <int BM, int BN>
static int check(int M, int N) {
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  std::vector<unsigned char> hit((size_t)M * N, 0);
  for (int w = 0; w < tiles; ++w) {
    const gemm_sched::WorkItem wi = gemm_sched::work_item<BM, BN, 8>(tiles_m, tiles_n, w);
    if (wi.m0 % BM || wi.n0 % BN || wi.m0 < 0 || wi.n0 < 0) return 5;
    for (int r = wi.m0; r < wi.m0 + BM && r < M; ++r)
      for (int c = wi.n0; c < wi.n0 + BN && c < N; ++c)
        if (hit[(size_t)r * N + c]++) return 6;  // produced twice
  }
  for (unsigned char h : hit)
    if (h != 1) return 7;  // never produced
  return 0;
}

int main() {
  const int shapes[][2] = {{128, 256},  {4096, 4096}, {4096, 12288}, {200, 264},  {77, 8},
                           {1024, 1024}, {2048, 22016}, {8192, 4096}, {1152, 512}, {3000, 1000},
                           {256, 256},  {129, 257},   {9 * 128, 3 * 256}};
  int checked = 0;
  for (auto& s : shapes) {
    if (int rc = check<128, 256>(s[0], s[1])) {
      std::fprintf(stderr, "128x256 tiles: M=%d N=%d: code %d\n", s[0], s[1], rc);
      return 1;
    }
    if (int rc = check<256, 256>(s[0], s[1])) {
      std::fprintf(stderr, "256x256 tiles: M=%d N=%d: code %d\n", s[0], s[1], rc);
      return 1;
    }
    checked += 2;
  }
  std::printf("ok: %d schedules cover their outputs exactly once\n", checked);
  return 0;
}
