// Host check of the GEMM tile scheduler (csrc/gemm_schedule.cuh), built by
// tests/test_gemm_schedule.py with g++: for many (M, N, grid) the work items of the one-CTA
// kernel (128 x 256 tiles) and of the CTA-pair kernel (256 x 256) must cover every element of C
// exactly once, with and without the split tail; a split must happen exactly when the last
// wave fills at most half of the grid, and then no worker may get more than one half tile.
#include <cstdio>
#include <vector>

#define __host__
#define __device__
#include "gemm_schedule.cuh"

template <int BM, int BN, bool SPLIT>
static int check(int M, int N, int grid) {
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int tiles = tiles_m * tiles_n;
  if (grid > tiles) grid = tiles;
  int full = 0, items = 0;
  const bool split = gemm_sched::plan_tail(tiles, grid, SPLIT, &full, &items);
  const int tail = tiles % grid;
  if (split != (SPLIT && tail > 0 && 2 * tail <= grid)) return 1;
  if (!split && (full != tiles || items != tiles)) return 2;
  if (split && (full % grid != 0 || items - full != 2 * tail || items - full > grid)) return 3;
  std::vector<unsigned char> hit((size_t)M * N, 0);
  for (int w = 0; w < items; ++w) {
    const gemm_sched::WorkItem wi =
        split ? gemm_sched::work_item<BM, BN, 8, true>(tiles_m, tiles_n, full, w)
              : gemm_sched::work_item<BM, BN, 8, false>(tiles_m, tiles_n, full, w);
    if (wi.bn != (split && w >= full ? BN / 2 : BN)) return 4;
    if (wi.m0 % BM || wi.n0 % (BN / 2) || wi.m0 < 0 || wi.n0 < 0) return 5;
    for (int r = wi.m0; r < wi.m0 + BM && r < M; ++r)
      for (int c = wi.n0; c < wi.n0 + wi.bn && c < N; ++c)
        if (hit[(size_t)r * N + c]++) return 6;  // produced twice
  }
  for (unsigned char h : hit)
    if (h != 1) return 7;  // never produced
  return 0;
}

int main() {
  const int Ms[] = {1, 77, 128, 200, 256, 384, 1000, 1024, 4096};
  const int Ns[] = {8, 128, 136, 256, 264, 512, 1000, 4096};
  const int grids[] = {1, 2, 3, 4, 7, 24, 74, 148};
  long long cases = 0;
  for (int M : Ms)
    for (int N : Ns)
      for (int g : grids) {
        int rc;
        if ((rc = check<128, 256, false>(M, N, g)) || (rc = check<128, 256, true>(M, N, g)) ||
            (rc = check<256, 256, false>(M, N, g)) || (rc = check<256, 256, true>(M, N, g))) {
          std::fprintf(stderr, "M=%d N=%d grid=%d: failure %d\n", M, N, g, rc);
          return 1;
        }
        cases += 4;
      }
  // the case the split is for: 4096 x 4096 on 148 CTAs = 3 full waves + 68 tiles -> 136 halves
  int full = 0, items = 0;
  if (!gemm_sched::plan_tail(512, 148, true, &full, &items) || full != 444 || items != 580)
    return 2;
  std::printf("ok: %lld cases\n", cases);
  return 0;
}
