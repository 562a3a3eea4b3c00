// Tile scheduling of the persistent tcgen05 GEMM kernels, as host/device functions so that the
// CPU test tier can check that every element of C is produced exactly once.
//
// Work items are numbered 0 .. work_items-1 and taken round-robin by the CTAs (or CTA pairs)
// of the persistent grid.  Items [0, full_tiles) are whole BM x BN tiles, grouped along M so
// that CTAs running at the same time share B tiles in L2; with a split tail every later tile
// is cut into two BM x BN/2 halves, so that a last wave which fills at most half of the grid
// takes half a tile time.
#pragma once

namespace gemm_sched {

struct WorkItem {
  int m0, n0, bn;  // rows [m0, m0 + BM), columns [n0, n0 + bn) of C
};

template <int GROUP_M>
__host__ __device__ inline void tile_coords(int tiles_m, int tiles_n, int t, int* tm, int* tn) {
  const int per_group = GROUP_M * tiles_n;
  const int group = t / per_group;
  const int first_m = group * GROUP_M;
  const int rest = tiles_m - first_m;
  const int gsz = rest < GROUP_M ? rest : GROUP_M;
  const int r = t - group * per_group;
  *tm = first_m + r % gsz;
  *tn = r / gsz;
}

template <int BM, int BN, int GROUP_M, bool SPLIT_TAIL>
__host__ __device__ inline WorkItem work_item(int tiles_m, int tiles_n, int full_tiles, int w) {
  int tile = w, half = 0, bn = BN;
  if constexpr (SPLIT_TAIL) {
    if (w >= full_tiles) {
      const int u = w - full_tiles;
      tile = full_tiles + (u >> 1);
      half = u & 1;
      bn = BN / 2;
    }
  }
  int tm, tn;
  tile_coords<GROUP_M>(tiles_m, tiles_n, tile, &tm, &tn);
  return WorkItem{tm * BM, tn * BN + half * (BN / 2), bn};
}

// Host: decides whether the tail of `tiles` tiles on `grid` workers is split.
// Returns true when it is; *full_tiles / *work_items describe the numbering either way.
inline bool plan_tail(int tiles, int grid, bool allow_split, int* full_tiles, int* work_items) {
  const int tail = tiles % grid;
  const bool split = allow_split && tail > 0 && 2 * tail <= grid;
  *full_tiles = split ? tiles - tail : tiles;
  *work_items = tiles + (split ? tail : 0);
  return split;
}

}  // namespace gemm_sched
