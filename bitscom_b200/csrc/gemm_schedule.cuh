// Tile scheduling of the persistent tcgen05 GEMM kernels, as host/device functions so that the
// CPU test tier can check that every element of C is produced exactly once.
//
// Tiles are numbered 0 .. tiles-1 and taken round-robin by the CTAs (or CTA pairs) of the
// persistent grid; they are grouped along M so that CTAs running at the same time share B
// tiles in L2.
#pragma once

namespace gemm_sched {

struct WorkItem {
  int m0, n0;  // rows [m0, m0 + BM), columns [n0, n0 + BN) of C
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

template <int BM, int BN, int GROUP_M>
__host__ __device__ inline WorkItem work_item(int tiles_m, int tiles_n, int w) {
  int tm, tn;
  tile_coords<GROUP_M>(tiles_m, tiles_n, w, &tm, &tn);
  return WorkItem{tm * BM, tn * BN};
}

}  // namespace gemm_sched
