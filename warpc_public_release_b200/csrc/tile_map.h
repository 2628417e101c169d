// CTA tile index -> origin of the tile in C, shared by the kernel and the host (tests compare
// it with the reference's map, backend/tiles.ml:32-80).  The index's digits, fastest first:
// the CTA's rank in its pair (pairs sit side by side along columns), the row within a group
// of `group` cluster rows (a power of two), the cluster column, the band of groups; with
// `serp`, odd bands run right to left so consecutive bands share their last columns in L2.
#pragma once
#if defined(__CUDACC__)
#define WB_HD __host__ __device__ __forceinline__
#else
#define WB_HD inline
#endif

WB_HD void wb_tile_origin(int tile, int cg, int tile_m, int tile_n, int group, int cl_n, int serp, int* row, int* col) {
  const int rank = tile % cg, c = tile / cg;
  const int rig = c & (group - 1), rest = c / group;
  int colc = rest % cl_n;
  const int band = rest / cl_n;
  if (serp && (band & 1)) colc ^= (cl_n - 1);
  *row = (band * group + rig) * tile_m;
  *col = (colc * cg + rank) * tile_n;
}
