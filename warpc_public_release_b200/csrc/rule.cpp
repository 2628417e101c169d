// Host side of the operator surface: the per-shape rule (`warpc gemm M N K`), the geometry
// a decision implies, how this library's kernels realise it, and the launch header text.
//
// Rule: backend/programs.ml:46-80.  Geometry: backend/gemm_swapped.ml:50-108 (swapped),
// backend/gemm_pair.ml:16-43 (pair), backend/gemm_one.ml:17-30 (one).
// Header: backend/compile.ml:86-88, 165-186.
#include <climits>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/warpc_b200.h"
#include "kernel_table.h"

namespace {

constexpr int kSms = 148;
constexpr int kTileK = 64;

// clusters of `ctas` CTAs resident at once on 148 SMs (backend/gemm_swapped.ml:27)
int resident_clusters(int ctas) {
  switch (ctas) {
    case 1: return kSms;
    case 2: return 74;
    case 4: return 33;
    case 8: return 15;
    default: return 0;
  }
}

int pow2_cols(int n) {  // tensor-memory allocation: a power of two, 32 at least (backend/atom.ml:216-218)
  int c = 32;
  while (c < n) c *= 2;
  return c;
}

wg_variant blank(int prog, int tm, int tn, int depth) {
  wg_variant v;
  std::memset(&v, 0, sizeof v);
  v.prog = prog, v.tile_m = tm, v.tile_n = tn, v.tile_k = kTileK, v.depth = depth;
  v.cluster_n = 1, v.group = 8, v.split = 1, v.split_grid = 1;
  return v;
}

int derive_swapped(int m, int n, int k, wg_variant* v) {
  const int pair = 2;
  if (v->cluster_n < 1) v->cluster_n = 1;
  if (v->split < 1) v->split = 1;
  if (v->split_grid < 1) v->split_grid = 1;
  if (v->group < 1) v->group = 8;
  // the builder's refusals (backend/gemm_swapped.ml:32-48)
  if (v->streamk && (v->clc || v->cluster_n > 1 || (v->direct != 0) == (v->split_add != 0))) return WG_E_VARIANT;
  if (v->split > 1 && (v->split > 4 || v->cluster_n != v->split || v->clc || v->streamk || !v->direct)) return WG_E_VARIANT;
  if (v->split_grid > 1 && (v->split > 1 || v->clc || v->streamk || (v->direct != 0) == (v->split_add != 0))) return WG_E_VARIANT;
  if (v->split_add && v->split_grid == 1 && !v->streamk) return WG_E_VARIANT;
  if (v->tile_m <= 0 || v->tile_n <= 0 || v->depth <= 0 || m <= 0 || n <= 0 || k <= 0) return WG_E_VARIANT;

  const int ctas = pair * v->cluster_n;
  const int rows_needed = v->tile_n * pair;
  const int atom_m = rows_needed < 256 ? rows_needed : 256;
  if (rows_needed % atom_m != 0) return WG_E_VARIANT;
  // kind::f16 pair shapes (backend/atom.ml:146-154)
  if (!(atom_m == 128 || atom_m == 256)) return WG_E_VARIANT;
  if (!(v->tile_m % 16 == 0 && v->tile_m >= 16 && v->tile_m <= 256)) return WG_E_VARIANT;
  v->atom_m = atom_m;
  v->reps = rows_needed / atom_m;
  const int a_rows = atom_m / pair;                   // B^T rows a CTA feeds one atom
  const int sb_rows = v->reps * a_rows;               // = tile_n
  const int sa_rows = v->tile_m / pair;               // A rows a CTA loads
  const int acc_rows = atom_m / pair;                 // accumulator rows a CTA holds per atom
  const int span = (acc_rows == 128) ? v->tile_m : v->tile_m / 2;  // backend/atom.ml:235-251
  if (v->reps * acc_rows != v->tile_n) return WG_E_VARIANT;
  v->tiles_m = (m + v->tile_m - 1) / v->tile_m;
  v->tiles_n = (n + v->tile_n - 1) / v->tile_n;
  const int sharing = v->split > 1 ? 1 : v->cluster_n;
  if (v->tiles_m % sharing != 0 || v->tiles_n % pair != 0 || k % (kTileK * v->split) != 0 || k / kTileK < v->split_grid)
    return WG_E_VARIANT;
  if (v->direct && (m % v->tile_m != 0 || n % v->tile_n != 0)) return WG_E_VARIANT;
  if (sb_rows % sharing != 0) return WG_E_VARIANT;
  v->a_box_rows = sa_rows;
  v->bt_box_rows = sb_rows / sharing;
  v->tmem_cols = pow2_cols(v->reps * span);
  v->total_tiles = v->tiles_m * v->tiles_n;
  v->nbuf = v->bufs > 0 ? v->bufs : ((2 * v->tmem_cols <= 512 && v->total_tiles > kSms) ? 2 : 1);
  if (v->tmem_cols * v->nbuf > 512) return WG_E_VARIANT;
  v->alloc_cols = pow2_cols(v->tmem_cols * v->nbuf);
  v->ctas = ctas;
  v->persistent = (v->split == 1 && v->split_grid == 1 && (v->clc || v->total_tiles > kSms)) ? 1 : 0;
  if (resident_clusters(ctas) == 0) return WG_E_VARIANT;
  if (v->streamk) v->grid = kSms / ctas * ctas;
  else if (v->split > 1) v->grid = v->total_tiles * v->split;
  else if (v->split_grid > 1) v->grid = v->total_tiles * v->split_grid;
  else if (v->clc || v->total_tiles <= kSms) v->grid = v->total_tiles;
  else v->grid = resident_clusters(ctas) * ctas;
  if (v->split_grid > 1 && v->grid / ctas > resident_clusters(ctas)) return WG_E_VARIANT;
  v->stage_bytes = sa_rows * kTileK * 2 + sb_rows * kTileK * 2;
  v->tx_bytes = pair * v->stage_bytes;
  v->kt = k / kTileK / v->split;
  if (v->streamk && !v->split_add) {
    const int clusters = v->grid / ctas, units = v->total_tiles / ctas * v->kt;
    if (units / clusters < v->kt) return WG_E_VARIANT;
  }
  const int staging = v->direct ? 0 : 4 * 2 * (8 * 32 * 4);
  v->ref_dynsmem = v->depth * v->stage_bytes + staging;
  if (v->ref_dynsmem + 0x400 + 0x400 > 232448) return WG_E_VARIANT;  // backend/mem.ml:228
  v->ref_mbarriers = 2 * v->depth + 2 * v->nbuf + (v->clc ? 2 : 0) + (v->split > 1 ? 1 : 0);
  if (v->split_add) v->nflags = v->streamk ? v->grid + v->total_tiles : v->grid;
  else if (v->streamk || v->split_grid > 1) v->nflags = v->grid;
  else v->nflags = 0;
  return WG_OK;
}

int derive_pair(int m, int n, int k, wg_variant* v) {
  // backend/gemm_pair.ml:16-43: 2x1 cluster along M, M = 256 x N = 128 atom
  v->tile_m = 128, v->tile_n = 128, v->tile_k = kTileK;
  if (m % 256 != 0 || n % 128 != 0 || k % kTileK != 0 || v->depth <= 0) return WG_E_VARIANT;
  v->cluster_n = 1, v->split = 1, v->split_grid = 1, v->group = 8;
  v->atom_m = 256, v->reps = 1, v->tmem_cols = 128, v->nbuf = 1, v->alloc_cols = 128;
  v->tiles_m = m / 128, v->tiles_n = n / 128, v->total_tiles = v->tiles_m * v->tiles_n;
  v->ctas = 2;
  v->grid = v->total_tiles <= kSms ? v->total_tiles : kSms / 2 * 2;
  v->persistent = 1;
  v->kt = k / kTileK;
  v->a_box_rows = 128, v->bt_box_rows = 64;
  v->stage_bytes = 128 * 128 + 64 * 128;
  v->tx_bytes = 2 * v->stage_bytes;
  v->ref_dynsmem = v->depth * v->stage_bytes + 4 * 2 * (32 * 32 * 4);
  if (v->ref_dynsmem + 0x800 > 232448) return WG_E_VARIANT;
  v->ref_mbarriers = 2 * v->depth + 2;
  return WG_OK;
}

int derive_one(int m, int n, int k, wg_variant* v) {
  // backend/gemm_one.ml:17-30: one CTA a 128 x 128 tile, cta_group::1
  v->tile_m = 128, v->tile_n = 128, v->tile_k = kTileK;
  if (m % 128 != 0 || n % 128 != 0 || k % kTileK != 0 || v->depth <= 0) return WG_E_SHAPE;
  v->cluster_n = 1, v->split = 1, v->split_grid = 1, v->group = 1, v->direct = 1;
  v->atom_m = 128, v->reps = 1, v->tmem_cols = 128, v->nbuf = 1, v->alloc_cols = 128;
  v->tiles_m = m / 128, v->tiles_n = n / 128, v->total_tiles = v->tiles_m * v->tiles_n;
  v->ctas = 1, v->grid = v->total_tiles, v->kt = k / kTileK;
  v->a_box_rows = 128, v->bt_box_rows = 128;
  v->stage_bytes = 2 * 128 * 128;
  v->tx_bytes = v->stage_bytes;
  v->ref_dynsmem = v->depth * v->stage_bytes;
  if (v->ref_dynsmem + 0x800 > 232448) return WG_E_VARIANT;
  v->ref_mbarriers = 2 * v->depth + 1;
  return WG_OK;
}

// the group of cluster rows a walk really uses (backend/tiles.ml:42-47)
int effective_group(int group, int walked, int other) {
  int g = 1;
  while (g * 2 <= walked && g < group) g *= 2;
  const bool pow2_other = other > 0 && (other & (other - 1)) == 0;
  return (pow2_other && walked % g == 0) ? g : 1;
}

void append(std::string& s, const char* fmt, ...) {
  char line[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(line, sizeof line, fmt, ap);
  va_end(ap);
  s += line;
  s += '\n';
}

}  // namespace

extern "C" int wg_derive(int M, int N, int K, wg_variant* v) {
  if (!v) return WG_E_ARG;
  switch (v->prog) {
    case WG_PROG_SWAPPED: return derive_swapped(M, N, K, v);
    case WG_PROG_PAIR: return derive_pair(M, N, K, v);
    case WG_PROG_ONE: return derive_one(M, N, K, v);
    default: return WG_E_VARIANT;
  }
}

extern "C" int wg_choose(int m, int n, int k, int sm, wg_variant* out) {
  if (!out || (sm != WG_SM_100A && sm != WG_SM_103A)) return WG_E_ARG;
  if (m <= 0 || n <= 0 || k <= 0) return WG_E_SHAPE;
  const int tiles = m / 128 * (n / 128);
  const bool pair_fits = m % 256 == 0 && n % 128 == 0 && k % 64 == 0;
  const bool swapped_fits = n % 256 == 0 && m % 64 == 0 && k % 64 == 0 && (m + 255) / 256 * (n / 128) >= kSms;
  auto waves = [&](int cn) {
    const int rc = resident_clusters(2 * cn);
    return (m % (128 * cn) == 0) ? (tiles / (2 * cn) + rc - 1) / rc : INT_MAX;
  };
  const int pair_tiles = (m % 256 == 0 && n % 512 == 0) ? m / 256 * (n / 512) : 0;
  const int runs = pair_tiles > 0 ? resident_clusters(2) / pair_tiles : 0;
  const int mn = m < n ? m : n, mnk = mn < k ? mn : k;
  wg_variant v;
  if (swapped_fits && n % 512 == 0 && m % 256 == 0 && mnk >= 8192) {
    v = blank(WG_PROG_SWAPPED, 256, 256, 4);
    v.clc = 1, v.ask_ahead = 1, v.serpentine = 1;
  } else if (swapped_fits && k <= 1024 && m % 256 == 0) {
    v = blank(WG_PROG_SWAPPED, 256, 128, 5);
    v.late_launch = 1;
  } else if (swapped_fits) {
    v = blank(WG_PROG_SWAPPED, 192, 128, 7);
    v.clc = k >= 4096;
  } else if (2 * tiles <= kSms && n % 128 == 0 && m % 128 == 0 && k % 64 == 0) {
    if (k >= 65536 && runs >= 2 && k / 64 >= runs) {
      v = blank(WG_PROG_SWAPPED, 256, 256, 4);
      v.split_grid = runs, v.split_add = 1, v.ask_ahead = 1;
    } else if (k >= 16384 && n / 128 % 2 == 0 && k % 128 == 0 && tiles / 2 <= resident_clusters(4)) {
      v = blank(WG_PROG_SWAPPED, 128, 128, 9);
      v.split = 2, v.cluster_n = 2, v.direct = 1;
    } else {
      v = blank(WG_PROG_SWAPPED, 128, 64, 13);
      v.direct = 1, v.ask_ahead = 1, v.late_launch = (sm == WG_SM_103A);
    }
  } else if (tiles <= kSms && n % 256 == 0 && m % 128 == 0 && k % 64 == 0) {
    v = blank(WG_PROG_SWAPPED, 128, 128, 6);
    v.direct = 1, v.late_launch = 1;
  } else if (tiles > kSms && k >= 16384 && m % 512 == 0 && n % 256 == 0 && m / 512 * (n / 256) <= resident_clusters(4)) {
    v = blank(WG_PROG_SWAPPED, 256, 128, 6);
    if (sm == WG_SM_100A) v.streamk = 1, v.split_add = 1, v.bufs = 2, v.ask_ahead = 1;
    else v.cluster_n = 2, v.late_launch = 1;
  } else if (tiles > kSms && n % 256 == 0 && k % 64 == 0 && waves(2) != INT_MAX) {
    const int cluster_n = waves(4) <= waves(2) ? 4 : (waves(1) <= waves(2) ? 1 : 2);
    v = blank(WG_PROG_SWAPPED, 128, 128, k >= 8192 ? 9 : 8);
    v.clc = cluster_n > 1, v.cluster_n = cluster_n, v.late_launch = cluster_n == 4, v.group = 16;
  } else if (pair_fits) {
    v = blank(WG_PROG_PAIR, 128, 128, 8);
  } else {
    v = blank(WG_PROG_ONE, 128, 128, 4);
  }
  const int r = wg_derive(m, n, k, &v);
  if (r != WG_OK) return r == WG_E_VARIANT ? WG_E_SHAPE : r;
  v.retile = 1;
  *out = v;
  return WG_OK;
}

// How this library runs a variant.  Differences from the reference's own launch, all in the
// direction of fewer hardware features: a cluster is always the pair alone (the reference's
// 2 x cluster_n clusters exist to multicast B^T tiles; here each CTA fetches its own tiles and
// the L2 serves the duplicates), and split-K inside such a cluster becomes split-K over the
// grid with the partial sums added in the L2.
extern "C" int wg_realise(const wg_variant* v, int M, int N, int K, wg_launch_info* out) {
  if (!v || !out) return WG_E_ARG;
  std::memset(out, 0, sizeof *out);
  wg_launch_info& li = *out;
  li.threads = 256;
  li.depth = v->depth;
  li.ask_ahead = v->ask_ahead;
  li.split = 1;
  if (v->prog == WG_PROG_ONE) {
    li.cg = 1, li.tile_m = 128, li.tile_n = 128, li.direct = 1;
    li.grid = v->grid, li.cluster = 1, li.sched = 0, li.nbuf = 1, li.group = 1, li.cl_n = v->tiles_n;
  } else if (v->prog == WG_PROG_PAIR) {
    // same pair tile (256 x 128) in the swapped orientation: 256 x 64 a CTA, an M = 128 pair
    li.cg = 2, li.tile_m = 256, li.tile_n = 64, li.direct = 0;
    const int tiles_m = M / 256, tiles_n = N / 64, total = tiles_m * tiles_n;
    li.cluster = 2;
    li.grid = total <= kSms ? total : kSms / 2 * 2;
    li.sched = total <= kSms ? 0 : 1;
    li.nbuf = (total > kSms) ? 2 : 1;
    li.cl_n = tiles_n / 2;
    li.group = effective_group(8, tiles_m, li.cl_n);
  } else {
    // K shared between CTAs (split in the cluster, split over the grid, stream-K).  A variant named explicitly runs in the
    // form it names: partial sums through a workspace, added up in a fixed order by the CTA that stores the block
    // (backend/gemm_swapped.ml:716-832; store from the registers), or added in the L2 (split_add).  Split inside a cluster
    // (`split`) is the same split over the grid, two pairs a tile, through the workspace.  The rule's own choices
    // (retile) always add in the L2: same sums, no workspace, and measured faster.
    const bool shares_k = v->streamk || v->split_grid > 1 || v->split > 1;
    const bool via_ws = shares_k && v->direct && !v->split_add && !v->retile;
    li.cg = 2, li.tile_m = v->tile_m, li.tile_n = v->tile_n, li.direct = v->direct && (!shares_k || via_ws);
    li.cluster = 2;
    li.nbuf = v->nbuf;
    int group = v->group, clc = v->clc, streamk = v->streamk;
    const bool plain = !v->streamk && v->split_grid <= 1 && v->split <= 1;
    if (v->retile && plain) {
      // Measured on a B200 (no TMA multicast): one tcgen05.mma costs 55-90 cycles to issue whatever
      // its N, so MMAs narrower than N = 256 (tile_m < 256) cannot keep the tensor pipe full; and
      // a fixed grid walking tiles by stride beats cluster launch control until tiles are 256 x 256.
      li.direct = 0;
      const int pair_tiles_256 = (M % 256 == 0 && N % 256 == 0) ? (M / 256) * (N / 256) : 0;
      if (v->tile_m < 256 && v->tile_n == 128 && pair_tiles_256 >= 50) {
        li.tile_m = 256, li.tile_n = 128, li.depth = 6, clc = 0, group = 8;
        li.nbuf = (2 * pair_tiles_256 > kSms) ? 2 : 1;
      }
      // A last wave that fills under nine tenths of the machine costs more than stream-K's extra
      // partial tiles (measured 87.0 against 91.3 us at 4096^3, 3.46 waves), once a tile's K is long
      // enough to share: the units of K are then dealt evenly to the 74 clusters.
      if (li.tile_m == 256 && li.tile_n == 128 && pair_tiles_256 > kSms / 2 && K / 64 >= 32) {
        const int clusters = kSms / 2, waves = (pair_tiles_256 + clusters - 1) / clusters;
        if (10 * pair_tiles_256 < 9 * waves * clusters) streamk = 1, li.nbuf = 2;
      }
      // The store: where a CTA's tiles are whole and K is not shared, 128-column tiles go out from the registers
      // (isolated calls, both input families: 2048^3 18.9 against 20.4 us, 3072x1280x2048 18.8 / 20.4, 4096x4096x1024
      // 34.3 / 37.8, 1536^3 12.7 / 13.8).  A one-tile launch ends on its store either way, and a TMA store's source is
      // only read ~1 us after it is issued, which the CTA has to wait out before it may leave; on the fixed-grid walk
      // the register stores of tile t run beside tile t+1's loads without taking the copy engine from them, and the
      // ring gets the staging copies' room (one more stage).  The 64-column fold tile (1024^3) measured the same both
      // ways in the full kernel and 7.9 against 8.5 us in the simple instance (below), which only stores from the
      // registers; the 256 x 256 tile's exposed 256 KB store is faster through the copy engine and stays staged.
      if (!streamk && !clc && li.tile_n <= 128 && M % li.tile_m == 0 && N % li.tile_n == 0) li.direct = 1;
    }
    const int tiles_m = (M + li.tile_m - 1) / li.tile_m, tiles_n = (N + li.tile_n - 1) / li.tile_n;
    const int total = tiles_m * tiles_n;
    li.cl_n = tiles_n / 2;
    li.group = effective_group(group, tiles_m, li.cl_n);
    li.serpentine = v->serpentine && li.cl_n > 1 && (li.cl_n & (li.cl_n - 1)) == 0;
    if (streamk) {
      li.sched = 4, li.grid = kSms / 2 * 2;
      li.nflags = li.grid + total;
      // Where this library chose stream-K itself (a poorly filled last wave), only the last whole wave and the remainder are
      // shared: the waves before them are walked whole, by stride, in step.  Dealing every tile's k-steps out (the
      // reference's stream-K, kept for variants named explicitly) leaves the 74 clusters at 74 different places of the walk,
      // reading different operand panels at any one time: 8192x2048x4096 then reads its operands 2.5 times from DRAM.
      // Measured, each call alone, pair tiles walked whole 0 / 74 / 148 / 222 of 256: 4096^3 91.1 / 90.9 / 89.0 / 89.7 us,
      // 8192x2048x4096 92.0 / 91.1 / 88.8 / 89.3 (uniform inputs alike): one wave and the remainder shared is the best.
      if (v->retile && !v->streamk) {
        const int clusters = li.grid / 2, waves = (total / 2) / clusters;
        li.sk_dp = waves > 1 ? (waves - 1) * clusters : 0;
      }
    } else if (v->split_grid > 1 || v->split > 1) {
      li.split = v->split_grid > 1 ? v->split_grid : v->split;
      li.sched = 3, li.grid = total * li.split;
      li.nflags = li.grid;
      if (li.grid / 2 > resident_clusters(2)) return WG_E_VARIANT;
    } else if (clc) {
      li.sched = 2, li.grid = total;
    } else if (total <= kSms) {
      li.sched = 0, li.grid = total;
    } else {
      li.sched = 1, li.grid = resident_clusters(2) * 2;
    }
  }
  // Launches of whole tiles, one a CTA or a fixed grid by stride, stored from the registers, run in the "simple" instance
  // of their tile where there is one: the same kernel compiled without launch control, shared K, further copies of C
  // and phase stamps, 26-29 KB of code instead of 67-90.  These are the launches of ten to thirty microseconds, where
  // every role's first pass through its code is a visible part of the time: measured, full -> simple instance,
  // 1024^3 9.6 -> 8.5 us, 1536^3 12.3 -> 11.5, 2048^3 17.8 -> 16.9, 4096x4096x1024 31.8 -> 30.3.
  const wb_kernel_entry* e = nullptr;
  if (li.direct && li.sched <= 1 && M % li.tile_m == 0 && N % li.tile_n == 0) e = wb_find_kernel(li.cg, li.tile_m, li.tile_n, 1, 1, -1);
  // ... and the long programs in the instance compiled for their one scheduling mode, where there is one (52-89 KB of code
  // against 135-173).  Measured against the full instance of the same tile, call by call in one process, same bits:
  // 4096^3 81.6 against 82.5 us, 8192x2048x4096 83.7 / 84.6, 2048x2048x16384 87.6 / 87.9, 1024x1024x65536 84.6 / 87.3,
  // 8192^3 692 / 694.
  if (!e) e = wb_find_kernel(li.cg, li.tile_m, li.tile_n, li.direct, 0, li.sched);
  if (!e) e = wb_find_kernel(li.cg, li.tile_m, li.tile_n, li.direct, 0, -1);
  if (!e) return WG_E_NOKERNEL;
  li.kernel_id = e->id;
  li.epi_rows = e->epi_rows;
  li.tmem_cols = e->ncols * li.nbuf > 32 ? pow2_cols(e->ncols * li.nbuf) : 32;
  if (e->ncols * li.nbuf > 512) return WG_E_VARIANT;
  // this kernel's staging copies and control block are larger than the reference's: where the
  // reference's ring depth no longer fits beside them, the ring is one or two stages shorter.
  // Shared memory beside the ring: alignment slack, control block and the epilogue's cycling staging
  // copies -- which a launch of one tile a CTA never uses when the ring can hold the tile (every tile is
  // then its CTA's last and is staged in the drained ring), so there the ring gets their room as well
  auto fit_depth = [&](size_t fixed, int depth) {
    while (depth > 2 && fixed + size_t(depth) * e->stage_bytes > 232448) depth -= 1;
    // the rule's own programs take the deepest ring that fits: ring slack against L2 latency is what the
    // k loop's pace depends on most (256 x 128: 560 cycles a k-step at depth 6, 620 at 5, 750 at 4)
    if (v->retile && v->prog == WG_PROG_SWAPPED)
      while (depth < 16 && fixed + size_t(depth + 1) * e->stage_bytes <= 232448) depth += 1;
    return depth;
  };
  size_t fixed = e->smem_fixed;
  li.staging_bytes = e->staging_bytes;
  if (!li.direct && li.sched == 0 && e->staging_bytes > 0) {
    const size_t without = e->smem_fixed - size_t(e->staging_bytes);
    const int d = fit_depth(without, li.depth);
    if (size_t(d) * size_t(e->stage_bytes) >= size_t(li.tile_m) * size_t(li.tile_n) * 4) fixed = without, li.staging_bytes = 0;
  }
  li.depth = fit_depth(fixed, li.depth);
  li.dynsmem = int(fixed + size_t(li.depth) * e->stage_bytes);
  if (li.dynsmem > 232448 || li.depth > 16) return WG_E_VARIANT;
  li.a_box_rows = li.tile_m / li.cg;
  li.bt_box_rows = li.tile_n;
  li.c_box_rows = li.direct ? 0 : li.epi_rows;
  // How many k-steps the ring hands over at a time (one full and one empty barrier a round): one
  // k-step's barrier round costs the issuing thread more than four narrow MMAs take to run, so
  // the slots of the N = 128 tiles go in fours (16 KB) or pairs (24 KB); larger slots keep a round per
  // k-step, where handing over 64 KB at a time would leave the producer too little slack.
  li.stage_bytes = e->stage_bytes;
  li.ksub = (e->reps != 1 || e->stage_bytes > 24 * 1024) ? 1 : (e->stage_bytes <= 16 * 1024 ? 4 : 2);
  while (li.ksub > 1 && li.depth / li.ksub < 2) li.ksub /= 2;
  if (e->simple && e->ksub != 0 && e->ksub != li.ksub) {
    // the simple instance fixes its round at compile time: another round runs in the full instance of the same tile
    e = wb_find_kernel(li.cg, li.tile_m, li.tile_n, li.direct, 0, -1);
    if (!e) return WG_E_NOKERNEL;
    li.kernel_id = e->id;
  }
  li.rounds = li.depth / li.ksub;
  li.mbarriers = 2 * li.rounds + 4 + 3;  // full + empty a round, two accumulators' full + empty, scheduler's three
  // a CTA's last tile is staged whole in the ring when the ring can hold it
  li.wide_rows = (!li.direct && size_t(li.depth) * size_t(e->stage_bytes) >= size_t(li.tile_m) * size_t(li.tile_n) * 4) ? e->wide_rows : 0;
  li.ws_words = (li.direct && (li.sched == 3 || li.sched == 4)) ? li.grid * li.tile_m * li.tile_n : 0;
  (void)K;
  return WG_OK;
}

extern "C" int wg_header(const wg_variant* v, int M, int N, int K, char* buf, size_t cap) {
  if (!v || !buf) return WG_E_ARG;
  wg_launch_info li;
  const int r = wg_realise(v, M, N, K, &li);
  if (r != WG_OK) return r;
  std::string s;
  char name[128];
  if (v->prog == WG_PROG_SWAPPED) snprintf(name, sizeof name, "swapped_%d_%d_%d_%dx%d_s%d", M, N, K, v->tile_m, v->tile_n, v->depth);
  else if (v->prog == WG_PROG_PAIR) snprintf(name, sizeof name, "pair_%d_%d_%d_s%d", M, N, K, v->depth);
  else snprintf(name, sizeof name, "one_%d_%d_%d_s%d", M, N, K, v->depth);
  if (v->prog == WG_PROG_SWAPPED) {
    append(s, "# gemm_swapped %dx%dx%d: %dx%d a CTA, ring depth %d, cluster 2x%d, %d accumulator%s, %s%s%s%s%s%s", M, N, K,
           v->tile_m, v->tile_n, v->depth, v->cluster_n, v->nbuf, v->nbuf > 1 ? "s" : "",
           v->clc ? "cluster launch control" : "a fixed grid", v->ask_ahead ? ", asking a stage ahead" : "",
           v->direct ? ", the store from the registers" : "",
           v->split > 1 ? ", K split in the cluster" : "", v->split_grid > 1 ? ", K split over the grid" : "",
           v->split_add ? ", the runs adding in the L2" : "");
  } else if (v->prog == WG_PROG_PAIR) {
    append(s, "# gemm_pair %dx%dx%d, ring depth %d, a 2x1 cluster sharing a cta_group::2 MMA", M, N, K, v->depth);
  } else {
    append(s, "# gemm_one %dx%dx%d, ring depth %d, one CTA a 128x128 tile", M, N, K, v->depth);
  }
  append(s, "# b200 kernel %s: %dx%d a CTA, ring depth %d, %d accumulator%s, sched %d, cluster %d, tensor memory %d columns",
         wg_kernel_name(li.kernel_id), li.tile_m, li.tile_n, li.depth, li.nbuf, li.nbuf > 1 ? "s" : "", li.sched, li.cluster, li.tmem_cols);
  // every rule field, so a runner given only this text can rebuild the exact program (a comment to the reference's reader)
  append(s, "# variant prog=%d tile_m=%d tile_n=%d depth=%d cluster_n=%d clc=%d ask_ahead=%d direct=%d serpentine=%d group=%d streamk=%d "
            "split=%d split_grid=%d split_add=%d late_launch=%d bufs=%d retile=%d",
         v->prog, v->tile_m, v->tile_n, v->depth, v->cluster_n, v->clc, v->ask_ahead, v->direct, v->serpentine, v->group, v->streamk, v->split,
         v->split_grid, v->split_add, v->late_launch, v->bufs, v->retile);
  append(s, ".kernel %s", name);
  append(s, ".sm sm_100a");
  append(s, ".barriers 2");
  append(s, ".threads %d", li.threads);
  append(s, ".smem 0");
  append(s, ".dynsmem %d", li.dynsmem);
  append(s, ".tile %d %d %d", li.tile_m, li.tile_n, kTileK);
  if (li.direct) append(s, ".ptr c %d %d 4", M, N);
  else append(s, ".tmap c %d %d 4 %d 32 0", M, N, li.c_box_rows);
  append(s, ".tmap a %d %d 2 %d 64 128", M, K, li.a_box_rows);
  append(s, ".tmap bt %d %d 2 %d 64 128", N, K, li.bt_box_rows);
  if (li.nflags > 0) append(s, ".ptr flags 1 %d 4", li.nflags);
  if (li.ws_words > 0) append(s, ".ptr ws %d %d 4", li.grid, li.tile_m * li.tile_n);
  append(s, ".grid %d 1", li.grid);
  append(s, ".mbarriers %d", li.mbarriers);
  append(s, ".cluster %d", li.cluster);
  append(s, ".tcgen05");
  append(s, li.ws_words > 0 ? ".params 8 8 8 8 8" : li.nflags > 0 ? ".params 8 8 8 8" : ".params 8 8 8");
  if (s.size() + 1 > cap) return WG_E_ARG;
  std::memcpy(buf, s.c_str(), s.size() + 1);
  return int(s.size());
}

extern "C" const char* wg_strerror(int code) {
  switch (code) {
    case WG_OK: return "ok";
    case WG_E_SHAPE: return "no program for this shape";
    case WG_E_VARIANT: return "inconsistent variant";
    case WG_E_ARG: return "bad argument";
    case WG_E_NOKERNEL: return "no compiled kernel realises the variant";
    case WG_E_DEVICE_WAIT: return "a device-side wait gave up";
    case WG_E_NODRIVER: return "CUDA driver not available";
    case WG_E_LIMIT: return "size beyond the stated maximum";
    default: return code > 0 ? "CUDA error" : "unknown error";
  }
}
