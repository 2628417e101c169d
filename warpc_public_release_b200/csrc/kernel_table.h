// The compiled kernel instances: which (cta group, tile, store path) each is and what its
// launch needs.  Filled in api.cu where the templates are instantiated.
#pragma once
#include <stddef.h>

struct wb_kernel_entry {
  int id;
  int cg, tile_m, tile_n, direct;
  int simple;          // whole tiles, one a CTA or by stride, stored from the registers: the kernel holds no other path
  int ksub;            // k-steps a ring round when the instance fixes it (0: a launch parameter)
  int mode;            // the one scheduling mode the instance is compiled for (-1: a launch parameter)
  int reps;            // stacked MMA atoms a CTA (2 for 256-column tiles)
  int epi_rows;        // C rows per epilogue block (the C tensor map's box rows)
  int wide_rows;       // C rows per store of a CTA's last tile, staged whole in the drained ring
  int ncols;           // tensor-memory columns of one accumulator
  int stage_bytes;     // shared memory of one ring stage
  size_t smem_fixed;   // alignment slack + staging + control block
  int staging_bytes;   // the epilogue warps' cycling staging copies (part of smem_fixed)
  const char* name;
  const void* fn;      // the __global__ function
};

const wb_kernel_entry* wb_find_kernel(int cg, int tile_m, int tile_n, int direct, int simple, int mode);
const wb_kernel_entry* wb_kernel_at(int id);
int wb_kernel_total();
