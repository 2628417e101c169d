/* warpc_b200 -- C ABI of the B200-native fp16-in / fp32-out GEMM  C[M,N] = A[M,K] * Bt[N,K]^T.
 *
 * The reference (silares-ai/Warpc-public-release) has no C FFI: its operator surface is the
 * `warpc gemm M N K` command (backend/warpc.ml:19-52), the launch header that command writes
 * (backend/compile.ml:165-186, parsed by backend/node/header.py:12-32) and the launch / check /
 * time harness backend/node/run_tma.py:47-216.  This library is what a binding for that surface
 * calls: the rule and the header as functions, and the kernel behind a plan / launch pair.
 *
 * Conventions: every function returns 0 on success, > 0 a cudaError_t / CUresult value,
 * < 0 a library error (WG_E_*).  Callers own A, Bt and C; a plan owns its tensor maps,
 * hand-off flags and status words.  A plan is used from one host thread and one stream at a
 * time.  Every entry point that touches the GPU makes the plan's (or the named) device current
 * for the call and restores the caller's current device before it returns, so one thread may
 * drive plans on several GPUs.  Nothing synchronises unless stated.  There is no CPU fallback: without a CUDA device
 * every function that touches the GPU returns an error.
 */
#ifndef WARPC_B200_H
#define WARPC_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  WG_OK = 0,
  WG_E_SHAPE = -1,       /* the rule has no program for the shape (reference: OCaml failwith) */
  WG_E_VARIANT = -2,     /* inconsistent explicit variant (reference: gemm_swapped.ml:32-48 failwith) */
  WG_E_ARG = -3,         /* null / misaligned pointer, bad size, buffer too small */
  WG_E_NOKERNEL = -4,    /* no compiled kernel realises the variant */
  WG_E_DEVICE_WAIT = -5, /* a bounded device-side wait gave up; see wg_last_device_status */
  WG_E_NODRIVER = -6,    /* CUDA driver entry points not available (no GPU / no libcuda) */
  WG_E_LIMIT = -7        /* size beyond a stated maximum */
};

enum { WG_PROG_SWAPPED = 0, WG_PROG_PAIR = 1, WG_PROG_ONE = 2 };
enum { WG_SM_100A = 100, WG_SM_103A = 103 };

/* What the reference's rule decides for a shape, plus the geometry its kernel builder
 * derives from that decision.  Rule fields: backend/programs.ml:46-80 (the optional
 * arguments of Gemm_swapped.build, backend/gemm_swapped.mli:25-42).  Derived fields:
 * backend/gemm_swapped.ml:50-108. */
typedef struct wg_variant {
  int prog;                 /* WG_PROG_* */
  int tile_m, tile_n, tile_k, depth;
  int cluster_n;            /* pairs along the rows that share a B^T tile in the reference */
  int clc, ask_ahead, direct, serpentine, group;
  int streamk, split, split_grid, split_add, late_launch;
  int bufs;                 /* 0 = derive */
  /* derived, as the reference's builder computes them */
  int reps, atom_m, tmem_cols, nbuf, alloc_cols;
  int tiles_m, tiles_n, total_tiles, ctas, grid, persistent, kt;
  int a_box_rows, bt_box_rows, stage_bytes, tx_bytes, ref_dynsmem, ref_mbarriers, nflags;
  /* 1 (set by wg_choose): wg_realise may run the program on the tile this library measured
   * fastest on a B200 without TMA multicast; 0 (wg_derive): the tile named is the tile run. */
  int retile;
} wg_variant;

/* How this library launches a variant (its own kernel's contract, what wg_header prints). */
typedef struct wg_launch_info {
  int kernel_id;           /* index into the compiled kernel table */
  int cg, tile_m, tile_n, direct, epi_rows;
  int grid, cluster, threads, dynsmem, mbarriers, tmem_cols;
  int sched;               /* 0 one tile a CTA, 1 fixed grid by stride, 2 cluster launch control, 3 split-K over the grid, 4 stream-K */
  int depth, nbuf, group, cl_n, serpentine, ask_ahead, split, nflags;
  int a_box_rows, bt_box_rows, c_box_rows;
  int ksub, rounds;        /* the ring is handed over ksub k-steps (slots) at a time: rounds = depth / ksub barrier pairs */
  int wide_rows;           /* C rows per store of a CTA's last tile when it is staged whole in the drained ring, else 0 */
  int stage_bytes;         /* one ring slot: this CTA's A half-tile and B^T tile of one k-step */
  int staging_bytes;       /* the epilogue's cycling staging copies; 0 where every tile is staged in the drained ring */
  int ws_words;            /* fp32 words of workspace (a slot of tile_m x tile_n per CTA) when K is shared through a workspace, else 0 */
  int sk_dp;               /* stream-K: pair tiles walked whole, by stride (a multiple of the resident pairs); the k-steps of the rest are dealt out evenly */
} wg_launch_info;

/* `warpc gemm M N K`: the program chosen for a shape (backend/programs.ml:46-80).
 * sm is WG_SM_100A or WG_SM_103A (backend/warpc.ml:32-36). */
int wg_choose(int M, int N, int K, int sm, wg_variant* out);

/* `warpc swapped M N K TM TN DEPTH [flags]`, `warpc pair ...`, `warpc one ...`
 * (backend/warpc.ml:21-28): fill the rule fields of *v (zero the rest), then derive.
 * Returns WG_E_VARIANT where the reference's builder refuses the combination. */
int wg_derive(int M, int N, int K, wg_variant* v);

/* The kernel of this library that realises a variant, and its launch geometry. */
int wg_realise(const wg_variant* v, int M, int N, int K, wg_launch_info* out);

/* The launch header (`.kernel/.sm/.threads/.smem/.dynsmem/.tile/.tmap/.ptr/.grid/.mbarriers/
 * .cluster/.tcgen05/.params`, backend/compile.ml:171-186) as text; returns the length
 * written (excluding the terminator) or WG_E_ARG when cap is too small. */
int wg_header(const wg_variant* v, int M, int N, int K, char* buf, size_t cap);

/* A plan: tensor maps for dA (M x K fp16), dBt (N x K fp16), dC (M x N fp32), all row-major,
 * 16-byte aligned device pointers on `device`; hand-off flags and status words allocated and
 * zeroed once (backend/node/run_tma.py:88-113).  timeout_ms bounds every device-side wait
 * (0 = the default, 2000 ms). */
int wg_plan_create(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC,
                   void** plan);
/* The same for a product that is a COLUMN BLOCK of a wider C: dC points at the block's first entry and consecutive rows
 * of C are `ldc` fp32 words apart (ldc >= N, a multiple of 4).  dBt is then the block's N rows of the wider B^T.  Used to
 * run one problem as several launches side by side (no reference counterpart: its harness launches one kernel). */
int wg_plan_create_block(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC, int ldc,
                         void** plan);
int wg_plan_set_timeout_ms(void* plan, unsigned ms);
int wg_plan_info(void* plan, wg_launch_info* out);
/* One launch on `cuda_stream` (a cudaStream_t, NULL = the default stream); asynchronous. */
int wg_launch(void* plan, void* cuda_stream);
/* Synchronise the device and read the status words: out[0] = 0 when every launch so far ran
 * to completion, else the wait that gave up (role code), out[1] its detail, out[2] the CTA,
 * out[3] the parity / target.  Returns WG_E_DEVICE_WAIT when out[0] != 0. */
int wg_last_device_status(void* plan, unsigned out[4]);
/* Re-zero the flags and status words (after a launch that gave up). */
int wg_plan_reset(void* plan);
int wg_plan_destroy(void* plan);

/* A replicated C, fused into the GEMM (no counterpart in the reference, which runs on one GPU): `n` further copies of
 * this plan's C -- device pointers this process can write, typically other GPUs' memory opened through CUDA IPC with
 * peer access enabled, each M x N fp32 row-major with the same row pitch as dC.  Every launch that follows sends each
 * tile of C it has stored on to all of them (a warp of the kernel reads the tile back from this GPU's L2 and stores it
 * over NVLink while the next tiles are computed; a CTA's last tile goes out by TMA stores from its staged copy), so the
 * transfer overlaps the tensor cores' work; the copies are complete when the launch is.  Only for programs that store
 * through staging copies and do not share K between CTAs (one tile a CTA, fixed grid, launch control), with M and N
 * whole multiples of the tile; WG_E_VARIANT otherwise.
 * n = 0 turns it off.  No TMA load ever touches these pointers. */
int wg_plan_set_replicas(void* plan, int n, void* const* peer_dC);

/* Sharing a device buffer between the processes of one box (one process per GPU), for wg_plan_set_replicas: the owner
 * exports a pointer (anywhere inside an allocation) as 64 opaque bytes plus its offset inside the allocation; another
 * process imports it WITH ITS OWN DEVICE CURRENT (`device`), which maps the owner's memory into that device's address
 * space with peer access, and gets a pointer it may hand to wg_plan_set_replicas.  (CUDA IPC; an import of an allocation
 * this process has already imported returns the same mapping, counted.)  wg_ipc_release undoes one import.
 * Returns a cudaError_t / CUresult on failure, WG_E_ARG for a pointer that was not imported. */
int wg_ipc_export(int device, const void* dptr, unsigned char handle[64], unsigned long long* offset);
int wg_ipc_import(int device, const unsigned char handle[64], unsigned long long offset, void** dptr);
int wg_ipc_release(int device, void* dptr);

/* Host-buffer entry: a plan that owns device copies of A, Bt and C.  wg_host_run copies
 * hA, hBt in, launches, copies C out to hC and synchronises -- the call the reference's
 * harness makes around a launch (backend/node/run_tma.py:68-70, 142).  A large problem (>= 256 MB moved, M and N
 * multiples of 2048) runs as a pipeline instead of copy / launch / copy: C in blocks of 2048 x 2048, each the rule's
 * program for 2048 x 2048 x K, launched as its row panels of A and Bt land and copied out as it completes (pinned host
 * buffers make the three overlap; pageable ones still give the right C).  `v` then names only the one-shot program. */
int wg_host_plan_create(int device, const wg_variant* v, int M, int N, int K, void** plan);
int wg_host_run(void* plan, const void* hA, const void* hBt, void* hC);
/* device pointers of a host plan: which = 0 A, 1 Bt, 2 C */
void* wg_host_plan_buffer(void* plan, int which);

/* Mean milliseconds of `repeat` back-to-back launches between two CUDA events on the default
 * stream after `warmup` untimed ones (backend/node/run_tma.py:171-175, backend/node/cuda.py:79-92). */
int wg_time_launches(void* plan, int warmup, int repeat, float* ms_mean);

/* Dependent launch (backend/node/clusterlaunch.py:54-74 `pdl`, the AB_PDL mode of backend/node/ab.py:95-118): launches
 * that follow carry the programmatic-stream-serialization attribute, so a launch may begin while the one before it
 * in the stream runs; the kernel waits (griddepcontrol.wait) before it touches global memory. Off by default. */
int wg_plan_set_dependent_launch(void* plan, int on);

/* Timing builds (the reference's: backend/stamp.ml:9-16, decoded in run_tma.py:176-192): turn per-phase stamps on or
 * off for the launches that follow, and read them back: grid * 256 words, 64 events x 4 tiles per CTA. Events 0-10
 * and 16-21 are times on the GPU nanosecond timer (entry, set-up, first/last load, first/last MMA, accumulator ready,
 * stored, roles done, exit, accumulator free; barriers initialised, tensor memory allocated, first tile found, last
 * stores read, CTAs met, tensor memory freed); 11-14 cycle sums of the first epilogue warp; 15 cycles entry to exit.
 * wg_plan_read_stamps synchronises and returns the words written.  A plan whose kernel is one of the "simple"
 * instances (whole tiles, one a CTA or a fixed grid, stored from the registers: compiled without the stamps) launches
 * the full instance of the same tile and store while its stamps are on: same geometry, the timeline of the larger code. */
int wg_plan_enable_stamps(void* plan, int on);
int wg_plan_read_stamps(void* plan, unsigned long long* out, size_t cap_words);

/* Test hook for the bounded device-side waits (the reference's kernels spin without bound,
 * backend/sass.ml:339; its harness only has a reader for "waits that gave up",
 * backend/node/run_tma.py:129-137): overwrite hand-off word `index` of a split-K / stream-K plan. */
int wg_plan_debug_set_flag(void* plan, int index, unsigned value);

/* Tuning hook (no reference counterpart).  Bits 8-11: k-steps the ring hands over per barrier
 * round in the launches that follow (1, 2 or 4; results stay exact), 0 = the library's own
 * choice.  Bits 0-7 must be zero: they select modes that skip loads or MMAs to time one role
 * alone, and exist only in builds made with -DWB_TIMING_EXPERIMENTS. */
int wg_plan_debug_set_mode(void* plan, unsigned flags);

/* Where CTA tile index `tile` sits in C under a launch's tile walk (backend/tiles.ml:32-80). */
int wg_tile_origin(const wg_launch_info* li, int tile, int* row, int* col);

/* One launch that allocates nothing.  It has no counterpart in the reference (whose harness
 * allocates every buffer up front, backend/node/run_tma.py:68-95).  It is for callers that
 * cannot allocate device memory where they call: inside another framework's memory pool or a
 * fixed memory budget, in a latency-critical loop (cudaMalloc synchronises the device), or
 * after the application has given all free memory to its own allocator.  The kernel's own
 * words (split-K / stream-K hand-off flags, status) live in a device array built into the
 * library: wg_noalloc_max_flags() + 8 words (16 KiB + 32 B) held by every GPU that loads it.
 *   - v == NULL takes the rule's program for the shape (wg_choose); dA, dBt, dC as wg_plan_create.
 *   - WG_E_LIMIT when the program needs more hand-off words than wg_noalloc_max_flags(), or a
 *     workspace for partial sums (the explicitly named workspace forms of split-K / stream-K).
 *   - The first call on a device looks up the array's device address; make that call before
 *     any stream capture begins.
 *   - Every call on a device shares the array: the call clears the words it uses on `cuda_stream`
 *     ahead of its kernel, so calls on one stream are safe back to back, but two calls that
 *     overlap on the GPU (different streams, no dependency) race on it.
 *   - No cudaMalloc / cudaFree / allocating library routine is called.
 * wg_noalloc_status synchronises the device and reports the status words of the MOST RECENT call
 * only: each wg_launch_noalloc clears them on its stream (its waits read them), so a give-up must
 * be read before the next wg_launch_noalloc on that device -- unlike wg_last_device_status, which
 * is sticky across a plan's launches. */
int wg_launch_noalloc(int device, const wg_variant* v, int M, int N, int K, const void* dA, const void* dBt, void* dC,
                      void* cuda_stream);
int wg_noalloc_status(int device, unsigned out[4]);
int wg_noalloc_max_flags(void);

/* Number of compiled kernels and the name of each (for listing): one template, an instance per (CTA group, tile, store
 * path), "simple" instances of three tiles that hold nothing but the one-tile / fixed-grid path from the registers, and
 * three instances compiled for one scheduling mode each (stream-K, launch control, split-K over the grid). */
int wg_kernel_count(void);
const char* wg_kernel_name(int kernel_id);

const char* wg_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
