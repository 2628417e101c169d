// The fp16-in / fp32-out GEMM kernel, C[M,N] = A[M,K] * Bt[N,K]^T, hand-written for sm_100a.
//
// Orientation ("swapped", as the reference's gemm_swapped.ml:1-21 and gemm_one.ml:1-9
// describe it): the tile of B^T is the MMA's A operand and the tile of A its B operand,
// so a CTA's accumulator in tensor memory holds output COLUMNS as lanes and output ROWS
// as columns.  One tcgen05.ld then gives every lane of a warp 32 consecutive columns of
// one C row per register, and each register goes out as one contiguous 128-byte row
// segment -- no transpose through shared memory is needed.
//
// CG == 2: two CTAs of a cluster share each tcgen05.mma.cta_group::2; the CTAs sit side
// by side along the output's columns, each loading its own TN rows of B^T and half of
// the TM rows of A.  CG == 1: one CTA a 128 x 128 tile (the rule's last fallback).
//
// Warp roles (256 threads): warp 0 TMA producer, warp 1 MMA issuer (the pair leader's)
// and tensor-memory owner, warp 2 tile scheduler (cluster launch control), warp 3
// barrier set-up, warps 4-7 epilogue.  Every wait on a barrier or a flag is bounded:
// when it runs out the kernel records where in `status`, every other wait gives up at
// its next poll, and all warps fall through to the common teardown, so a protocol error
// never leaves the GPU spinning.
#pragma once
#include "sm100_ptx.cuh"
#include "tile_map.h"

namespace wb {

enum : int { SCHED_ONE = 0, SCHED_STRIDE = 1, SCHED_CLC = 2, SCHED_SPLITK = 3, SCHED_STREAMK = 4 };

// status[0] codes
enum : uint32_t {
  ST_OK = 0,
  ST_WAIT_EMPTY = 1,      // producer: ring stage never released
  ST_WAIT_FULL = 2,       // MMA warp: ring stage never filled
  ST_WAIT_ACC_EMPTY = 3,  // MMA warp: accumulator never released
  ST_WAIT_ACC_FULL = 4,   // epilogue: accumulator never completed
  ST_WAIT_SCHED = 5,      // a role: no answer from the scheduler
  ST_WAIT_SCHED_EMPTY = 6,
  ST_WAIT_CLC = 7,
  ST_WAIT_FLAG = 8,       // split-K / stream-K: a partner's flag never came up
  ST_TMEM = 9
};

struct KParams {
  int M, N, K;
  int ldc;        // fp32 words between rows of C (N, or more when C is a block of a wider matrix): the store from the registers
  int kt;         // K / 64 k-steps
  int ntiles;     // CTA tiles in all
  int cl_n;       // clusters (CG CTAs side by side) across the output
  int group;      // cluster rows walked down before moving across; a power of two
  int serp;       // odd bands of `group` rows run right to left
  int depth;      // ring stages
  int nbuf;       // accumulators in tensor memory (1 or 2)
  int sched;      // SCHED_*
  int ask_ahead;  // probe the next stage before releasing this one
  int split;      // SCHED_SPLITK: runs of K per tile
  int sk_q, sk_r, sk_clusters;  // SCHED_STREAMK: units = q * clusters + r
  int sk_dp;                    // SCHED_STREAMK: the first sk_dp cluster tiles (a multiple of the clusters) are walked whole, by stride,
                                // after the units of the rest have been dealt out evenly
  int staging_bytes;            // the cycling staging copies (0: every tile is a CTA's last and is staged in the ring)
  int l2_hints;                 // bit 0: C's lines leave the L2 first; bit 1: operand lines leave it last
  int late_launch;              // the next grid in the stream is let go when the producer's last load is out, not at entry
  int ksub, rounds;             // the ring is handed over `ksub` k-steps (slots) at a time: rounds = depth / ksub barrier pairs
  int epi_ring;                 // the ring holds a whole C tile: a CTA's last tile is staged there, one copy per block
  float* C;                     // direct store
  uint32_t* flags;              // split-K / stream-K hand-off words
  float* ws;                    // split-K / stream-K through a workspace: a slot of TM x TN partial sums per CTA
  const CUtensorMap* replicas;  // further copies of C (other GPUs' memory): per copy the block map and the wide map, in global memory
  float* const* rep_ptrs;       // the same copies' addresses (of this plan's C inside each), in global memory
  int nrep;                     // how many; every tile is sent on to each of them
  uint32_t* status;             // 8 words: [0] code, [1] site detail, [2] CTA, [3] parity/stage
  unsigned long long timeout_ns;
#ifdef WB_TIMING_EXPERIMENTS
  unsigned int debug;           // bit 0 the producer loads nothing, bit 1 no MMAs are issued, bits 4-5 flip the L2 hints
#endif
  unsigned long long* stamps;   // timing builds: 32 events x 4 tiles per CTA, or null
};

// Timing builds (-DWB_SIMPLE_STAMPS) keep the phase stamps in the simple instances too.
#ifdef WB_SIMPLE_STAMPS
constexpr bool kSimpleStamps = true;
#else
constexpr bool kSimpleStamps = false;
#endif

// Builds with -DWB_TIMING_EXPERIMENTS carry a word of switches that make a launch skip its loads or
// its MMAs (wrong results, for timing one role alone); the library as shipped has no such switch.
#ifdef WB_TIMING_EXPERIMENTS
#define WB_DEBUG_WORD(p) ((p).debug)
#else
#define WB_DEBUG_WORD(p) 0u
#endif

template <int CG_, int TM_, int TN_, bool DIRECT_, int EPI_ROWS_ = 32, int EPI_COPIES_ = 2, bool SIMPLE_ = false, int KSUB_ = 0, int MODE_ = -1>
struct Cfg {
  static constexpr int CG = CG_, TM = TM_, TN = TN_, TK = 64;
  static constexpr bool DIRECT = DIRECT_;
  // whole tiles, one a CTA or a fixed grid walking them by stride, stored from the registers, and nothing else: no launch
  // control, no K shared between CTAs, no further copies of C.  The launches that last ten to thirty microseconds are
  // these, and the code they never run is not in their kernel.
  static constexpr bool SIMPLE = SIMPLE_;
  // Simple instances of the small tiles rehearse their epilogue (epi_direct_tile) while the first k loop runs: measured,
  // one tile a CTA, 1024^3 7.6 -> 7.2 us (two blocks a warp: the code runs once), 1536^3 10.7 -> 10.4 (four blocks: the
  // loop's second turn finds it fetched anyway); eight blocks (256 x 128) gain nothing at 2048^3 and lose 0.45 us on the
  // fixed grid's four tiles at 4096 x 4096 x 1024, so those do not.
  static constexpr bool REHEARSE = SIMPLE_ && (TN_ == 256 ? 2 : 1) * ((CG_ == 2 && TN_ == 64 ? TM_ / 2 : TM_) / 32) <= 4;
  static constexpr int KSUB = KSUB_;  // k-steps a ring round, fixed at compile time (0: the launch says)
  // the one scheduling mode (SCHED_*) the instance is compiled for, or -1: the launch says.  An instance of one mode holds
  // no other mode's code (the walker's, the scheduler warp's, the epilogue's hand-offs), and none for further copies of C
  // where that mode cannot have them.
  static constexpr int MODE = MODE_;
  static constexpr bool REPLICAS = !DIRECT_ && !SIMPLE_ && (MODE_ < 0 || MODE_ <= 2);
  static_assert(!SIMPLE || DIRECT, "the simple instances store from the registers");
  static constexpr bool FOLD = (CG == 2 && TN == 64);  // M = 128 pair: 64 accumulator rows a CTA
  static constexpr int REPS = (TN == 256) ? 2 : 1;    // stacked MMA atoms
  static constexpr int MMA_M = (CG == 2) ? (FOLD ? 128 : 256) : 128;
  static constexpr int MMA_N = TM;
  static constexpr int SPAN = FOLD ? TM / 2 : TM;  // tensor-memory columns an atom's accumulator spans
  __host__ __device__ static constexpr int pow2_ge(int n) { int c = 32; while (c < n) c *= 2; return c; }
  static constexpr int NCOLS = pow2_ge(REPS * SPAN);  // columns of one accumulator
  static constexpr int A_ROWS = TM / CG;              // rows of A this CTA loads per stage
  static constexpr int B_ROWS = TN;                   // rows of B^T this CTA loads per stage
  static constexpr int A_BYTES = A_ROWS * TK * 2, B_BYTES = B_ROWS * TK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t TX_BYTES = CG * STAGE_BYTES;  // what lands on the leader's barrier per stage
  static constexpr int EPI_ROWS = DIRECT ? 32 : EPI_ROWS_;  // C rows per epilogue block
  static constexpr int EPI_COPY_BYTES = EPI_ROWS * 128;
  static constexpr int EPI_COPIES = EPI_COPIES_;  // staging copies a warp cycles through
  static constexpr int STAGING_BYTES = DIRECT ? 0 : 4 * EPI_COPIES * EPI_COPY_BYTES;
  static constexpr int CHUNKS = SPAN / EPI_ROWS;  // blocks per atom per warp
  static constexpr int NBLK = REPS * CHUNKS;
  // a CTA's last tile goes out in stores of WIDE_ROWS rows, from copies side by side in the drained ring
  static constexpr int WIDE_ROWS = DIRECT ? 32 : ((SPAN % 128 == 0) ? 128 : 64);
  static constexpr int WIDE_BLKS = WIDE_ROWS / EPI_ROWS;
  static constexpr int MAX_DEPTH = 16;
  static constexpr int CTRL_BYTES = 512;
  static_assert(A_BYTES % 1024 == 0 && B_BYTES % 1024 == 0, "ring slots keep the 1024-byte swizzle atom alignment");
  static_assert(SPAN % EPI_ROWS == 0 && SPAN % WIDE_ROWS == 0 && WIDE_ROWS % EPI_ROWS == 0, "whole epilogue blocks");
  static_assert((MMA_M == 128 && MMA_N % 16 == 0) || (MMA_M == 256 && MMA_N % 16 == 0), "UMMA shape");
  // kind::f16 instruction descriptor: f32 accumulator, f16 operands, both K-major
  static constexpr uint32_t IDESC = (1u << 4) | (uint32_t(MMA_N >> 3) << 17) | (uint32_t(MMA_M >> 4) << 24);
  static constexpr size_t smem_bytes(int depth) { return 1024 + size_t(depth) * STAGE_BYTES + STAGING_BYTES + CTRL_BYTES; }
};

// control block at the end of dynamic shared memory
struct Ctrl {
  uint32_t clc_answer[4];  // 16-byte aligned: written by the hardware, read with one 128-bit load
  uint64_t full[16];
  uint64_t empty[16];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t clc_bar;      // the cancel request's 16 bytes landed (scheduler's CTA)
  uint64_t sched_full;   // the decoded answer is in `sched_slot` (each CTA)
  uint64_t sched_empty;  // every taker has read it (first CTA)
  uint32_t sched_slot[2];  // valid, first CTA of the cancelled cluster
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t scratch;        // where a rehearsal of the epilogue (below) puts its stores
  uint64_t tmem_ready;     // pair leader's: the other CTA's tensor memory is allocated
  // a replicated C: the epilogue hands each tile it has stored to the forwarding warp through two slots
  uint64_t fwd_full[2];    // the four epilogue warps' stores of the slot's tile are written
  uint64_t fwd_empty[2];   // the forwarding warp has taken the slot's coordinates
  int32_t fwd_slot[2][2];  // row, column of the tile; row < 0: no more tiles
};
static_assert(sizeof(Ctrl) <= 512 && offsetof(Ctrl, clc_answer) % 16 == 0, "control block");


// K-major, 128-byte-swizzled operand tile: 8-row groups 1024 bytes apart.
WB_DEV uint64_t smem_desc(uint32_t addr) {
  return uint64_t((addr & 0x3FFFF) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}

WB_DEV uint32_t ld_shared_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
WB_DEV void st_shared_plain(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
WB_DEV void st_shared_u32(uint32_t addr, uint32_t v) { asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }

WB_DEV void record_failure(const KParams& p, uint32_t code, uint32_t detail, uint32_t parity) {
  if (atomicCAS(p.status, 0u, code) == 0u) {
    p.status[1] = detail;
    p.status[2] = blockIdx.x;
    p.status[3] = parity;
    __threadfence();
  }
}

// Phase stamps of a timing run (the reference's are backend/stamp.ml:9-16): event `ev` of
// the CTA's `slot`-th tile, on the GPU-wide nanosecond timer.
enum : int { EV_ENTRY = 0, EV_SETUP = 1, EV_LOAD_FIRST = 2, EV_LOAD_LAST = 3, EV_MMA_FIRST = 4, EV_MMA_LAST = 5,
             EV_ACC_READY = 6, EV_STORED = 7, EV_TEARDOWN = 8, EV_EXIT = 9, EV_ACC_FREE = 10 };
// 11-14: cycle sums of the first epilogue warp, 15: cycles entry to exit; 16 barriers initialised, 17 tensor memory
// allocated, 18 first tile found, 19 last stores have read their copies, 20 CTAs met at teardown, 21 tensor memory freed; 23 CTAs met at set-up, before the wait on the grid before; 22: cycles issuing the tcgen05.ld
// of the next block and releasing the accumulator (first epilogue warp)
WB_DEV void stamp_value(const KParams& p, int ev, int slot, long long value) {
  if (p.stamps != nullptr && slot < 4) p.stamps[(size_t(blockIdx.x) * 64 + ev) * 4 + slot] = (unsigned long long)value;
}
WB_DEV void stamp(const KParams& p, int ev, int slot) {
  if (p.stamps != nullptr && slot < 4) p.stamps[(size_t(blockIdx.x) * 64 + ev) * 4 + slot] = globaltimer();
}

// Bounded wait on an mbarrier phase.  Returns false when the kernel is giving up.
// WARP: called by a whole, converged warp (the outcome is made warp-uniform with a vote);
// otherwise by a single lane that runs its role alone (the TMA producer and the MMA issuer:
// one lane's try_wait is one request to the barrier unit, a warp's is thirty-two).
// The common case is one asm-internal spin.  Only when 4096 polls (each already sleeping in
// hardware) have failed does the waiter look at the abort words and the GPU-wide timer, which
// is slow to read.  CLUSTER: acquire at cluster scope (data another CTA stored before arriving).
template <bool CLUSTER, bool WARP>
__device__ __noinline__ bool wait_bar_timed(const KParams& p, uint32_t abort_addr, uint32_t bar, uint32_t parity, uint32_t code, uint32_t detail) {
  auto all = [](uint32_t ok) { return WARP ? (__all_sync(0xffffffffu, ok) != 0) : (ok != 0u); };
  auto any = [](bool bad) { return WARP ? (__any_sync(0xffffffffu, bad) != 0) : bad; };
  const uint64_t t0 = globaltimer();
  for (;;) {
    if (all(mbar_spin_wait<CLUSTER>(bar, parity, 64))) return true;
    uint32_t bad = ld_shared_u32(abort_addr) | ld_relaxed_gpu(p.status);
    const bool late = globaltimer() - t0 > p.timeout_ns;
    if (late && bad == 0u) record_failure(p, code, detail, parity);
    if (any(bad != 0u || late)) {
      st_shared_u32(abort_addr, 1u);
      return false;
    }
  }
}
// (the timed part is a function of its own, not inlined at the twenty places that wait: it runs only when something is badly late)
template <bool CLUSTER = false, bool WARP = true>
WB_DEV bool wait_bar(const KParams& p, uint32_t abort_addr, uint32_t bar, uint32_t parity, uint32_t code, uint32_t detail) {
  const uint32_t ok = mbar_spin_wait<CLUSTER>(bar, parity, 1u << 12);
  if (WARP ? (__all_sync(0xffffffffu, ok) != 0) : (ok != 0u)) return true;
  return wait_bar_timed<CLUSTER, WARP>(p, abort_addr, bar, parity, code, detail);
}

// Bounded wait until *flag == target (split-K / stream-K hand-off between CTAs).
WB_DEV bool wait_flag(const KParams& p, uint32_t abort_addr, const uint32_t* flag, uint32_t target, uint32_t detail) {
  uint32_t polls = 0;
  uint64_t t0 = 0;
  for (;;) {
    if (ld_relaxed_gpu(flag) == target) return true;
    if ((++polls & 255u) == 0u) {
      if (ld_shared_u32(abort_addr) != 0u) return false;
      if (ld_relaxed_gpu(p.status) != 0u) {
        st_shared_u32(abort_addr, 1u);
        return false;
      }
      const uint64_t now = globaltimer();
      if (t0 == 0) t0 = now;
      if (now - t0 > p.timeout_ns) {
        record_failure(p, ST_WAIT_FLAG, detail, target);
        st_shared_u32(abort_addr, 1u);
        return false;
      }
    }
  }
}

// The launch's scheduling mode and its number of further copies of C, as the instance sees them: constants where the
// instance is compiled for one mode, so the other modes' branches fold away.
template <class C>
WB_DEV int sched_of(const KParams& p) {
  if constexpr (C::MODE >= 0) return C::MODE;
  else return p.sched;
}
template <class C>
WB_DEV int nrep_of(const KParams& p) {
  if constexpr (C::REPLICAS) return p.nrep;
  else return 0;
}

// One unit of work for a role: an output tile and the k-steps [kb, ke) of it.
struct Work {
  int tile, kb, ke;
};

// The sequence of work units a CTA walks; every role of the CTA walks the same one.
template <class C>
struct Walker {
  const KParams& p;
  uint32_t abort_addr, sched_full, sched_slot, sched_empty_first;  // shared addresses (the last in the first CTA)
  uint32_t rank, lane;
  uint32_t sched_parity = 0;
  int tile = -1, seg = 0, t_first = 0, t_last = -1, kb_first = 0, ke_last = 0, dp_tile = 0;
  bool started = false, whole_tiles = false;

  WB_DEV Walker(const KParams& p_, uint32_t ctrl_addr, uint32_t rank_, uint32_t lane_) : p(p_), rank(rank_), lane(lane_) {
    abort_addr = ctrl_addr + offsetof(Ctrl, abort);
    sched_full = ctrl_addr + offsetof(Ctrl, sched_full);
    sched_slot = ctrl_addr + offsetof(Ctrl, sched_slot);
    sched_empty_first = mapa(ctrl_addr + offsetof(Ctrl, sched_empty), 0);
  }

  // WARP: called by a whole converged warp, else by one lane running its role alone
  template <bool WARP = true>
  WB_DEV bool next(Work& w) {
    const int sched = sched_of<C>(p);
    if (!started) {
      started = true;
      tile = blockIdx.x;
      w.tile = tile, w.kb = 0, w.ke = p.kt;
      if constexpr (C::SIMPLE) return tile < p.ntiles;
      if (sched == SCHED_SPLITK) {
        // cluster c is run (c mod S) of tile-cluster (c div S): k-steps [s q + s r / S, ...)
        const int c = blockIdx.x / C::CG, S = p.split, s = c % S, q = p.kt / S, r = p.kt % S;
        w.tile = (c / S) * C::CG + int(rank);
        w.kb = s * q + (s * r) / S;
        w.ke = (s + 1) * q + ((s + 1) * r) / S;
        return true;
      }
      if (sched == SCHED_STREAMK) {
        // cluster c owns units [c q + c r / G, (c+1) q + (c+1) r / G) of tiles x k-steps,
        // walked from its last tile down to its first
        // The shared part first, the whole tiles after it: the launch ends on a full wave of whole tiles in step
        // (its clusters read the same operand panels at the same time), and each cluster shares one or two tiles only.
        const int c = blockIdx.x / C::CG, G = p.sk_clusters;
        const int b = c * p.sk_q + (c * p.sk_r) / G, l = (c + 1) * p.sk_q + ((c + 1) * p.sk_r) / G - 1;
        dp_tile = c;
        t_first = b / p.kt, kb_first = b % p.kt, t_last = l / p.kt, ke_last = l % p.kt + 1;
        seg = t_last;
        if (l < b) seg = t_first - 1;  // no units of the shared part for this cluster
      } else {
        return tile < p.ntiles;
      }
    } else {
      if (sched == SCHED_ONE || sched == SCHED_SPLITK) return false;
      if (C::SIMPLE || sched == SCHED_STRIDE) {
        tile += gridDim.x;
        w.tile = tile, w.kb = 0, w.ke = p.kt;
        return tile < p.ntiles;
      }
      if (sched == SCHED_CLC) {
        if (!wait_bar<true, WARP>(p, abort_addr, sched_full, sched_parity, ST_WAIT_SCHED, 0)) return false;
        sched_parity ^= 1u;
        const uint32_t valid = ld_shared_u32(sched_slot), first = ld_shared_u32(sched_slot + 4);
        if (WARP) __syncwarp();
        if (lane == 0) mbar_arrive_cluster(sched_empty_first);
        if (!valid) return false;
        tile = int(first + rank);
        w.tile = tile, w.kb = 0, w.ke = p.kt;
        return true;
      }
      if (!whole_tiles) seg -= 1;  // stream-K
    }
    if (!whole_tiles && seg >= t_first) {
      w.tile = (p.sk_dp + seg) * C::CG + int(rank);
      w.kb = (seg == t_first) ? kb_first : 0;
      w.ke = (seg == t_last) ? ke_last : p.kt;
      return true;
    }
    whole_tiles = true;
    if (dp_tile >= p.sk_dp) return false;
    w.tile = dp_tile * C::CG + int(rank);
    w.kb = 0, w.ke = p.kt;
    dp_tile += p.sk_clusters;
    return true;
  }

  // `w` (the unit next() gave last) is known to be this CTA's final one.  Cluster launch
  // control only learns that from the answer after it, so it never says yes.
  WB_DEV bool is_last(const Work& w) const {
    const int sched = sched_of<C>(p);
    if (sched == SCHED_ONE || sched == SCHED_SPLITK) return true;
    if (C::SIMPLE || sched == SCHED_STRIDE) return w.tile + int(gridDim.x) >= p.ntiles;
    if (sched == SCHED_STREAMK) return whole_tiles ? dp_tile >= p.sk_dp : (seg == t_first && p.sk_dp == 0);
    return false;
  }
};

template <class C>
WB_DEV void tile_origin(const KParams& p, int tile, int& row, int& col) {
  wb_tile_origin(tile, C::CG, C::TM, C::TN, p.group, p.cl_n, p.serp, &row, &col);
}

// ------------------------------------------------------------------ epilogue pieces

// Issue the tcgen05.ld of block `i` of this warp: atom i / CHUNKS, rows chunk i % CHUNKS.
template <class C>
WB_DEV void epi_load(uint32_t tbase, int i, uint32_t* v) {
  const int r = i / C::CHUNKS, ch = i % C::CHUNKS;
  tmem_ld<C::EPI_ROWS>(tbase + uint32_t(r * C::SPAN + ch * C::EPI_ROWS), v);
}

// Output coordinates of block i, register 0, lane 0 for epilogue warp quarter q.
template <class C>
WB_DEV void epi_coords(int row, int col, int q, int i, int& y, int& x) {
  const int r = i / C::CHUNKS, ch = i % C::CHUNKS;
  if constexpr (C::FOLD) {
    // 64 accumulator rows a CTA: lanes 64-127 hold the upper half of the tile's rows
    x = col + 32 * (q & 1);
    y = row + (C::TM / 2) * (q >> 1) + ch * C::EPI_ROWS;
  } else {
    x = col + 128 * r + 32 * q;
    y = row + ch * C::EPI_ROWS;
  }
}

// One tile's accumulator out through the staging copies: each block loaded from tensor
// memory while the block before it is staged and handed to the copy engine.  `add` selects
// the reducing store (C += block, performed in the L2).  The accumulator is released on the
// leader's barrier as soon as the last block is in registers.  When the tile is the CTA's last
// and the operand ring (idle once the tile's accumulator is complete: every MMA that read it
// has retired) can hold it, every block gets a copy of its own there and no store is waited for.
template <class C>
WB_DEV void epi_staged_tile(const CUtensorMap* map_c, const CUtensorMap* map_cw, uint32_t tbase, uint32_t my_staging, int row, int col, int q, uint32_t lane,
                            bool add, uint32_t acc_empty_addr, uint64_t policy, uint32_t wide = 0, unsigned long long* prof = nullptr,
                            const CUtensorMap* replicas = nullptr, int nrep = 0) {
  uint32_t v[2][C::EPI_ROWS];
  long long t_ld = 0, t_copy = 0, t_sts = 0, t_tma = 0, t_issue = 0, t0 = 0;
  if (prof) t0 = clock64();
  epi_load<C>(tbase, 0, v[0]);
  if (prof) t_issue += clock64() - t0;
#pragma unroll
  for (int i = 0; i < C::NBLK; ++i) {
    if (prof) t0 = clock64();
    tmem_wait_ld();
    if (prof) t_ld += clock64() - t0;
    if (prof) t0 = clock64();
    if (i + 1 < C::NBLK) {
      epi_load<C>(tbase, i + 1, v[(i + 1) & 1]);
    } else {
      tc_fence_before();
      __syncwarp();
      if constexpr (C::CG == 2) mbar_arrive_cluster_relaxed_if(lane == 0 ? 1u : 0u, acc_empty_addr);
      else mbar_arrive_if(lane == 0 ? 1u : 0u, acc_empty_addr);
    }
    if (prof) t_issue += clock64() - t0;
    int y, x;
    epi_coords<C>(row, col, q, i, y, x);
    // `wide` != 0: this warp's NBLK private copies in the drained ring, nothing to wait for
    const uint32_t copy = wide != 0u ? wide + uint32_t(i) * C::EPI_COPY_BYTES : my_staging + uint32_t(i % C::EPI_COPIES) * C::EPI_COPY_BYTES;
    if (prof) t0 = clock64();
    if (wide == 0u) {
      bulk_wait_read<C::EPI_COPIES - 1>();  // the store that last read this copy is done with it (only the issuing lane has groups)
      __syncwarp();
    }
    if (prof) t_copy += clock64() - t0, t0 = clock64();
    // register j is one C row: the warp's 32 lanes write its 128 bytes side by side (no bank
    // conflict, so the staging box needs no swizzle)
    const uint32_t mine = copy + lane * 4u;
#pragma unroll
    for (int j = 0; j < C::EPI_ROWS; ++j) st_shared_plain(mine + uint32_t(j) * 128u, v[i & 1][j]);
    fence_proxy_async_smem();
    __syncwarp();
    if (prof) t_sts += clock64() - t0, t0 = clock64();
    // a replicated C: a CTA's last tile, staged whole in the drained ring, goes to every other copy (peer GPUs over NVLink)
    // from the same staged boxes; tiles that cycle through the two staging copies are sent on by the forwarding warp
    if (wide == 0u) {
      tma_store_commit_if(lane == 0 ? 1u : 0u, add ? 1u : 0u, map_c, x, y, copy, policy);
    } else if ((i + 1) % C::WIDE_BLKS == 0) {
      // the last WIDE_BLKS blocks are WIDE_ROWS consecutive rows of C and of the ring: one store
      for (int r = 0; r < nrep; ++r)
        tma_store_if(lane == 0 ? 1u : 0u, replicas + 2 * r + 1, x, y - (C::WIDE_BLKS - 1) * C::EPI_ROWS,
                     copy - uint32_t(C::WIDE_BLKS - 1) * C::EPI_COPY_BYTES, policy);
      tma_store_commit_if(lane == 0 ? 1u : 0u, add ? 1u : 0u, map_cw, x, y - (C::WIDE_BLKS - 1) * C::EPI_ROWS,
                          copy - uint32_t(C::WIDE_BLKS - 1) * C::EPI_COPY_BYTES, policy);
    }
    if (prof) t_tma += clock64() - t0;
  }
  if (prof && lane == 0) prof[0] = t_ld, prof[4] = t_copy, prof[8] = t_sts, prof[12] = t_tma, prof[44] = t_issue;  // events 11-14 and 22
}

// A replicated C, for a tile that went out through the two cycling staging copies.  The tile is stored to this GPU's C as
// always; the epilogue warps then hand its coordinates to the forwarding warp (warp 3, idle after set-up), which reads
// the tile back (it is still in the L2) and writes it to every other copy -- plain 16-byte loads and stores, the stores
// crossing NVLink -- while the epilogue and the MMA warp carry on with the next tiles.  The link takes what it takes: a
// burst of every CTA's tile at once, or more bytes a tile than a tile's time carries, only makes the forwarding warp run
// behind, not the epilogue (whose staging copies a TMA store to a peer would hold until the link had taken them).
//
// Epilogue side, all four warps: once this warp's stores of the tile are written (not just read out of the staging
// copies) it arrives on the slot's `full` barrier; the first warp puts the coordinates in the slot before it does, having
// waited for the forwarding warp to be done with the slot's use two tiles ago.  row < 0 says there are no more tiles.
WB_DEV bool fwd_hand_over(const KParams& p, uint32_t abort_addr, uint32_t ctrl, uint32_t& count, int row, int col, bool first_warp, uint32_t lane) {
  const uint32_t s = count & 1u, phase = (count >> 1) & 1u;
  const uint32_t slot = ctrl + uint32_t(offsetof(Ctrl, fwd_slot)) + 8u * s;
  bool ok = true;
  if (lane == 0 && row >= 0) {
    bulk_wait<0>();
    fence_proxy_async_global();  // written by the copy engine, read next by ordinary loads of another warp
  }
  if (first_warp) {
    ok = wait_bar(p, abort_addr, ctrl + uint32_t(offsetof(Ctrl, fwd_empty)) + 8u * s, phase ^ 1u, ST_WAIT_EMPTY, 0x300u + s);
    if (lane == 0) st_shared_u32(slot, uint32_t(row)), st_shared_u32(slot + 4u, uint32_t(col));
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(ctrl + uint32_t(offsetof(Ctrl, fwd_full)) + 8u * s);
  ++count;
  return ok;
}

// Forwarding warp: one CTA tile of this GPU's C (whole: the host refuses further copies of a C with ragged tiles) to every
// other copy, eight rows of loads in flight at a time.
template <class C>
WB_DEV void fwd_copy_tile(const KParams& p, int row, int col, uint32_t lane) {
  constexpr int ROW_BYTES = C::TN * 4, V = (ROW_BYTES + 511) / 512, BATCH = 8;
  const size_t ld = size_t(p.ldc);
  const bool live[2] = {int(lane) * 16 < ROW_BYTES, int(lane) * 16 + 512 < ROW_BYTES};
#pragma unroll 1
  for (int r0 = 0; r0 < C::TM; r0 += BATCH) {
    float4 v[BATCH][V];
    const size_t at = size_t(row + r0) * ld + size_t(col) + lane * 4u;
#pragma unroll
    for (int b = 0; b < BATCH; ++b)
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (live[j]) v[b][j] = __ldcg(reinterpret_cast<const float4*>(p.C + at + size_t(b) * ld + size_t(j) * 128));
    for (int r = 0; r < p.nrep; ++r) {
      float* dst = p.rep_ptrs[r] + at;
#pragma unroll
      for (int b = 0; b < BATCH; ++b)
#pragma unroll
        for (int j = 0; j < V; ++j)
          if (live[j]) *reinterpret_cast<float4*>(dst + size_t(b) * ld + size_t(j) * 128) = v[b][j];
    }
  }
}

// Straight from the registers: register j of a block is row y + j, the warp's lanes are 32
// consecutive columns, so each register goes out as one 128-byte row segment.
// `rehearsal` (a generic address of a word of this CTA's shared memory, or null): run the same instructions with every
// store going to that word and the accumulator not released.  A launch of one tile a CTA runs this code exactly once, at
// its very end, and pays for fetching it then; run once before, while the warp only waits for the k loop, it is in the
// instruction caches when it counts.  What the rehearsal reads from tensor memory is whatever is there.
template <class C>
WB_DEV void epi_direct_tile(const KParams& p, uint32_t tbase, int row, int col, int q, uint32_t lane, uint32_t acc_empty_addr,
                            float* rehearsal = nullptr) {
  uint32_t v[2][C::EPI_ROWS];
  const size_t ld = rehearsal ? size_t(0) : size_t(p.ldc);
  // whole tiles only (the host refuses the store from the registers otherwise): no bounds to test
  auto store = [&](int i, const uint32_t* regs) {
    int y, x;
    epi_coords<C>(row, col, q, i, y, x);
    float* dst = rehearsal ? rehearsal : p.C + size_t(y) * ld + size_t(x) + lane;
#pragma unroll
    for (int j = 0; j < C::EPI_ROWS; ++j) dst[size_t(j) * ld] = __uint_as_float(regs[j]);
  };
  auto release = [&]() {
    if (rehearsal) return;
    tc_fence_before();
    __syncwarp();
    if constexpr (C::CG == 2) mbar_arrive_cluster_relaxed_if(lane == 0 ? 1u : 0u, acc_empty_addr);
    else mbar_arrive_if(lane == 0 ? 1u : 0u, acc_empty_addr);
  };
  epi_load<C>(tbase, 0, v[0]);
  if constexpr (C::NBLK % 2 == 0) {
    // two blocks a turn of a loop that is not unrolled (the two register sets alternate): an eight-block tile's store is a
    // quarter of the code, which a launch of one tile a CTA runs exactly once, cold
#pragma unroll 1
    for (int i = 0; i < C::NBLK; i += 2) {
      tmem_wait_ld();
      epi_load<C>(tbase, i + 1, v[1]);
      store(i, v[0]);
      tmem_wait_ld();
      if (i + 2 < C::NBLK) epi_load<C>(tbase, i + 2, v[0]);
      else release();
      store(i + 1, v[1]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < C::NBLK; ++i) {
      tmem_wait_ld();
      if (i + 1 < C::NBLK) epi_load<C>(tbase, i + 1, v[(i + 1) & 1]);
      else release();
      store(i, v[i & 1]);
    }
  }
}

// One copy of that code per kernel, called (not inlined) from both places a simple instance uses it: the rehearsal warms
// the instruction caches only if the real store runs the same instructions at the same addresses.
template <class C>
__device__ __noinline__ void epi_direct_tile_once(const KParams& p, uint32_t tbase, int row, int col, int q, uint32_t lane, uint32_t acc_empty_addr,
                                                  float* rehearsal) {
  epi_direct_tile<C>(p, tbase, row, col, q, lane, acc_empty_addr, rehearsal);
}

// ------------------------------------------------------------------ K shared through a workspace
// The reference's other way of sharing a tile's K between CTAs (backend/gemm_swapped.ml:716-832): a CTA leaves its
// partial accumulator in its slot of a workspace in global memory, in the order its threads hold it (the "fragment
// order" of backend/store.ml:106-114: block, register, lane, so every store and every load is a whole 128-byte
// line), and one CTA per 32-row block adds the partial sums up in a fixed order and stores C.  Unlike sums added in
// the L2, the order of the additions does not depend on timing: every launch gives the same bits.

// word offset of register 0 of block i, epilogue warp quarter q, in a CTA's slot; register j is 32 words further on
template <class C>
WB_DEV size_t ws_offset(int i, int q, uint32_t lane) { return size_t(i * 4 + q) * (C::EPI_ROWS * 32) + lane; }

// This warp's blocks of the accumulator into the CTA's slot; with S > 1 the blocks run s will sum up itself stay behind.
template <class C>
WB_DEV void epi_ws_put(float* slot, uint32_t tbase, int q, uint32_t lane, int S, int s) {
  uint32_t v[C::EPI_ROWS];
#pragma unroll 1
  for (int i = 0; i < C::NBLK; ++i) {
    if (S > 1 && i * S / C::NBLK == s) continue;
    epi_load<C>(tbase, i, v);
    tmem_wait_ld();
    float* dst = slot + ws_offset<C>(i, q, lane);
#pragma unroll
    for (int j = 0; j < C::EPI_ROWS; ++j) dst[j * 32] = __uint_as_float(v[j]);
  }
}

// The blocks this CTA sums up (all of them when S == 1; with S > 1 block i belongs to run i S / NBLK): its own part
// from tensor memory plus the slots src0 + j * src_stride, j = 0 .. nsrc - 1 except `skip`, added in that order, then
// stored to C from the registers.  Releases the accumulator.
template <class C>
WB_DEV void epi_ws_sum(const KParams& p, uint32_t tbase, int row, int col, int q, uint32_t lane, uint32_t acc_empty_addr,
                       const float* src0, size_t src_stride, int nsrc, int skip, int S, int s) {
  uint32_t v[C::EPI_ROWS];
  const size_t ld = size_t(p.ldc);
#pragma unroll 1
  for (int i = 0; i < C::NBLK; ++i) {
    if (S > 1 && i * S / C::NBLK != s) continue;
    epi_load<C>(tbase, i, v);
    tmem_wait_ld();
    for (int j = 0; j < nsrc; ++j) {
      if (j == skip) continue;
      const float* src = src0 + size_t(j) * src_stride + ws_offset<C>(i, q, lane);  // written by another SM: read in the L2
#pragma unroll
      for (int r = 0; r < C::EPI_ROWS; ++r) v[r] = __float_as_uint(__fadd_rn(__uint_as_float(v[r]), __ldcg(src + r * 32)));
    }
    int y, x;
    epi_coords<C>(row, col, q, i, y, x);
    float* dst = p.C + size_t(y) * ld + size_t(x) + lane;
#pragma unroll
    for (int r = 0; r < C::EPI_ROWS; ++r) dst[size_t(r) * ld] = __uint_as_float(v[r]);
  }
  tc_fence_before();
  __syncwarp();
  if constexpr (C::CG == 2) mbar_arrive_cluster_relaxed_if(lane == 0 ? 1u : 0u, acc_empty_addr);
  else mbar_arrive_if(lane == 0 ? 1u : 0u, acc_empty_addr);
}

template <class C>
__global__ void __launch_bounds__(256, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_cw,
            const __grid_constant__ KParams p) {
  constexpr int CG = C::CG;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring = smem_base;
  const uint32_t staging = ring + uint32_t(p.depth) * C::STAGE_BYTES;
  const uint32_t ctrl = staging + uint32_t(p.staging_bytes);
  auto ctrl_at = [&](size_t off) { return ctrl + uint32_t(off); };
  const uint32_t abort_addr = ctrl_at(offsetof(Ctrl, abort));

  // warp index, cluster rank and (below) the tensor-memory base are the same in every lane: a
  // shuffle from lane 0 lets the compiler see that, so what the single-lane issue paths compute
  // from them can live in uniform registers
  const uint32_t warp = warp_uniform(threadIdx.x >> 5), lane = threadIdx.x & 31;
  const uint32_t rank = (CG == 2) ? warp_uniform(cluster_ctarank()) : 0u;
  const bool leader = (rank == 0);
  const int nbuf = p.nbuf, rounds = p.rounds, ksub = (C::KSUB != 0) ? C::KSUB : p.ksub;
  // the simple instances take no phase stamps (a plan that is asked for stamps launches the full instance of the same tile)
  auto stamp = [](const KParams& pp, int ev, int slot) {
    if constexpr (!C::SIMPLE || kSimpleStamps) wb::stamp(pp, ev, slot);
  };
  auto stamp_value = [](const KParams& pp, int ev, int slot, long long value) {
    if constexpr (!C::SIMPLE || kSimpleStamps) wb::stamp_value(pp, ev, slot, value);
  };
  const long long cycles_at_entry = C::SIMPLE ? 0 : clock64();
  // Dependent launch (the reference's PREEXIT / ACQBULK, backend/sass.ml:496-502, gemm_swapped.ml:169-172, 232, 368):
  // under the programmatic-stream-serialization launch attribute the next grid in the stream may
  // take SMs as this grid's CTAs leave, from this instruction on -- or, "late launch", once the
  // producer's last load is out, so its CTAs do not sit on idle SMs through this grid.  Without
  // the attribute both instructions do nothing.
  if (threadIdx.x == 0 && !p.late_launch) griddep_launch_dependents();
  if (threadIdx.x == 0) stamp(p, EV_ENTRY, 0);

  auto full_bar = [&](int s) { return ctrl_at(offsetof(Ctrl, full) + 8 * s); };
  auto empty_bar = [&](int s) { return ctrl_at(offsetof(Ctrl, empty) + 8 * s); };
  auto acc_full_bar = [&](int b) { return ctrl_at(offsetof(Ctrl, acc_full) + 8 * b); };
  auto acc_empty_bar = [&](int b) { return ctrl_at(offsetof(Ctrl, acc_empty) + 8 * b); };

  // ---------------------------------------------------------------- set-up
  if (warp == 3) {
    // one barrier (or pair of them) a lane, so the set-up is one instruction deep, not forty
    if (int(lane) < rounds) {
      mbar_init(full_bar(int(lane)), 1);   // the leader's one arrival stating the pair's bytes
      mbar_init(empty_bar(int(lane)), 1);  // one commit from the MMA warp
    } else if (lane == 16 || lane == 17) {
      mbar_init(acc_full_bar(int(lane) - 16), 1);        // one commit
      mbar_init(acc_empty_bar(int(lane) - 16), 4 * CG);  // every epilogue warp of the pair
    } else if (lane == 18) {
      // (the lanes of this warp take their branches one after the other: a simple instance, which has no launch control
      // and no forwarding warp, leaves those barriers alone, and the tensor maps' prefetch is warp 2's)
      if constexpr (!C::SIMPLE) {
        mbar_init(ctrl_at(offsetof(Ctrl, clc_bar)), 1);
        mbar_init(ctrl_at(offsetof(Ctrl, sched_full)), 1);
        // takers of an answer: a producer a CTA, the leader's MMA warp, four epilogue warps a CTA
        mbar_init(ctrl_at(offsetof(Ctrl, sched_empty)), CG + 1 + 4 * CG);
      }
      if constexpr (CG == 2) mbar_init(ctrl_at(offsetof(Ctrl, tmem_ready)), 1);  // the other CTA's warp 1
      st_shared_u32(abort_addr, 0u);
    } else if (!C::SIMPLE && (lane == 20 || lane == 21)) {
      mbar_init(ctrl_at(offsetof(Ctrl, fwd_full) + 8 * (lane - 20)), 4);   // the four epilogue warps
      mbar_init(ctrl_at(offsetof(Ctrl, fwd_empty) + 8 * (lane - 20)), 1);  // the forwarding warp
    }
    fence_mbar_init();
    __threadfence_block();  // the abort word, for this CTA's own warps (the arrival at the barrier below is a relaxed one)
    if (lane == 0) stamp(p, 16, 0);
  }
  if (warp == 2 && lane == 0) {
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    if constexpr (!C::DIRECT) prefetch_tmap(&map_c), prefetch_tmap(&map_cw);
  }
  // (a pair's CTAs allocate their tensor memory after they have arrived at the barrier below)
  if (CG == 1 && warp == 1) {
    tmem_alloc<CG>(ctrl_at(offsetof(Ctrl, tmem_base)), uint32_t(C::pow2_ge(C::NCOLS * nbuf)));
    tmem_relinquish<CG>();
    if (lane == 0) stamp(p, 17, 0);
  }
  // every role's first unit of work and its tile's origin, found while the barriers and the
  // tensor memory are being set up rather than after the CTAs have met
  Walker<C> walk(p, ctrl, rank, lane);
  Work w;
  bool have = walk.template next<true>(w);
  int row = 0, col = 0;
  if (have) tile_origin<C>(p, w.tile, row, col);
  if (threadIdx.x == 0) stamp(p, 18, 0);
  // (the producer's constants too: its first load goes out the sooner after the pair has met)
  const uint64_t load_policy = (warp != 0) ? 0ull : ((((WB_DEBUG_WORD(p) >> 4) ^ uint32_t(p.l2_hints)) & 2u) ? l2_policy_evict_last() : l2_policy_evict_normal());
  const uint32_t full_leader0 = (CG == 2) ? mapa(full_bar(0), 0) : full_bar(0);
  tc_fence_before();
  if constexpr (CG == 2) {
    // What one CTA needs to see of the other's set-up is its barriers' initialisation, which warp 3 has fenced
    // (fence.mbarrier_init.release.cluster) before this arrival; within the CTA, the tensor-memory base is ordered by the
    // tcgen05 fences either side and the abort word by warp 3's CTA-scope fence.  The arrival itself orders nothing
    // more: a releasing one put the pair's meeting at 1.06 us after entry, this one at 0.80.
    cluster_arrive_relaxed();
    // The paired tcgen05.alloc (each CTA into its own slot word) takes 0.15 us longer than the barriers' initialisation,
    // and nothing needs it before the first MMA, a microsecond on: warp 1 allocates between its arrival and its wait, so
    // the pair meets without it.  Its readers are told otherwise: this CTA's epilogue warps at a named barrier, the
    // leader's MMA lane (which writes into both CTAs' tensor memory) at a barrier of its own that the other CTA's
    // warp 1 arrives at.
    if (warp == 1) {
      tmem_alloc<CG>(ctrl_at(offsetof(Ctrl, tmem_base)), uint32_t(C::pow2_ge(C::NCOLS * nbuf)));
      tmem_relinquish<CG>();
      if (lane == 0) stamp(p, 17, 0);
      tc_fence_before();
      named_bar_arrive(3, 160);
    }
    cluster_wait();
    // (a relaxed arrival: tcgen05.alloc has returned, and the tcgen05 fences either side order it against the MMAs)
    if (warp == 1 && !leader) mbar_arrive_cluster_relaxed_if(lane == 0 ? 1u : 0u, mapa(ctrl_at(offsetof(Ctrl, tmem_ready)), 0));
  } else {
    __syncthreads();
  }
  tc_fence_after();
  if (threadIdx.x == 0) stamp(p, 23, 0);
  // nothing above touched global memory (a timing build's entry stamp aside); everything below
  // may read what the grid before this one wrote
  griddep_wait();
  if (CG == 2 && warp >= 4) {
    named_bar_sync(3, 160);
    tc_fence_after();
  }
  // (warp 1 and the epilogue warps use it; a pair's other warps may be here before it is written)
  const uint32_t tmem_base = (warp == 1 || warp >= 4) ? warp_uniform(ld_shared_u32(ctrl_at(offsetof(Ctrl, tmem_base)))) : 0u;
  if (threadIdx.x == 0) stamp(p, EV_SETUP, 0);

  // ---------------------------------------------------------------- roles
  bool arrived = false;  // this warp has already arrived at the teardown's cluster barrier
  if (warp == 0) {
    // ===== producer: TMA loads into this CTA's ring, counted on the leader's barrier.  One lane
    // runs the role; a tile's k-steps are one asm loop (load_k_loop), re-entered after the bounded,
    // timed wait whenever a slot stayed taken beyond the loop's own poll limit.
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      int nth = 0;
      bool ok = true;
      for (; ok && have; have = ok && walk.template next<false>(w)) {
        if (nth != 0) tile_origin<C>(p, w.tile, row, col);
        // a pair's CTAs sit side by side: same rows, so they split the A tile between them
        const int a_row = row + int(rank) * C::A_ROWS;
        uint32_t kleft = uint32_t(w.ke - w.kb);
        int x = w.kb * C::TK;
        stamp(p, EV_LOAD_FIRST, nth);
        while (kleft != 0u) {
          uint32_t gave_up;
          if ((C::KSUB == 0 || C::KSUB == 2) && ksub == 2)
            gave_up = load_rounds<CG, 2>(1u, kleft, uint32_t(rounds), stage, phase, x, empty_bar(0), full_bar(0), full_leader0, leader ? 1u : 0u,
                                         C::TX_BYTES, ring, 2u * C::STAGE_BYTES, uint32_t(C::A_BYTES), &map_a, a_row, &map_b, col, 1u << 14, WB_DEBUG_WORD(p),
                                         uint32_t(C::STAGE_BYTES), load_policy);
          else if ((C::KSUB == 0 || C::KSUB == 4) && ksub == 4)
            gave_up = load_rounds<CG, 4>(1u, kleft, uint32_t(rounds), stage, phase, x, empty_bar(0), full_bar(0), full_leader0, leader ? 1u : 0u,
                                         C::TX_BYTES, ring, 4u * C::STAGE_BYTES, uint32_t(C::A_BYTES), &map_a, a_row, &map_b, col, 1u << 14, WB_DEBUG_WORD(p),
                                         uint32_t(C::STAGE_BYTES), load_policy);
          else
            gave_up = load_k_loop<CG>(1u, kleft, uint32_t(rounds), stage, phase, x, empty_bar(0), full_bar(0), full_leader0, leader ? 1u : 0u,
                                      C::TX_BYTES, ring, uint32_t(C::STAGE_BYTES), uint32_t(C::A_BYTES), &map_a, a_row, &map_b, col, 1u << 14, WB_DEBUG_WORD(p), load_policy);
          if (gave_up != 0u && !wait_bar<false, false>(p, abort_addr, empty_bar(int(stage)), phase ^ 1u, ST_WAIT_EMPTY, stage)) {
            ok = false;
            break;
          }
        }
        stamp(p, EV_LOAD_LAST, nth);
        ++nth;
      }
      if (p.late_launch) griddep_launch_dependents();
      // every stage this CTA filled has been released before it leaves
      for (int i = 0; ok && i < rounds; ++i) {
        ok = wait_bar<false, false>(p, abort_addr, empty_bar(int(stage)), phase ^ 1u, ST_WAIT_EMPTY, 0x100u + stage);
        if (++stage == uint32_t(rounds)) stage = 0, phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===== MMA issuer: one lane of the pair leader's warp 1 issues for both CTAs; a tile's
    // k-steps are one asm loop (mma_k_loop): wait full[s], REPS x 4 MMAs, commit to empty[s].
    if (leader && lane == 0) {
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      int acc = 0, nth = 0;
      bool ok = true;
      constexpr uint16_t mask = (CG == 2) ? 0x3 : 0x1;
      // shared-memory descriptors: the high word is fixed (SBO 1024 B, version 1, 128-byte swizzle);
      // the low word is (address >> 4) | LBO field, so a stage, an atom or a 16-element k-step on
      // is a plain add to it
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4, ATOM16 = uint32_t((C::MMA_M / CG) * 128) >> 4;
      const uint32_t a_lo0 = ((ring & 0x3FFFFu) >> 4) | (1u << 16);  // stage 0's A tile (the MMA's B operand)
      const uint32_t b_lo0 = a_lo0 + (C::A_BYTES >> 4);              // stage 0's B^T tile (the MMA's A operand)
      // the other CTA's half of every accumulator exists (long since: the first operands are still on their way)
      if (CG == 2 && have) ok = wait_bar<false, false>(p, abort_addr, ctrl_at(offsetof(Ctrl, tmem_ready)), 0u, ST_WAIT_ACC_EMPTY, 0x200u);
      for (; ok && have; have = ok && walk.template next<false>(w)) {
        if (!wait_bar<false, false>(p, abort_addr, acc_empty_bar(acc), acc_phase ^ 1u, ST_WAIT_ACC_EMPTY, uint32_t(acc))) {
          ok = false;
          break;
        }
        tc_fence_after();
        stamp(p, EV_ACC_FREE, nth);
        const uint32_t d = tmem_base + uint32_t(acc * C::NCOLS);
        uint32_t kleft = uint32_t(w.ke - w.kb), accumulate = 0;
        // timing runs: when the tile's first round of operands has landed (the loop's own first poll then passes at once)
        if ((!C::SIMPLE || kSimpleStamps) && p.stamps != nullptr && !wait_bar<false, false>(p, abort_addr, full_bar(int(stage)), phase, ST_WAIT_FULL, stage)) {
          ok = false;
          break;
        }
        stamp(p, EV_MMA_FIRST, nth);
        while (kleft != 0u) {
          uint32_t gave_up;
          if (C::REPS == 1 && (C::KSUB == 0 || C::KSUB == 2) && ksub == 2)
            gave_up = mma_rounds<CG, 2>(1u, kleft, uint32_t(rounds), stage, phase, accumulate, full_bar(0), empty_bar(0), d, uint32_t(C::SPAN),
                                        b_lo0, STAGE16, a_lo0, 2u * STAGE16, DESC_HI, C::IDESC, 1u << 14, WB_DEBUG_WORD(p));
          else if (C::REPS == 1 && (C::KSUB == 0 || C::KSUB == 4) && ksub == 4)
            gave_up = mma_rounds<CG, 4>(1u, kleft, uint32_t(rounds), stage, phase, accumulate, full_bar(0), empty_bar(0), d, uint32_t(C::SPAN),
                                        b_lo0, STAGE16, a_lo0, 4u * STAGE16, DESC_HI, C::IDESC, 1u << 14, WB_DEBUG_WORD(p));
          else
            gave_up = mma_k_loop<CG, C::REPS>(1u, kleft, uint32_t(rounds), stage, phase, accumulate, full_bar(0), empty_bar(0), d, uint32_t(C::SPAN),
                                              b_lo0, ATOM16, a_lo0, STAGE16, DESC_HI, C::IDESC, 1u << 14, WB_DEBUG_WORD(p));
          if (gave_up != 0u && !wait_bar<false, false>(p, abort_addr, full_bar(int(stage)), phase, ST_WAIT_FULL, stage)) {
            ok = false;
            break;
          }
        }
        if (!ok) break;
        umma_commit<CG>(acc_full_bar(acc), mask);  // the accumulator is complete in both CTAs
        stamp(p, EV_MMA_LAST, nth);
        if (++acc == nbuf) acc = 0, acc_phase ^= 1u;
        ++nth;
      }
      // every accumulator has been read out in both CTAs before leaving
      for (int i = 0; ok && i < nbuf; ++i) {
        ok = wait_bar<false, false>(p, abort_addr, acc_empty_bar(acc), acc_phase ^ 1u, ST_WAIT_ACC_EMPTY, 0x100u + uint32_t(acc));
        if (++acc == nbuf) acc = 0, acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ===== scheduler (cluster launch control): the cluster's first CTA asks for one more
    // cluster's tiles at a time and hands the answer to every taker of both CTAs
    if (!C::SIMPLE && sched_of<C>(p) == SCHED_CLC && leader) {
      const uint32_t clc_bar = ctrl_at(offsetof(Ctrl, clc_bar)), answer = ctrl_at(offsetof(Ctrl, clc_answer));
      const uint32_t sched_empty = ctrl_at(offsetof(Ctrl, sched_empty));
      uint32_t pf = 0, pe = 0;
      for (;;) {
        if (!wait_bar(p, abort_addr, sched_empty, pe ^ 1u, ST_WAIT_SCHED_EMPTY, 0)) break;
        pe ^= 1u;
        if (lane == 0) {
          mbar_arrive_expect_tx(clc_bar, 16);
          clc_try_cancel(answer, clc_bar);
        }
        __syncwarp();
        if (!wait_bar(p, abort_addr, clc_bar, pf, ST_WAIT_CLC, 0)) break;
        pf ^= 1u;
        uint32_t first = 0;
        const uint32_t valid = clc_decode(answer, &first);
        fence_proxy_async_smem();  // this read of the answer before the next request's write
        __syncwarp();
        if (lane == 0) {
          for (uint32_t r = 0; r < uint32_t(CG); ++r) {
            const uint32_t slot = mapa(ctrl_at(offsetof(Ctrl, sched_slot)), r);
            st_cluster_u32(slot, valid);
            st_cluster_u32(slot + 4, first);
            mbar_arrive_cluster(mapa(ctrl_at(offsetof(Ctrl, sched_full)), r));
          }
        }
        __syncwarp();
        if (!valid) break;
      }
    }
  } else if (warp == 3) {
    // ===== forwarding warp (a replicated C): tiles the epilogue has stored, on to the other GPUs' copies
    if constexpr (!C::DIRECT) {
      if (nrep_of<C>(p) > 0) {
        for (uint32_t taken = 0;; ++taken) {
          const uint32_t s = taken & 1u, phase = (taken >> 1) & 1u;
          if (!wait_bar(p, abort_addr, ctrl_at(offsetof(Ctrl, fwd_full) + 8 * s), phase, ST_WAIT_FULL, 0x300u + s)) break;
          const int t_row = int(ld_shared_u32(ctrl_at(offsetof(Ctrl, fwd_slot) + 8 * s)));
          const int t_col = int(ld_shared_u32(ctrl_at(offsetof(Ctrl, fwd_slot) + 8 * s + 4)));
          __syncwarp();
          if (lane == 0) mbar_arrive(ctrl_at(offsetof(Ctrl, fwd_empty) + 8 * s));
          if (t_row < 0) break;
          fwd_copy_tile<C>(p, t_row, t_col, lane);
        }
      }
    }
  } else if (warp >= 4) {
    // ===== epilogue: tensor memory -> registers -> C
    const int q = int(warp & 3u);
    const bool first_warp = (warp == 4);
    int acc = 0, nth = 0;
    uint32_t acc_phase = 0, handed = 0;
    bool ok = true;
    const uint32_t acc_empty_leader = (CG == 2) ? mapa(acc_empty_bar(0), 0) : acc_empty_bar(0);
    const uint64_t store_policy = (((WB_DEBUG_WORD(p) >> 4) ^ uint32_t(p.l2_hints)) & 1u) ? l2_policy_evict_first() : l2_policy_evict_normal();
    const uint32_t my_staging = staging + uint32_t(q) * uint32_t(C::EPI_COPIES) * C::EPI_COPY_BYTES;
    // K split between CTAs (split-K over the grid, stream-K): hand-off words count launches,
    // never reset: every CTA's own word holds how many launches have gone by, so one past it
    // is the value all flags of this launch reach (gemm_swapped.ml:608-626)
    const bool shared_k = !C::DIRECT && (sched_of<C>(p) == SCHED_SPLITK || sched_of<C>(p) == SCHED_STREAMK);
    // the same sharing through a workspace (store from the registers): split-K counts launches in the CTA's word like
    // the L2 form; stream-K raises the word to 1 and the CTA that takes the partial sum puts it back to 0
    const bool ws_k = C::DIRECT && !C::SIMPLE && (sched_of<C>(p) == SCHED_SPLITK || sched_of<C>(p) == SCHED_STREAMK);
    float* ws_slot = ws_k ? p.ws + size_t(blockIdx.x) * size_t(C::TM * C::TN) : nullptr;
    uint32_t target = 0;
    if (ws_k && sched_of<C>(p) == SCHED_SPLITK) target = ld_relaxed_gpu(p.flags + blockIdx.x) + 1u;
    if (shared_k) {
      target = ld_relaxed_gpu(p.flags + blockIdx.x) + 1u;
      if (sched_of<C>(p) == SCHED_STREAMK) {
        named_bar_sync(2, 128);  // every epilogue thread has read the word before it moves on
        if (first_warp && lane == 0) st_relaxed_gpu(p.flags + blockIdx.x, target);
      }
    }
    if constexpr (C::REHEARSE) {
      // the epilogue's code once through while there is nothing to do but wait for the first tile's k loop
      if (have) epi_direct_tile_once<C>(p, tmem_base + (uint32_t(q * 32) << 16), row, col, q, lane, 0u,
                                        reinterpret_cast<float*>(__cvta_shared_to_generic(size_t(ctrl_at(offsetof(Ctrl, scratch))))));
    }
    for (; have; have = walk.template next<true>(w)) {
      if (nth != 0) tile_origin<C>(p, w.tile, row, col);
      const uint32_t wide = (p.epi_ring != 0 && walk.is_last(w)) ? ring + uint32_t(q) * uint32_t(C::NBLK) * C::EPI_COPY_BYTES : 0u;
      const uint32_t tbase = tmem_base + uint32_t(acc * C::NCOLS) + (uint32_t(q * 32) << 16);
      const uint32_t acc_empty_addr = acc_empty_leader + 8u * uint32_t(acc);
      if constexpr (C::DIRECT) {
        if (ws_k && sched_of<C>(p) == SCHED_SPLITK) {
          // ---- split-K through the workspace (gemm_swapped.ml:737-791): every run leaves the blocks it does not sum up
          // itself in its slot and raises its flag; once the tile's other runs' flags are up it adds their parts of its
          // own blocks, in run order, and stores them.  No warp leaves this block early: all four meet at the barriers.
          const int S = p.split, c = int(blockIdx.x) / CG, s = c % S, base = (c / S) * S;
          ok = wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
          tc_fence_after();
          if (first_warp && lane == 0) stamp(p, EV_ACC_READY, nth);
          if (ok) epi_ws_put<C>(ws_slot, tbase, q, lane, S, s);
          __threadfence();  // every store of the partial is visible GPU-wide before the flag
          named_bar_sync(2, 128);
          if (ok && first_warp && lane == 0) st_relaxed_gpu(p.flags + blockIdx.x, target);
          if (first_warp) {
            for (int j = int(lane); ok && j < S; j += 32)
              if (j != s) ok = wait_flag(p, abort_addr, p.flags + (base + j) * CG + int(rank), target, uint32_t(j));
          }
          fence_acq_rel_gpu();
          named_bar_sync(2, 128);
          ok = ok && (ld_shared_u32(abort_addr) == 0u);
          if (ok) epi_ws_sum<C>(p, tbase, row, col, q, lane, acc_empty_addr, p.ws + size_t(base * CG + int(rank)) * size_t(C::TM * C::TN),
                                size_t(CG) * size_t(C::TM * C::TN), S, s, S, s);
        } else if (ws_k && w.ke < p.kt) {
          // ---- stream-K through the workspace (gemm_swapped.ml:793-832): a segment that ends before its tile does leaves
          // its partial in this CTA's slot and raises this CTA's word
          ok = wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
          tc_fence_after();
          if (ok) {
            epi_ws_put<C>(ws_slot, tbase, q, lane, 1, 0);
            tc_fence_before();
            __syncwarp();
            if constexpr (CG == 2) mbar_arrive_cluster_relaxed_if(lane == 0 ? 1u : 0u, acc_empty_addr);
            else mbar_arrive_if(lane == 0 ? 1u : 0u, acc_empty_addr);
          }
          __threadfence();
          named_bar_sync(2, 128);
          if (ok && first_warp && lane == 0) st_relaxed_gpu(p.flags + blockIdx.x, 1u);
        } else if (ws_k && w.kb != 0) {
          // ... and the segment that starts after its tile does (the next cluster's: every cluster holds a tile's worth of
          // k-steps at least, so a tile has two parts at most) waits for that word, puts it back, and adds the slot
          uint32_t* before = p.flags + blockIdx.x - CG;
          if (first_warp) ok = wait_flag(p, abort_addr, before, 1u, uint32_t(w.tile));
          fence_acq_rel_gpu();
          named_bar_sync(2, 128);
          ok = ok && (ld_shared_u32(abort_addr) == 0u);
          if (ok && first_warp && lane == 0) st_relaxed_gpu(before, 0u);
          ok = ok && wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
          tc_fence_after();
          if (ok) epi_ws_sum<C>(p, tbase, row, col, q, lane, acc_empty_addr, ws_slot - size_t(CG) * size_t(C::TM * C::TN), 0, 1, -1, 1, 0);
        } else {
          if (!wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc))) break;
          tc_fence_after();
          if (first_warp && lane == 0) stamp(p, EV_ACC_READY, nth);
          if constexpr (C::REHEARSE) epi_direct_tile_once<C>(p, tbase, row, col, q, lane, acc_empty_addr, nullptr);
          else epi_direct_tile<C>(p, tbase, row, col, q, lane, acc_empty_addr);
        }
      } else if (!shared_k || (sched_of<C>(p) == SCHED_STREAMK && w.kb == 0 && w.ke == p.kt)) {
        // (a tile one cluster computes whole has no other part to wait for or to tell: stored like any tile)
        if (!wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc))) break;
        tc_fence_after();
        if (first_warp && lane == 0) stamp(p, EV_ACC_READY, nth);
        // timing runs: the first warp's cycles in each part of the tile's store, events 11-14
        unsigned long long* prof = (!C::SIMPLE && p.stamps != nullptr && first_warp && nth < 4) ? p.stamps + (size_t(blockIdx.x) * 64 + 11) * 4 + nth : nullptr;
        epi_staged_tile<C>(&map_c, &map_cw, tbase, my_staging, row, col, q, lane, false, acc_empty_addr, store_policy, wide, prof, p.replicas, nrep_of<C>(p));
        if (nrep_of<C>(p) > 0 && wide == 0u) ok = fwd_hand_over(p, abort_addr, ctrl, handed, row, col, first_warp, lane);
      } else if (sched_of<C>(p) == SCHED_SPLITK) {
        // ---- split-K over the grid, adding in the L2 (gemm_swapped.ml:660-710).  The S runs
        // of a tile first zero disjoint shares of it (while their k loops run), raise their
        // flags, and once all S flags are up each adds its whole accumulator to C.
        // No warp leaves this block early: all four meet at the named barriers.
        const int S = p.split, c = int(blockIdx.x) / CG, s = c % S;
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < C::EPI_ROWS; ++j) st_shared_u32(my_staging + uint32_t(j) * 128u + lane * 4u, 0u);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          for (int i = 0; i < C::NBLK; ++i) {
            if (i * S / C::NBLK != s) continue;
            int y, x;
            epi_coords<C>(row, col, q, i, y, x);
            tma_store_2d(&map_c, x, y, my_staging);
          }
          bulk_commit();
          bulk_wait<0>();  // the zeros are written, not just read out of shared memory
          fence_proxy_async_global();
        }
        __syncwarp();
        fence_acq_rel_gpu();
        named_bar_sync(2, 128);
        if (first_warp && lane == 0) st_relaxed_gpu(p.flags + blockIdx.x, target);
        ok = wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
        tc_fence_after();
        if (first_warp && lane == 0) stamp(p, EV_ACC_READY, nth);
        if (first_warp) {
          // the flags of the tile's S runs, same rank: lane j polls run j's
          const int base = (c / S) * S;
          for (int j = int(lane); ok && j < S; j += 32)
            ok = wait_flag(p, abort_addr, p.flags + (base + j) * CG + int(rank), target, uint32_t(j));
        }
        fence_acq_rel_gpu();
        fence_proxy_async_global();
        named_bar_sync(2, 128);
        ok = ok && (ld_shared_u32(abort_addr) == 0u);
        if (ok) epi_staged_tile<C>(&map_c, &map_cw, tbase, my_staging, row, col, q, lane, true, acc_empty_addr, store_policy, wide);
      } else {
        // ---- stream-K, adding in the L2 (gemm_swapped.ml:633-659): the segment holding the
        // tile's first k-step stores and raises the tile's flag; the others wait for it and add.
        uint32_t* tile_flag = p.flags + gridDim.x + w.tile;
        if (w.kb == 0) {
          ok = wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
          tc_fence_after();
          if (ok) epi_staged_tile<C>(&map_c, &map_cw, tbase, my_staging, row, col, q, lane, false, acc_empty_addr, store_policy, wide);
          if (lane == 0) {
            bulk_wait<0>();
            fence_proxy_async_global();
          }
          __syncwarp();
          fence_acq_rel_gpu();
          named_bar_sync(2, 128);
          if (ok && first_warp && lane == 0) st_relaxed_gpu(tile_flag, target);
        } else {
          if (first_warp) ok = wait_flag(p, abort_addr, tile_flag, target, uint32_t(w.tile));
          fence_acq_rel_gpu();
          fence_proxy_async_global();
          named_bar_sync(2, 128);
          ok = ok && (ld_shared_u32(abort_addr) == 0u);
          ok = ok && wait_bar(p, abort_addr, acc_full_bar(acc), acc_phase, ST_WAIT_ACC_FULL, uint32_t(acc));
          tc_fence_after();
          if (ok) epi_staged_tile<C>(&map_c, &map_cw, tbase, my_staging, row, col, q, lane, true, acc_empty_addr, store_policy, wide);
        }
      }
      if (!ok) break;
      if (first_warp && lane == 0) stamp(p, EV_STORED, nth);
      if (++acc == nbuf) acc = 0, acc_phase ^= 1u;
      ++nth;
    }
    if constexpr (!C::DIRECT) {
      if (nrep_of<C>(p) > 0) fwd_hand_over(p, abort_addr, ctrl, handed, -1, 0, first_warp, lane);  // the forwarding warp may leave
      // this warp is done with its partner CTA (its last word there was the accumulator's
      // release): it says so before waiting for its own stores, not after
      if (CG == 2 && ld_shared_u32(abort_addr) == 0u) {
        tc_fence_before();
        cluster_arrive_relaxed();
        arrived = true;
      }
      if (lane == 0) bulk_wait_read<0>();  // the last stores have read their staging copies
      __syncwarp();
      if (first_warp && lane == 0) stamp(p, 19, 0);
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (threadIdx.x == 0) stamp(p, EV_TEARDOWN, 0);
  if (ld_shared_u32(abort_addr) != 0u) {
    // giving up: let copies and MMAs in flight land before the shared and tensor memory go away
    const uint64_t t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  if constexpr (CG == 2 && !C::SIMPLE) {
    // the pair's CTAs meet before either leaves: launch control's last answer is released on the first CTA's barrier by
    // takers of both CTAs, and nobody waits for that
    if (!arrived) cluster_arrive_relaxed();
    cluster_wait();
  } else {
    // A simple instance's CTA leaves when its own roles are done, after a barrier of its own threads (tensor memory is
    // freed once its epilogue warps have read it out).  Every word the other CTA sends it has been waited for by one of
    // its roles by then: the loads that report to the leader's full barriers by its MMA issuer, the commits on both CTAs'
    // empty and accumulator barriers by their producers and epilogue warps, the other CTA's four releases of the
    // accumulator by the leader's MMA issuer's last wait; and the MMAs that read its ring and write its tensor memory
    // are complete when those commits arrive.  (Checked on the host: protocol.py, teardown="cta".)  Measured: 0.1-0.25 us
    // off a launch of eight to thirty; letting the warps leave one by one, with no barrier at all and an mbarrier for
    // the tensor memory, measured the same as this.
    __syncthreads();
  }
  if (threadIdx.x == 0) stamp(p, 20, 0);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, uint32_t(C::pow2_ge(C::NCOLS * nbuf)));
    if (lane == 0) stamp(p, 21, 0);
  }
  if (threadIdx.x == 0) stamp(p, EV_EXIT, 0), stamp_value(p, 15, 0, clock64() - cycles_at_entry);
}

}  // namespace wb
