// Inline-PTX wrappers for the Blackwell (sm_100a) instructions the GEMM kernels use:
// mbarriers, TMA tiled copies, tcgen05 (MMA, commit, tensor-memory alloc/ld),
// cluster barriers and cluster launch control.
//
// The reference generates these same instructions from its SASS-to-PTX lifter
// (backend/lift.ml:211-447 lists which PTX each kernel step is); here each is a
// one-line device function so the kernels read as CUDA C++.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wb {

#define WB_DEV __device__ __forceinline__

WB_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

WB_DEV uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

WB_DEV uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Dependent launch: let the next grid in the stream be scheduled / wait for the grids before this one.
WB_DEV void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
WB_DEV void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Address of the same shared-memory offset in CTA `rank` of this cluster.
WB_DEV uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

// ---------------------------------------------------------------- mbarrier
WB_DEV void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
WB_DEV void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

WB_DEV void mbar_arrive_expect_tx(uint32_t bar, uint32_t tx) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx) : "memory");
}
WB_DEV void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// `bar` is a shared::cluster address (from mapa): an arrival on another CTA's barrier.
WB_DEV void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// CTA-scope acquire (the default): enough for data landed by TMA / released by tcgen05.commit,
// and cheap -- these waits sit on the ring's critical path.
WB_DEV uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Cluster-scope acquire: for words another CTA of the cluster wrote with ordinary stores
// before its remote arrive (the scheduler's forwarded answer).
WB_DEV uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
WB_DEV uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Spin on a barrier phase inside one asm block (no compiler-visible branch on a per-thread
// value, so the code around it stays provably warp-uniform): up to `limit` try_waits, each of
// which already sleeps in hardware.  Returns 1 when the phase completed.
template <bool CLUSTER>
WB_DEV uint32_t mbar_spin_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
  uint32_t ok;
  if constexpr (CLUSTER) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
        "WB_SPIN:\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WB_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra WB_SPIN;\n"
        "WB_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(limit)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .u32 n;\n\tmov.u32 n, 0;\n"
        "WB_SPIN:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WB_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 q, n, %3;\n\t"
        "@q bra WB_SPIN;\n"
        "WB_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(limit)
        : "memory");
  }
  return ok;
}

// A value every lane of a converged warp holds alike, in a form the compiler can see is uniform.
WB_DEV uint32_t warp_uniform(uint32_t v) { return __shfl_sync(0xffffffffu, v, 0); }

// ---------------------------------------------------------------- fences
WB_DEV void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
WB_DEV void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
WB_DEV void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
WB_DEV void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
WB_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
WB_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

WB_DEV void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
WB_DEV void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Arrival that orders nothing: for the barrier the CTAs of a pair meet at before they leave.  Every word one CTA writes
// into the other's shared or tensor memory has been waited for by its reader by then; a releasing arrival would hold each
// thread until its own global stores (a tile of C from the registers) had been performed.
WB_DEV void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }

WB_DEV void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// a warp that only announces (it does not wait for the others of the barrier)
WB_DEV void named_bar_arrive(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------- flags in global memory
WB_DEV uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
WB_DEV void st_relaxed_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---------------------------------------------------------------- TMA
WB_DEV void prefetch_tmap(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Tiled 2-D load global -> this CTA's shared memory. With CG == 2 the completion
// bytes may be counted on the pair leader's barrier (`bar` is then a shared::cluster
// address); no multicast is ever used.
template <int CG>
WB_DEV void tma_load_2d(uint32_t dst, const void* map, int x, int y, uint32_t bar) {
  if constexpr (CG == 2) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}

WB_DEV void tma_store_2d(const void* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
// The copy engine's reducing store: C[box] += smem box, performed in the L2.
WB_DEV void tma_reduce_add_2d(const void* map, int x, int y, uint32_t src) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
WB_DEV void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
WB_DEV void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
WB_DEV void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tensor memory
template <int CG>
WB_DEV void tmem_alloc(uint32_t slot, uint32_t ncols) {
  if constexpr (CG == 2)
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
}
template <int CG>
WB_DEV void tmem_relinquish() {
  if constexpr (CG == 2)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int CG>
WB_DEV void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 2)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA (pair).
template <int CG>
WB_DEV void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (CG == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Arrive on `bar` (same shared-memory offset in every CTA of `mask`) once all MMAs
// this thread issued before have completed.
template <int CG>
WB_DEV void umma_commit(uint32_t bar, uint16_t mask) {
  if constexpr (CG == 2) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(mask)
        : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

WB_DEV void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// tcgen05.ld.32x32b: the warp reads its quarter's 32 lanes; lane l gets N consecutive
// columns of tensor-memory lane (quarter*32 + l) into N registers.
WB_DEV void tmem_ld_x8(uint32_t taddr, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
WB_DEV void tmem_ld_x16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
WB_DEV void tmem_ld_x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
template <int N>
WB_DEV void tmem_ld(uint32_t taddr, uint32_t* v) {
  static_assert(N == 8 || N == 16 || N == 32, "tcgen05.ld width");
  if constexpr (N == 8) tmem_ld_x8(taddr, v);
  if constexpr (N == 16) tmem_ld_x16(taddr, v);
  if constexpr (N == 32) tmem_ld_x32(taddr, v);
}

// ---------------------------------------------------------------- predicated single-lane issue
// The instructions one lane issues for its warp (TMA copies, MMAs, commits, arrives) are
// predicated INSIDE the asm block on `issuer` (non-zero in the issuing lane) rather than wrapped
// in a C++ `if`: the warp then never diverges around them, and the operands -- the same in every
// lane -- can be computed on the uniform datapath instead of being moved there per instruction.
WB_DEV void mbar_arrive_expect_tx_if(uint32_t issuer, uint32_t bar, uint32_t tx) {
  asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%1], %2;\n\t}" ::"r"(issuer),
               "r"(bar), "r"(tx)
               : "memory");
}
WB_DEV void mbar_arrive_if(uint32_t issuer, uint32_t bar) {
  asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t@e mbarrier.arrive.shared::cta.b64 _, [%1];\n\t}" ::"r"(issuer), "r"(bar) : "memory");
}
// The same arrival ordering nothing: for the accumulator's release.  What the MMA issuer must not overtake is this warp's
// tcgen05.ld of the accumulator, which tcgen05.wait::ld and the tcgen05 fences either side of the barrier order; a releasing
// arrival would also wait for the warp's global stores of the tile (measured: 2 000-3 500 cycles with a tile's stores in flight).
WB_DEV void mbar_arrive_cluster_relaxed_if(uint32_t issuer, uint32_t bar) {
  asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t@e mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%1];\n\t}" ::"r"(issuer),
               "r"(bar)
               : "memory");
}
WB_DEV void mbar_arrive_cluster_if(uint32_t issuer, uint32_t bar) {
  asm volatile("{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t@e mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%1];\n\t}" ::"r"(issuer),
               "r"(bar)
               : "memory");
}
template <int CG>
WB_DEV void tma_load_2d_if(uint32_t issuer, uint32_t dst, const void* map, int x, int y, uint32_t bar) {
  if constexpr (CG == 2) {
    asm volatile(
        "{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%1], [%2, {%3, %4}], [%5];\n\t}" ::"r"(issuer),
        "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%1], [%2, {%3, %4}], [%5];\n\t}" ::"r"(issuer),
        "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}
// store (add == 0) or reducing store (add != 0) of one staged box, then close the bulk group
// `policy`: an L2 cache policy (l2_policy_*): C is written once and not read again by this
// kernel, so its lines are the first the L2 should give up.
WB_DEV void tma_store_commit_if(uint32_t issuer, uint32_t add, const void* map, int x, int y, uint32_t src, uint64_t policy) {
  asm volatile(
      "{\n\t.reg .pred e, s, r;\n\t"
      "setp.ne.u32 e, %0, 0;\n\t"
      "setp.eq.and.u32 s, %1, 0, e;\n\t"
      "setp.ne.and.u32 r, %1, 0, e;\n\t"
      "@s cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%2, {%3, %4}], [%5], %6;\n\t"
      "@r cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group.L2::cache_hint [%2, {%3, %4}], [%5], %6;\n\t"
      "@e cp.async.bulk.commit_group;\n\t}" ::"r"(issuer),
      "r"(add), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src), "l"(policy)
      : "memory");
}
// the same store without closing the bulk group (further stores of the same box follow, then one commit)
WB_DEV void tma_store_if(uint32_t issuer, const void* map, int x, int y, uint32_t src, uint64_t policy) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "setp.ne.u32 e, %0, 0;\n\t"
      "@e cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%1, {%2, %3}], [%4], %5;\n\t}" ::"r"(issuer),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src), "l"(policy)
      : "memory");
}
WB_DEV uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
WB_DEV uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
WB_DEV uint64_t l2_policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
template <int CG>
WB_DEV void umma_f16_if(uint32_t issuer, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (CG == 2) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t"
        "setp.ne.b32 p, %5, 0;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, p;\n\t}" ::"r"(issuer),
        "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t"
        "setp.ne.b32 p, %5, 0;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, p;\n\t}" ::"r"(issuer),
        "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
template <int CG>
WB_DEV void umma_commit_if(uint32_t issuer, uint32_t bar, uint16_t mask) {
  if constexpr (CG == 2) {
    asm volatile(
        "{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%1], %2;\n\t}" ::"r"(issuer),
        "r"(bar), "h"(mask)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred e;\n\tsetp.ne.u32 e, %0, 0;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t}" ::"r"(issuer),
        "r"(bar)
        : "memory");
  }
}

// ---------------------------------------------------------------- k loops, written out
// The two loops a tile's time is spent in -- the producer's and the MMA issuer's -- each as ONE
// asm block: barrier wait, issue, release and ring bookkeeping are ~30 instructions per k-step
// with nothing the compiler adds in between.  That matters because one tcgen05.mma takes
// 65-90 cycles to issue and the tensor pipe queues little: any cycles spent between two stages'
// MMAs are cycles the tensor cores idle.  (The reference's hand-scheduled loops are 45 and 22
// SASS instructions; docs/warpc.md:274-275.)
//
// Every lane of the warp runs the loop; `issuer` is non-zero in the lane whose instructions
// take effect.  A wait that does not complete within `limit` polls ends the loop with status 1
// and the state (stage, phase, k-steps left, ...) as of that k-step, so the caller can run its
// bounded, timed wait and re-enter: the asm itself never spins without limit.  The polls are
// test_wait (they return at once) rather than try_wait: a try_wait that finds the phase open
// suspends the thread, and the wake-up after the arrival costs several hundred cycles -- more
// than a ring of four to eight stages can hide.

// No tcgen05.fence sits between the wait and the MMAs: operand tiles arrive through the async
// proxy and the mbarrier's completion orders them for the MMAs that read them; the tcgen05
// fences are for hand-offs of tensor memory between threads (once per tile, around the
// accumulator barriers), and one inside this loop would drain the tensor pipe at every k-step.
// MMA issuer: for each of `kleft` k-steps wait full[stage], issue REPS x 4 MMAs (A operand =
// the stage's B^T tile, low descriptor word ma_lo0 + stage * step16, atoms atom16 apart; B operand
// = its A tile, mb_lo0 + ...; +2 per 16 K-elements; atom r accumulates at column d + r * span),
// commit to empty[stage].  `accumulate` is 0 until the tile's first MMA has been issued.
#define WB_KL_MMA(G, D, A, B, PRED)                                   \
  "mov.b64 da, {" A ", %16};\n\tmov.b64 db, {" B ", %16};\n\t"        \
  "@e tcgen05.mma.cta_group::" G ".kind::f16 [" D "], da, db, %17, " PRED ";\n\t"
#define WB_KL_MMA_J(G, D, A0, J, PRED) \
  "add.u32 ta, " A0 ", " J ";\n\tadd.u32 tb, mb, " J ";\n\t" WB_KL_MMA(G, D, "ta", "tb", PRED)
// Order inside one k-step: the commit that frees the stage BEFORE comes after the first MMA (issued while that MMA
// runs), the ring's bookkeeping for the next stage (in place: index, barrier addresses, descriptor offset, parity) after
// the second, the count and a non-blocking probe of the next stage's barrier (its answer is back before the loop comes
// round) after the third; only the loop's branch sits between the last MMA of one k-step and the first of the next.
// Measured, the placement of the bookkeeping does not matter (nor do twelve more dependent ALU instructions a k-step):
// the pace is the tensor pipe's with operands from shared memory, about 75 ns (135 cycles) an N = 256 MMA in the kernel.
#define WB_KL_HEAD                                                                                   \
  "{\n\t.reg .pred e, ec, p, q, w, pa, pt, c, pr, pv;\n\t"                                           \
  ".reg .b32 n, fb, eb, s16, ta, tb, d1, a1, ma, mb, dbg, pb;\n\t"                                   \
  ".reg .b64 da, db;\n\t.reg .b16 mk;\n\t"                                                           \
  "setp.ne.u32 ec, %5, 0;\n\tand.b32 dbg, %15, 2;\n\tsetp.eq.and.u32 e, dbg, 0, ec;\n\t"             \
  "setp.eq.u32 pt, 0, 0;\n\tsetp.ne.u32 pa, %4, 0;\n\tmov.b16 mk, 3;\n\t"                            \
  "setp.eq.u32 pr, 1, 0;\n\tsetp.eq.u32 pv, 1, 0;\n\tmov.u32 pb, 0;\n\t"                             \
  "mov.u32 %0, 0;\n\t"                                                                               \
  "mad.lo.u32 fb, %1, 8, %7;\n\tmad.lo.u32 eb, %1, 8, %8;\n\tmul.lo.u32 s16, %1, %14;\n\t"           \
  "add.u32 d1, %9, %10;\n"                                                                           \
  "WB_KL_LOOP:\n\t"                                                                                  \
  "@pr bra WB_KL_GO;\n\t"                                                                            \
  "mov.u32 n, 0;\n"                                                                                  \
  "WB_KL_WAIT:\n\t"                                                                                  \
  "mbarrier.test_wait.parity.shared::cta.b64 p, [fb], %2;\n\t"                                       \
  "@p bra WB_KL_GO;\n\t"                                                                             \
  "add.u32 n, n, 1;\n\tsetp.lt.u32 q, n, %18;\n\t@q bra WB_KL_WAIT;\n\t"                             \
  "mov.u32 %0, 1;\n\tbra WB_KL_OUT;\n"                                                               \
  "WB_KL_GO:\n\t"                                                                                    \
  "add.u32 ma, %11, s16;\n\tadd.u32 mb, %13, s16;\n\t"
#define WB_KL_COMMIT2 "@pv tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [pb], mk;\n\t"
#define WB_KL_COMMIT1 "@pv tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [pb];\n\t"
// this stage is handed back by the commit of the NEXT k-step (or the one after the loop); the ring moves on, in place
#define WB_KL_NEXT                                                                                   \
  "mov.u32 pb, eb;\n\tsetp.ne.u32 pv, %5, 0;\n\t"                                                    \
  "add.u32 %1, %1, 1;\n\tadd.u32 fb, fb, 8;\n\tadd.u32 eb, eb, 8;\n\tadd.u32 s16, s16, %14;\n\t"     \
  "setp.eq.u32 w, %1, %6;\n\t"                                                                       \
  "@w mov.u32 %1, 0;\n\t@w mov.u32 fb, %7;\n\t@w mov.u32 eb, %8;\n\t@w mov.u32 s16, 0;\n\t@w xor.b32 %2, %2, 1;\n\t"
// one k-step fewer to go, and a probe of the next stage's full barrier (not past the last k-step)
#define WB_KL_PROBE                                                                                  \
  "sub.u32 %3, %3, 1;\n\tsetp.ne.u32 c, %3, 0;\n\tsetp.eq.u32 pr, 1, 0;\n\t"                         \
  "@c mbarrier.test_wait.parity.shared::cta.b64 pr, [fb], %2;\n\t"
#define WB_KL_TAIL(COMMIT)                                                                           \
  "setp.eq.u32 pa, 0, 0;\n\tmov.u32 %4, 1;\n\t@c bra WB_KL_LOOP;\n"                        \
  "WB_KL_OUT:\n\t"                                                                                   \
  COMMIT                                                                                             \
  "}"
// one k-step's MMAs for one atom (REPS == 1) or two stacked atoms (REPS == 2)
#define WB_KL_STEP1(G, COMMIT)                                                                       \
  WB_KL_MMA(G, "%9", "ma", "mb", "pa") COMMIT WB_KL_MMA_J(G, "%9", "ma", "2", "pt") WB_KL_NEXT      \
  WB_KL_MMA_J(G, "%9", "ma", "4", "pt") WB_KL_PROBE WB_KL_MMA_J(G, "%9", "ma", "6", "pt")
#define WB_KL_STEP2(G, COMMIT)                                                                       \
  WB_KL_MMA(G, "%9", "ma", "mb", "pa") COMMIT WB_KL_MMA_J(G, "%9", "ma", "2", "pt") WB_KL_NEXT      \
  WB_KL_MMA_J(G, "%9", "ma", "4", "pt") WB_KL_PROBE WB_KL_MMA_J(G, "%9", "ma", "6", "pt")           \
  "add.u32 a1, ma, %12;\n\t"                                                                         \
  WB_KL_MMA(G, "d1", "a1", "mb", "pa") WB_KL_MMA_J(G, "d1", "a1", "2", "pt")                        \
  WB_KL_MMA_J(G, "d1", "a1", "4", "pt") WB_KL_MMA_J(G, "d1", "a1", "6", "pt")
#define WB_KL_ARGS                                                                                          \
  : "=r"(status), "+r"(stage), "+r"(phase), "+r"(kleft), "+r"(accumulate)                                   \
  : "r"(issuer), "r"(depth), "r"(full0), "r"(empty0), "r"(d), "r"(span), "r"(ma_lo0), "r"(atom16), "r"(mb_lo0), \
    "r"(step16), "r"(debug), "r"(hi), "r"(idesc), "r"(limit)                                                \
  : "memory"

template <int CG, int REPS>
WB_DEV uint32_t mma_k_loop(uint32_t issuer, uint32_t& kleft, uint32_t depth, uint32_t& stage, uint32_t& phase, uint32_t& accumulate,
                           uint32_t full0, uint32_t empty0, uint32_t d, uint32_t span, uint32_t ma_lo0, uint32_t atom16, uint32_t mb_lo0,
                           uint32_t step16, uint32_t hi, uint32_t idesc, uint32_t limit, uint32_t debug = 0) {
  uint32_t status;
  if constexpr (CG == 2 && REPS == 1) asm volatile(WB_KL_HEAD WB_KL_STEP1("2", WB_KL_COMMIT2) WB_KL_TAIL(WB_KL_COMMIT2) WB_KL_ARGS);
  if constexpr (CG == 2 && REPS == 2) asm volatile(WB_KL_HEAD WB_KL_STEP2("2", WB_KL_COMMIT2) WB_KL_TAIL(WB_KL_COMMIT2) WB_KL_ARGS);
  if constexpr (CG == 1 && REPS == 1) asm volatile(WB_KL_HEAD WB_KL_STEP1("1", WB_KL_COMMIT1) WB_KL_TAIL(WB_KL_COMMIT1) WB_KL_ARGS);
  if constexpr (CG == 1 && REPS == 2) asm volatile(WB_KL_HEAD WB_KL_STEP2("1", WB_KL_COMMIT1) WB_KL_TAIL(WB_KL_COMMIT1) WB_KL_ARGS);
  return status;
}

// Producer: for each of `kleft` k-steps wait empty[stage], (pair leader) state the pair's bytes
// on its own full[stage], then load the A half-tile and the B^T tile of k column x into the
// stage's slot, both completing on full_remote0 + 8*stage (the pair leader's barrier).
template <int CG>
WB_DEV uint32_t load_k_loop(uint32_t issuer, uint32_t& kleft, uint32_t depth, uint32_t& stage, uint32_t& phase, int& x, uint32_t empty0,
                            uint32_t full0, uint32_t full_remote0, uint32_t is_leader, uint32_t tx, uint32_t ring, uint32_t stage_bytes,
                            uint32_t a_bytes, const void* map_a, int a_row, const void* map_b, int col, uint32_t limit, uint32_t debug, uint64_t policy) {
  uint32_t status;
#define WB_LD_BODY(CGQ)                                                                                          \
  "{\n\t.reg .pred e, ei, pl, pn, p, q, w, c;\n\t.reg .b32 n, eb, fl, fr, sa, sb, par, dbg;\n\t"                 \
  "setp.ne.u32 ei, %5, 0;\n\tand.b32 dbg, %19, 1;\n\tsetp.eq.and.u32 e, dbg, 0, ei;\n\t"                          \
  "setp.ne.and.u32 pl, %10, 0, e;\n\tsetp.ne.and.u32 pn, %10, 0, ei;\n\tsetp.ne.and.u32 pn, dbg, 0, pn;\n\tmov.u32 %0, 0;\n\t" \
  "mad.lo.u32 eb, %1, 8, %7;\n\tmad.lo.u32 fl, %1, 8, %8;\n\tmad.lo.u32 fr, %1, 8, %9;\n\tmad.lo.u32 sa, %1, %13, %12;\n" \
  "WB_LD_LOOP:\n\tmov.u32 n, 0;\n\txor.b32 par, %2, 1;\n"                                                        \
  "WB_LD_WAIT:\n\t"                                                                                              \
  "mbarrier.test_wait.parity.shared::cta.b64 p, [eb], par;\n\t"                                                  \
  "@p bra WB_LD_GO;\n\t"                                                                                         \
  "add.u32 n, n, 1;\n\tsetp.lt.u32 q, n, %20;\n\t@q bra WB_LD_WAIT;\n\t"                                         \
  "mov.u32 %0, 1;\n\tbra WB_LD_OUT;\n"                                                                           \
  "WB_LD_GO:\n\t"                                                                                                \
  "@pl mbarrier.arrive.expect_tx.shared::cta.b64 _, [fl], %11;\n\t"                                              \
  "@pn mbarrier.arrive.shared::cta.b64 _, [fl];\n\t"                                                             \
  "add.u32 sb, sa, %14;\n\t"                                                                                     \
  "@e cp.async.bulk.tensor.2d" CGQ ".shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [sa], [%15, {%4, %16}], [fr], %21;\n\t" \
  "@e cp.async.bulk.tensor.2d" CGQ ".shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [sb], [%17, {%4, %18}], [fr], %21;\n\t" \
  "add.s32 %4, %4, 64;\n\tadd.u32 %1, %1, 1;\n\tadd.u32 eb, eb, 8;\n\tadd.u32 fl, fl, 8;\n\tadd.u32 fr, fr, 8;\n\tadd.u32 sa, sa, %13;\n\t" \
  "setp.eq.u32 w, %1, %6;\n\t"                                                                                   \
  "@w mov.u32 %1, 0;\n\t@w mov.u32 eb, %7;\n\t@w mov.u32 fl, %8;\n\t@w mov.u32 fr, %9;\n\t@w mov.u32 sa, %12;\n\t@w xor.b32 %2, %2, 1;\n\t" \
  "sub.u32 %3, %3, 1;\n\tsetp.ne.u32 c, %3, 0;\n\t@c bra WB_LD_LOOP;\n"                                          \
  "WB_LD_OUT:\n\t}"
#define WB_LD_ARGS                                                                                               \
  : "=r"(status), "+r"(stage), "+r"(phase), "+r"(kleft), "+r"(x)                                                 \
  : "r"(issuer), "r"(depth), "r"(empty0), "r"(full0), "r"(full_remote0), "r"(is_leader), "r"(tx), "r"(ring), "r"(stage_bytes), \
    "r"(a_bytes), "l"(reinterpret_cast<uint64_t>(map_a)), "r"(a_row), "l"(reinterpret_cast<uint64_t>(map_b)), "r"(col), "r"(debug), "r"(limit), \
    "l"(policy)                                                                                                  \
  : "memory"
  if constexpr (CG == 2) asm volatile(WB_LD_BODY(".cta_group::2") WB_LD_ARGS);
  else asm volatile(WB_LD_BODY("") WB_LD_ARGS);
#undef WB_LD_BODY
#undef WB_LD_ARGS
  return status;
}

// ---------------------------------------------------------------- k loops in rounds
// The same two loops with the ring handed over KSUB k-steps at a time: a ROUND is KSUB
// consecutive slots behind one full and one empty barrier.  One k-step of four MMAs costs its
// issuing thread about 4 x 64 cycles for the MMAs plus about 360 for the commit, the probe and
// the ring bookkeeping -- more than the 512 cycles the tensor pipe needs for four N = 256 MMAs
// (and far more than the 256 of N = 128), so with a barrier round per k-step the issuing thread,
// not the tensor pipe, sets the pace.  A round of KSUB k-steps pays that overhead once.  A tile
// (or split-K run) whose k-steps are not a multiple of KSUB ends on a partly used round: the
// producer states and loads, and the issuer multiplies, only the k-steps that exist.
// Operands as in mma_k_loop / load_k_loop, with `stage` the round index, `depth` the number of
// rounds, step16 / stage_bytes the size of a ROUND and slot16 / slot_bytes that of one slot.
#define WB_KR_MMA(G, D, A, B, PRED, GUARD)                            \
  "mov.b64 da, {" A ", %16};\n\tmov.b64 db, {" B ", %16};\n\t"        \
  "@" GUARD " tcgen05.mma.cta_group::" G ".kind::f16 [" D "], da, db, %17, " PRED ";\n\t"
#define WB_KR_MMA_J(G, A0, B0, J, GUARD) \
  "add.u32 ta, " A0 ", " J ";\n\tadd.u32 tb, " B0 ", " J ";\n\t" WB_KR_MMA(G, "%9", "ta", "tb", "pt", GUARD)
// k-step g (>= 1) of the round: its slot's descriptors, four MMAs under the guard for "it exists"
#define WB_KR_GROUP(G, GUARD)                                                                        \
  "add.u32 ga, ga, %12;\n\tadd.u32 gb, gb, %12;\n\t"                                                 \
  WB_KR_MMA(G, "%9", "ga", "gb", "pt", GUARD) WB_KR_MMA_J(G, "ga", "gb", "2", GUARD)                \
  WB_KR_MMA_J(G, "ga", "gb", "4", GUARD) WB_KR_MMA_J(G, "ga", "gb", "6", GUARD)
// Whole rounds run in a loop of their own with no guards; a tile's last, partly used round (and a tile shorter than a
// round) runs once after it, every k-step past the first under the guard for "it exists".
#define WB_KR_HEAD(KSUB)                                                                             \
  "{\n\t.reg .pred e, e1, e2, e3, ec, p, q, w, pa, pt, c, pr, pv, pm, pf;\n\t"                       \
  ".reg .b32 n, fb, eb, s16, ta, tb, ga, gb, ma, mb, dbg, pb;\n\t"                                   \
  ".reg .b64 da, db;\n\t.reg .b16 mk;\n\t"                                                           \
  "setp.ne.u32 ec, %5, 0;\n\tand.b32 dbg, %15, 2;\n\tsetp.eq.and.u32 e, dbg, 0, ec;\n\t"             \
  "setp.eq.u32 pt, 0, 0;\n\tsetp.ne.u32 pa, %4, 0;\n\tmov.b16 mk, 3;\n\t"                            \
  "setp.eq.u32 pr, 1, 0;\n\tsetp.eq.u32 pv, 1, 0;\n\tmov.u32 pb, 0;\n\t"                             \
  "mov.u32 %0, 0;\n\t"                                                                               \
  "mad.lo.u32 fb, %1, 8, %7;\n\tmad.lo.u32 eb, %1, 8, %8;\n\tmul.lo.u32 s16, %1, %14;\n\t"           \
  "add.u32 ma, %11, s16;\n\tadd.u32 mb, %13, s16;\n\t"                                                \
  "setp.lt.u32 pf, %3, " KSUB ";\n\t@pf bra WB_KR_LAST;\n"                                           \
  "WB_KR_LOOP:\n\t"                                                                                  \
  "@pr bra WB_KR_GO;\n\t"                                                                            \
  "mov.u32 n, 0;\n"                                                                                  \
  "WB_KR_WAIT:\n\t"                                                                                  \
  "mbarrier.test_wait.parity.shared::cta.b64 p, [fb], %2;\n\t"                                       \
  "@p bra WB_KR_GO;\n\t"                                                                             \
  "add.u32 n, n, 1;\n\tsetp.lt.u32 q, n, %18;\n\t@q bra WB_KR_WAIT;\n\t"                             \
  "mov.u32 %0, 1;\n\tbra WB_KR_OUT;\n"                                                               \
  "WB_KR_GO:\n\t"
// the last round: entered with fewer than KSUB k-steps left (none: nothing to do)
#define WB_KR_LAST_HEAD                                                                              \
  "WB_KR_LAST:\n\t"                                                                                  \
  "setp.eq.u32 pf, %3, 0;\n\t@pf bra WB_KR_OUT;\n\t"                                                 \
  "@pr bra WB_KR_GO2;\n\t"                                                                           \
  "mov.u32 n, 0;\n"                                                                                  \
  "WB_KR_WAIT2:\n\t"                                                                                 \
  "mbarrier.test_wait.parity.shared::cta.b64 p, [fb], %2;\n\t"                                       \
  "@p bra WB_KR_GO2;\n\t"                                                                            \
  "add.u32 n, n, 1;\n\tsetp.lt.u32 q, n, %18;\n\t@q bra WB_KR_WAIT2;\n\t"                            \
  "mov.u32 %0, 1;\n\tbra WB_KR_OUT;\n"                                                               \
  "WB_KR_GO2:\n\t"                                                                                   \
  "add.u32 ma, %11, s16;\n\tadd.u32 mb, %13, s16;\n\tmov.u32 ga, ma;\n\tmov.u32 gb, mb;\n\t"         \
  "setp.gt.u32 e1, %3, 1;\n\tand.pred e1, e1, e;\n\t"                                                \
  "setp.gt.u32 e2, %3, 2;\n\tand.pred e2, e2, e;\n\t"                                                \
  "setp.gt.u32 e3, %3, 3;\n\tand.pred e3, e3, e;\n\t"
#define WB_KR_END(COMMIT)                                                                            \
  "mov.u32 %3, 0;\n\tsetp.eq.u32 pa, 0, 0;\n\tmov.u32 %4, 1;\n"                                      \
  "WB_KR_OUT:\n\t"                                                                                   \
  COMMIT                                                                                             \
  "}"
// A whole round.  An M = 256 pair MMA narrower than N = 256 takes the tensor pipe about 76 cycles whatever its N
// (stand-alone loop; 79-97 in the kernel).  The round's bookkeeping is dealt out over the gaps between its MMAs: the
// lagged commit of the round before after the first MMA; then, a few instructions a gap, the ring moved on (index,
// parity, the round's own empty barrier kept for the next commit, the next round's barriers and descriptor offset), the
// count, the probe of the next round's full barrier, and the next round's descriptors; nothing but the branch after the
// last MMA.  (Measured against the same bookkeeping in one piece after the round's last MMA: the same pace, 216 ns a
// k-step at 1536^3 either way.  Kept for the loop without guards it came with.)
#define WB_KR_G_A "mov.u32 pb, eb;\n\tadd.u32 %1, %1, 1;\n\tsetp.eq.u32 w, %1, %6;\n\t"
#define WB_KR_G_B "@w mov.u32 %1, 0;\n\t@w xor.b32 %2, %2, 1;\n\tsetp.ne.u32 pv, %5, 0;\n\t"
#define WB_KR_G_C "mad.lo.u32 fb, %1, 8, %7;\n\tmad.lo.u32 eb, %1, 8, %8;\n\tmul.lo.u32 s16, %1, %14;\n\t"
#define WB_KR_G_D(KSUB) "sub.u32 %3, %3, " KSUB ";\n\tsetp.ge.u32 c, %3, " KSUB ";\n\tsetp.ne.u32 pm, %3, 0;\n\t"
#define WB_KR_G_E "setp.eq.u32 pr, 1, 0;\n\t@pm mbarrier.test_wait.parity.shared::cta.b64 pr, [fb], %2;\n\t"
#define WB_KR_G_F "add.u32 ma, %11, s16;\n\tadd.u32 mb, %13, s16;\n\tsetp.eq.u32 pa, 0, 0;\n\tmov.u32 %4, 1;\n\t"
#define WB_KR_G_NEXTSLOT "add.u32 ga, ga, %12;\n\tadd.u32 gb, gb, %12;\n\t"
#define WB_KR_G_FIRSTSLOT "add.u32 ga, ma, %12;\n\tadd.u32 gb, mb, %12;\n\t"
// rounds of two: eight MMAs, seven gaps
#define WB_KR_ROUND2(G, COMMIT)                                                                      \
  WB_KR_MMA(G, "%9", "ma", "mb", "pa", "e") COMMIT                                                   \
  WB_KR_MMA_J(G, "ma", "mb", "2", "e") WB_KR_G_A                                                     \
  WB_KR_MMA_J(G, "ma", "mb", "4", "e") WB_KR_G_B                                                     \
  WB_KR_MMA_J(G, "ma", "mb", "6", "e") WB_KR_G_FIRSTSLOT                                             \
  WB_KR_MMA(G, "%9", "ga", "gb", "pt", "e") WB_KR_G_C                                                \
  WB_KR_MMA_J(G, "ga", "gb", "2", "e") WB_KR_G_D("2")                                                \
  WB_KR_MMA_J(G, "ga", "gb", "4", "e") WB_KR_G_E                                                     \
  WB_KR_G_F WB_KR_MMA_J(G, "ga", "gb", "6", "e")                                                     \
  "@c bra WB_KR_LOOP;\n"
// rounds of four: sixteen MMAs
#define WB_KR_ROUND4(G, COMMIT)                                                                      \
  WB_KR_MMA(G, "%9", "ma", "mb", "pa", "e") COMMIT                                                   \
  WB_KR_MMA_J(G, "ma", "mb", "2", "e") WB_KR_G_A                                                     \
  WB_KR_MMA_J(G, "ma", "mb", "4", "e") WB_KR_G_B                                                     \
  WB_KR_MMA_J(G, "ma", "mb", "6", "e") WB_KR_G_FIRSTSLOT                                             \
  WB_KR_MMA(G, "%9", "ga", "gb", "pt", "e") WB_KR_G_C                                                \
  WB_KR_MMA_J(G, "ga", "gb", "2", "e") WB_KR_MMA_J(G, "ga", "gb", "4", "e")                         \
  WB_KR_MMA_J(G, "ga", "gb", "6", "e") WB_KR_G_NEXTSLOT                                              \
  WB_KR_MMA(G, "%9", "ga", "gb", "pt", "e") WB_KR_G_D("4")                                           \
  WB_KR_MMA_J(G, "ga", "gb", "2", "e") WB_KR_MMA_J(G, "ga", "gb", "4", "e")                         \
  WB_KR_MMA_J(G, "ga", "gb", "6", "e") WB_KR_G_NEXTSLOT                                              \
  WB_KR_MMA(G, "%9", "ga", "gb", "pt", "e") WB_KR_G_E                                                \
  WB_KR_MMA_J(G, "ga", "gb", "2", "e") WB_KR_MMA_J(G, "ga", "gb", "4", "e")                         \
  WB_KR_G_F WB_KR_MMA_J(G, "ga", "gb", "6", "e")                                                     \
  "@c bra WB_KR_LOOP;\n"
// the same first k-step in the last round (the ring moves on after it, nothing is probed)
#define WB_KR_STEP0_LAST(G, COMMIT)                                                                  \
  WB_KR_MMA(G, "%9", "ma", "mb", "pa", "e") COMMIT WB_KR_MMA_J(G, "ma", "mb", "2", "e")             \
  WB_KL_NEXT WB_KR_MMA_J(G, "ma", "mb", "4", "e") WB_KR_MMA_J(G, "ma", "mb", "6", "e")
#define WB_KR_BODY2(G, COMMIT)                                                                       \
  WB_KR_ROUND2(G, COMMIT) WB_KR_LAST_HEAD WB_KR_STEP0_LAST(G, COMMIT) WB_KR_GROUP(G, "e1")
#define WB_KR_BODY4(G, COMMIT)                                                                       \
  WB_KR_ROUND4(G, COMMIT) WB_KR_LAST_HEAD WB_KR_STEP0_LAST(G, COMMIT) WB_KR_GROUP(G, "e1") WB_KR_GROUP(G, "e2") WB_KR_GROUP(G, "e3")

template <int CG, int KSUB>
WB_DEV uint32_t mma_rounds(uint32_t issuer, uint32_t& kleft, uint32_t depth, uint32_t& stage, uint32_t& phase, uint32_t& accumulate,
                           uint32_t full0, uint32_t empty0, uint32_t d, uint32_t span, uint32_t ma_lo0, uint32_t atom16, uint32_t mb_lo0,
                           uint32_t step16, uint32_t hi, uint32_t idesc, uint32_t limit, uint32_t debug = 0) {
  static_assert(KSUB == 2 || KSUB == 4, "rounds of two or four k-steps");
  uint32_t status;
  if constexpr (CG == 2 && KSUB == 2) asm volatile(WB_KR_HEAD("2") WB_KR_BODY2("2", WB_KL_COMMIT2) WB_KR_END(WB_KL_COMMIT2) WB_KL_ARGS);
  if constexpr (CG == 2 && KSUB == 4) asm volatile(WB_KR_HEAD("4") WB_KR_BODY4("2", WB_KL_COMMIT2) WB_KR_END(WB_KL_COMMIT2) WB_KL_ARGS);
  if constexpr (CG == 1 && KSUB == 2) asm volatile(WB_KR_HEAD("2") WB_KR_BODY2("1", WB_KL_COMMIT1) WB_KR_END(WB_KL_COMMIT1) WB_KL_ARGS);
  if constexpr (CG == 1 && KSUB == 4) asm volatile(WB_KR_HEAD("4") WB_KR_BODY4("1", WB_KL_COMMIT1) WB_KR_END(WB_KL_COMMIT1) WB_KL_ARGS);
  return status;
}

// Producer, a round at a time: wait empty[round], (pair leader) state the bytes of the round's
// k-steps that exist, load each of them into its slot.
template <int CG, int KSUB>
WB_DEV uint32_t load_rounds(uint32_t issuer, uint32_t& kleft, uint32_t depth, uint32_t& stage, uint32_t& phase, int& x, uint32_t empty0,
                            uint32_t full0, uint32_t full_remote0, uint32_t is_leader, uint32_t tx, uint32_t ring, uint32_t stage_bytes,
                            uint32_t a_bytes, const void* map_a, int a_row, const void* map_b, int col, uint32_t limit, uint32_t debug,
                            uint32_t slot_bytes, uint64_t policy) {
  static_assert(KSUB == 2 || KSUB == 4, "rounds of two or four k-steps");
  uint32_t status;
#define WB_LR_LOADS(CGQ, GUARD)                                                                                  \
  "add.u32 sb, sg, %14;\n\t"                                                                                     \
  "@" GUARD " cp.async.bulk.tensor.2d" CGQ ".shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [sg], [%15, {xg, %16}], [fr], %22;\n\t" \
  "@" GUARD " cp.async.bulk.tensor.2d" CGQ ".shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [sb], [%17, {xg, %18}], [fr], %22;\n\t" \
  "add.u32 sg, sg, %21;\n\tadd.s32 xg, xg, 64;\n\t"
#define WB_LR_BODY(CGQ, KSUB_S, MORE)                                                                            \
  "{\n\t.reg .pred e, e1, e2, e3, ei, pl, pn, p, q, w, c;\n\t.reg .b32 n, eb, fl, fr, sa, sb, sg, xg, par, dbg, use, txr;\n\t" \
  "setp.ne.u32 ei, %5, 0;\n\tand.b32 dbg, %19, 1;\n\tsetp.eq.and.u32 e, dbg, 0, ei;\n\t"                          \
  "setp.ne.and.u32 pl, %10, 0, e;\n\tsetp.ne.and.u32 pn, %10, 0, ei;\n\tsetp.ne.and.u32 pn, dbg, 0, pn;\n\tmov.u32 %0, 0;\n\t" \
  "mad.lo.u32 eb, %1, 8, %7;\n\tmad.lo.u32 fl, %1, 8, %8;\n\tmad.lo.u32 fr, %1, 8, %9;\n\tmad.lo.u32 sa, %1, %13, %12;\n" \
  "WB_LR_LOOP:\n\tmov.u32 n, 0;\n\txor.b32 par, %2, 1;\n"                                                        \
  "WB_LR_WAIT:\n\t"                                                                                              \
  "mbarrier.test_wait.parity.shared::cta.b64 p, [eb], par;\n\t"                                                  \
  "@p bra WB_LR_GO;\n\t"                                                                                         \
  "add.u32 n, n, 1;\n\tsetp.lt.u32 q, n, %20;\n\t@q bra WB_LR_WAIT;\n\t"                                         \
  "mov.u32 %0, 1;\n\tbra WB_LR_OUT;\n"                                                                           \
  "WB_LR_GO:\n\t"                                                                                                \
  "min.u32 use, %3, " KSUB_S ";\n\tmul.lo.u32 txr, %11, use;\n\t"                                                \
  "setp.gt.u32 e1, %3, 1;\n\tand.pred e1, e1, e;\n\tsetp.gt.u32 e2, %3, 2;\n\tand.pred e2, e2, e;\n\tsetp.gt.u32 e3, %3, 3;\n\tand.pred e3, e3, e;\n\t" \
  "@pl mbarrier.arrive.expect_tx.shared::cta.b64 _, [fl], txr;\n\t"                                              \
  "@pn mbarrier.arrive.shared::cta.b64 _, [fl];\n\t"                                                             \
  "mov.u32 sg, sa;\n\tmov.u32 xg, %4;\n\t"                                                                       \
  WB_LR_LOADS(CGQ, "e") WB_LR_LOADS(CGQ, "e1") MORE                                                              \
  "mad.lo.s32 %4, use, 64, %4;\n\tadd.u32 %1, %1, 1;\n\tadd.u32 eb, eb, 8;\n\tadd.u32 fl, fl, 8;\n\tadd.u32 fr, fr, 8;\n\tadd.u32 sa, sa, %13;\n\t" \
  "setp.eq.u32 w, %1, %6;\n\t"                                                                                   \
  "@w mov.u32 %1, 0;\n\t@w mov.u32 eb, %7;\n\t@w mov.u32 fl, %8;\n\t@w mov.u32 fr, %9;\n\t@w mov.u32 sa, %12;\n\t@w xor.b32 %2, %2, 1;\n\t" \
  "sub.u32 %3, %3, use;\n\tsetp.ne.u32 c, %3, 0;\n\t@c bra WB_LR_LOOP;\n"                                        \
  "WB_LR_OUT:\n\t}"
#define WB_LR_ARGS                                                                                               \
  : "=r"(status), "+r"(stage), "+r"(phase), "+r"(kleft), "+r"(x)                                                 \
  : "r"(issuer), "r"(depth), "r"(empty0), "r"(full0), "r"(full_remote0), "r"(is_leader), "r"(tx), "r"(ring), "r"(stage_bytes), \
    "r"(a_bytes), "l"(reinterpret_cast<uint64_t>(map_a)), "r"(a_row), "l"(reinterpret_cast<uint64_t>(map_b)), "r"(col), "r"(debug), "r"(limit), \
    "r"(slot_bytes), "l"(policy)                                                                                 \
  : "memory"
  if constexpr (CG == 2 && KSUB == 2) asm volatile(WB_LR_BODY(".cta_group::2", "2", "") WB_LR_ARGS);
  if constexpr (CG == 2 && KSUB == 4) asm volatile(WB_LR_BODY(".cta_group::2", "4", WB_LR_LOADS(".cta_group::2", "e2") WB_LR_LOADS(".cta_group::2", "e3")) WB_LR_ARGS);
  if constexpr (CG == 1 && KSUB == 2) asm volatile(WB_LR_BODY("", "2", "") WB_LR_ARGS);
  if constexpr (CG == 1 && KSUB == 4) asm volatile(WB_LR_BODY("", "4", WB_LR_LOADS("", "e2") WB_LR_LOADS("", "e3")) WB_LR_ARGS);
#undef WB_LR_BODY
#undef WB_LR_LOADS
#undef WB_LR_ARGS
  return status;
}

// ---------------------------------------------------------------- cluster launch control
// Ask the hardware to cancel a not-yet-launched cluster of this grid; the 16-byte
// answer lands in this CTA's shared memory and completes 16 bytes on `bar`.
WB_DEV void clc_try_cancel(uint32_t answer, uint32_t bar) {
  asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];" ::"r"(
                   answer),
               "r"(bar)
               : "memory");
}
// Decode: returns 1 and the cancelled cluster's first CTA x-index, or 0 when nothing was left.
WB_DEV uint32_t clc_decode(uint32_t answer, uint32_t* first_cta) {
  uint32_t valid, x;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b128 r;\n\t.reg .b32 y, z;\n\t"
      "ld.shared.b128 r, [%2];\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "mov.u32 %1, 0;\n\t"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid.v4.b32.b128 {%1, y, z, _}, r;\n\t}"
      : "=r"(valid), "=r"(x)
      : "r"(answer)
      : "memory");
  *first_cta = x;
  return valid;
}

// stores into another CTA's shared memory (address from mapa)
WB_DEV void st_cluster_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

}  // namespace wb
