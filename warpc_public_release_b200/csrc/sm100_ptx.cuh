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

WB_DEV void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
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
WB_DEV void tma_store_commit_if(uint32_t issuer, uint32_t add, const void* map, int x, int y, uint32_t src) {
  asm volatile(
      "{\n\t.reg .pred e, s, r;\n\t"
      "setp.ne.u32 e, %0, 0;\n\t"
      "setp.eq.and.u32 s, %1, 0, e;\n\t"
      "setp.ne.and.u32 r, %1, 0, e;\n\t"
      "@s cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%2, {%3, %4}], [%5];\n\t"
      "@r cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%2, {%3, %4}], [%5];\n\t"
      "@e cp.async.bulk.commit_group;\n\t}" ::"r"(issuer),
      "r"(add), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src)
      : "memory");
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
