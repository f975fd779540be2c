// Inline-PTX building blocks for sm_100a: mbarrier, TMA bulk-tensor loads,
// tcgen05 (tensor memory allocation, MMA issue, commit, TMEM loads) and the
// shared-memory / instruction descriptors tcgen05.mma consumes.
//
// Every wait here is bounded: a spin gives up after WaitCtx::limit_ns (2 s unless the
// "wait_limit_us" tuning knob says otherwise), records a code in the per-device status word
// and tells the rest of the CTA to leave.
#pragma once

#include "common.cuh"

#ifdef __CUDACC_RTC__
// cuda.h needs host headers; all device code needs of it is the size and alignment of a tensor map
struct alignas(64) CUtensorMap_st {
  unsigned long long opaque[16];
};
typedef CUtensorMap_st CUtensorMap;
#else
#include <cuda.h>
#endif

namespace nb200 {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ----------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking: has the phase with this parity completed?  Issued early, its latency hides
// behind other work; a false answer only means "ask again with mbar_wait".
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// What a role needs to give up cleanly: the CTA-wide abort flag, the device status word and
// how long one wait may last.
struct WaitCtx {
  volatile uint32_t* abort_flag;  // shared memory
  unsigned int* status;           // global, 4 words
  unsigned long long limit_ns;    // per wait
};

// Waits for the phase with the given parity.  Returns false when the CTA is
// aborting or when the wait ran out of time (recorded with `code`).
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          unsigned int code, unsigned int detail) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*ctx.abort_flag) return false;
      if (global_timer_ns() - t0 > ctx.limit_ns) {
        *ctx.abort_flag = 1;
        if (atomicCAS(&ctx.status[0], 0u, code) == 0u) ctx.status[1] = detail;
        __threadfence();
        return false;
      }
    }
  }
  return true;
}
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                                   unsigned int code, unsigned int detail) {
  return mbar_spin(bar, parity, ctx, code, detail);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          unsigned int code, unsigned int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctx, code, detail);
}
// The same with the spin loop in line, for kernels whose warpgroups re-divide the register
// file (setmaxnreg): ptxas cannot allocate registers for a function call made from a region
// whose register count was lowered.
__device__ __forceinline__ bool mbar_wait_nocall(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                                 unsigned int code, unsigned int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_spin(bar, parity, ctx, code, detail);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c,
                                             uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "r"(addr)
               : "memory");
}

// Named barriers 1..15 (0 is __syncthreads): `threads` threads take part, as whole warps;
// `arrive` counts toward the barrier without waiting for it.
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(uint32_t id, uint32_t threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// True in exactly one lane of a converged warp.  Issuing MMAs under this predicate (rather than
// inside a `lane == 0` branch) keeps the warp's control flow uniform, so descriptors and
// addresses stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- TMA ---------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory, completion on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// ---- tcgen05 -----------------------------------------------------------------

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Whole warp.  Writes the TMEM base address of `cols` columns into *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// The same for fp32 operands read as tf32 (8 K-elements per instruction).
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread
// (thread i of the warp gets lane base+i).  Whole warp.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 registers per thread -> 32 lanes x 32 consecutive 32-bit columns.  Whole warp.
// The same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// N consecutive columns (16 or a multiple of 32) of this thread's lane.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(N == 16 || N % 32 == 0, "column count");
  if constexpr (N == 16) {
    tmem_ld_32x32(taddr, r);
  } else {
#pragma unroll
    for (int q = 0; q < N / 32; ++q)
      tmem_ld_32x32(taddr + q * 32, *reinterpret_cast<uint32_t (*)[32]>(&r[q * 32]));
  }
}
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(N == 16 || N % 32 == 0, "column count");
  if constexpr (N == 16) {
    tmem_st_32x32(taddr, r);
  } else {
#pragma unroll
    for (int q = 0; q < N / 32; ++q)
      tmem_st_32x32(taddr + q * 32, *reinterpret_cast<const uint32_t (*)[32]>(&r[q * 32]));
  }
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- CTA pairs (cluster of two CTAs sharing one 256-row MMA) --------------------

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address valid in every CTA of the
// cluster) as seen in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr,
                                                              uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_addr),
               "r"(bytes)
               : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on a barrier
// that may live in the other CTA of the pair.  No multicast: each CTA fetches its own tile.
// A tile of shared memory written out to a tensor by the copy engine (no multicast, this GPU's
// memory): the issuing thread's writes to `src` must be behind a fence.proxy.async; the copy
// belongs to the thread's current bulk group; boxes that reach past the tensor's edges are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the sources of all but the N newest groups of this thread have been read / all of it is done
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x,
                                                 int y, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int x,
                                                 int y, int z, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
// One thread of the leader CTA issues; operands are read from both CTAs' shared memory at
// the same offsets, each CTA accumulates its own 128 rows in its own tensor memory.
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;"
      "\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;"
      "\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives on one barrier (anywhere in the cluster) once the pair's MMAs issued so far retire.
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   cluster_bar)
               : "memory");
}

// ---- descriptors -------------------------------------------------------------

// Shared-memory matrix descriptor, 128-byte swizzle.  Fields (bits):
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4,
//   [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout = 2.
// K-major operand (rows of 64 16-bit elements = 128 B, as TMA writes them with
// SWIZZLE_128B): SBO = 1024 (eight rows), LBO unused.
// MN-major operand (TMA box of 64 MN-elements x K rows): K rows are 128 B
// apart, groups of eight rows SBO = 1024 apart, successive 64-element slabs
// along MN are LBO bytes apart.
__host__ __device__ constexpr uint64_t smem_desc_sw128(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t((lbo_bytes >> 4) & 0x3fff) << 16) | (uint64_t((sbo_bytes >> 4) & 0x3fff) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// The same for an MN-major operand of 32-bit elements (tf32): the 128-byte swizzle works on
// 32-byte atoms there (address bits 5-6 XOR bits 7-8, a pattern of four 128-byte rows: layout
// type 1; TMA writes it with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B), so groups of four K rows
// are SBO = 512 bytes apart.
__host__ __device__ constexpr uint64_t smem_desc_sw128_atom32(uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t((lbo_bytes >> 4) & 0x3fff) << 16) | (uint64_t((sbo_bytes >> 4) & 0x3fff) << 32) |
         (uint64_t(1) << 46) | (uint64_t(1) << 61);
}
__device__ __forceinline__ uint64_t with_address(uint64_t desc, uint32_t smem_addr) {
  return desc | uint64_t((smem_addr >> 4) & 0x3fff);
}

// Instruction descriptor for kind::f16, fp32 accumulate.
//   [4,6) D format (1 = f32), [7,10) A format, [10,13) B format (0 = f16, 1 = bf16),
//   bit 15 A major, bit 16 B major (0 = K, 1 = MN), [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n, bool bf16, bool a_mn_major,
                                                      bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
// The same for kind::tf32 (A and B format 2 = tf32).
__host__ __device__ constexpr uint32_t instr_desc_tf32(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// three-input maximum and packed two-wide fp32 arithmetic (one issue slot for two values)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("sub.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 2^t for two values at once without the special-function unit: t is split into its nearest
// integer (adding 1.5 * 2^23 leaves it in the low mantissa bits, from where it is shifted into
// the exponent field of the result) and a remainder in [-0.5, 0.5], whose power of two is a
// cubic with a largest relative error of 7.5e-5 (minimax fit).  Arguments are clamped at -125;
// meant for t <= ~100.  Costs about eleven issue slots on the FMA and integer pipes, none on
// the unit `ex2.approx` runs on, which is the point: softmax loops are bound by that unit.
__device__ __forceinline__ void exp2_cubic2(unsigned long long t2, float& pa, float& pb) {
  const unsigned long long magic2 = pack2(12582912.0f, 12582912.0f);
  float ta, tb;
  unpack2(t2, ta, tb);
  t2 = pack2(fmaxf(ta, -125.0f), fmaxf(tb, -125.0f));
  const unsigned long long f2 = add2(t2, magic2);
  const unsigned long long r2 = sub2(t2, sub2(f2, magic2));
  unsigned long long q2 = fma2(pack2(0.05517146f, 0.05517146f), r2, pack2(0.24261086f, 0.24261086f));
  q2 = fma2(q2, r2, pack2(0.69326097f, 0.69326097f));
  q2 = fma2(q2, r2, pack2(0.99992812f, 0.99992812f));
  float qa, qb, fa, fb;
  unpack2(q2, qa, qb);
  unpack2(f2, fa, fb);
  pa = __uint_as_float(__float_as_uint(qa) + (__float_as_uint(fa) << 23));
  pb = __uint_as_float(__float_as_uint(qb) + (__float_as_uint(fb) << 23));
}

__device__ __forceinline__ float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

}  // namespace sm100

#ifndef __CUDACC_RTC__
// ---- host: tensor maps ---------------------------------------------------------

// Encodes a tiled tensor map of 16- or 32-bit elements with 128-byte swizzle and zero fill
// (`atom32`: the swizzle's 32-byte-atom form, for MN-major tf32 operands).
// dims/strides are given innermost first; `strides_bytes` has rank-1 entries.
// Returns 0 or an NB200_E_* code (message recorded).
int encode_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      bool atom32 = false);
int encode_tensor_map_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box);
#endif  // !__CUDACC_RTC__

}  // namespace nb200
