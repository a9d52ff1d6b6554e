// tcgen05 / TMA / mbarrier building blocks shared by the sm_100a tensor-core
// kernels: inline-PTX wrappers, bounded barrier waits, UMMA shared-memory matrix
// descriptors, and the host-side tensor-map encoder (resolved through the runtime,
// so the library does not link against the driver).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace b200 {
namespace {

constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

// --------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr uint32_t kSpinsBeforeClock = 4096;

// Waits for the phase of `parity` to complete. Gives up when the CTA aborted or
// after kWaitBudgetNs; returns false then (and raises the abort with `code`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int code, unsigned long long budget_ns = kWaitBudgetNs) {
  if (mbar_try_wait(bar, parity)) return true;
  // The wall clock (%globaltimer, slow to read) is only consulted once a wait has lasted
  // for kSpinsBeforeClock more tries: ordinary waits, of a microsecond or a few, never pay
  // for a read of it, and the budget starts a little late, which does not matter to a
  // limit of seconds.
  unsigned long long start = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      if (*abort_flag) return false;
      if (spin >= kSpinsBeforeClock) {
        const unsigned long long now = global_ns();
        if (start == 0) start = now;
        if (now - start > budget_ns) {
          *abort_flag = 1;
          if (status) atomicOr(status, code);
          return false;
        }
      }
    }
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y,
                                            int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// 4-D form (an M- or N-contiguous operand seen as 64-column chunks: column in chunk, k row,
// chunk, batch).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c0, int32_t c1,
                                            int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 5-D form (32x32-blocked operands: k, m, k block, m block, batch).
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c0, int32_t c1,
                                            int32_t c2, int32_t c3, int32_t c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// Store of a 2-D box from shared memory (128-byte-swizzled rows) to global memory, tracked
// by the issuing thread's bulk async-group. Parts of the box outside the tensor are dropped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(x),
               "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the committed stores have read their shared-memory source (it may be overwritten).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Until the committed stores have completed.
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// CG is the tcgen05 cta_group: 1 (one CTA per tile) or 2 (a CTA pair on one TPC shares a tile).
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t cols) {
  if (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(cols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(cols)
                 : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if (CG == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  if (CG == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// In the shared::cluster window a CTA's own shared addresses carry its rank in
// bit 24: clearing it names the same offset in the even (leader) CTA of a pair.
constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier of the pair's leader CTA (which may be this CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar & kLeaderMask) : "memory");
}
// TMA load of a CTA pair: the bytes are counted on the leader's barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                                 int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & kLeaderMask), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c0,
                                                 int32_t c1, int32_t c2, int32_t c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & kLeaderMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c0,
                                                 int32_t c1, int32_t c2, int32_t c3, int32_t c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & kLeaderMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
template <int CG>
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (CG == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The four MMAs of a 64-deep K block, preceded by a non-blocking test of another
// barrier whose result is only looked at after the MMAs: the test's latency then
// overlaps the issue of the MMAs instead of sitting between two K blocks (the tensor
// core idles for every cycle the issuing thread spends between blocks). Returns
// whether the tested phase had completed. `first_accumulate`: 0 overwrites the
// accumulator with the first product.
// `a_half` > 0: the descriptor distance from the first to the third K slice of A when the
// stage is not one contiguous run of slices (the second 32-wide K block of a 32x32-blocked
// operand); 0: four slices `a_step` apart. A compile-time choice of the caller: the plain
// form must not pay for the other in the issue loop.
template <int CG, bool A_SPLIT = false>
__device__ __forceinline__ uint32_t umma_bf16_x4_peek(uint32_t d_tmem, uint64_t a0, uint64_t b0, uint64_t a_step,
                                                      uint64_t b_step, uint32_t idesc, uint32_t first_accumulate,
                                                      uint32_t peek_bar, uint32_t peek_parity, uint64_t a_half = 0) {
  uint32_t ready;
  const uint64_t a1 = a0 + a_step, a2 = A_SPLIT ? a0 + a_half : a1 + a_step, a3 = a2 + a_step;
  const uint64_t b1 = b0 + b_step, b2 = b1 + b_step, b3 = b2 + b_step;
  if (CG == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred ready, first, always;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 ready, [%1], %2;\n\t"
        "setp.ne.b32 first, %3, 0;\n\t"
        "setp.eq.b32 always, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%4], %5, %6, %7, first;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%4], %8, %9, %7, always;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%4], %10, %11, %7, always;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%4], %12, %13, %7, always;\n\t"
        "selp.u32 %0, 1, 0, ready;\n\t"
        "}"
        : "=r"(ready)
        : "r"(peek_bar), "r"(peek_parity), "r"(first_accumulate), "r"(d_tmem), "l"(a0), "l"(b0), "r"(idesc), "l"(a1),
          "l"(b1), "l"(a2), "l"(b2), "l"(a3), "l"(b3)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred ready, first, always;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 ready, [%1], %2;\n\t"
        "setp.ne.b32 first, %3, 0;\n\t"
        "setp.eq.b32 always, 0, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%4], %5, %6, %7, first;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%4], %8, %9, %7, always;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%4], %10, %11, %7, always;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%4], %12, %13, %7, always;\n\t"
        "selp.u32 %0, 1, 0, ready;\n\t"
        "}"
        : "=r"(ready)
        : "r"(peek_bar), "r"(peek_parity), "r"(first_accumulate), "r"(d_tmem), "l"(a0), "l"(b0), "r"(idesc), "l"(a1),
          "l"(b1), "l"(a2), "l"(b2), "l"(a3), "l"(b3)
        : "memory");
  return ready;
}

// The same product with the A operand in tensor memory (lane = row, each 32-bit
// column two consecutive K elements; K = 16 per instruction = 8 columns) and B in
// shared memory. cta_group::1 only.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four such MMAs over consecutive K slices (A advancing by 8 tensor-memory columns, B by
// `b_step` descriptor units), with the same carried barrier test as umma_bf16_x4_peek.
__device__ __forceinline__ uint32_t umma_bf16_ts_x4_peek(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, uint64_t b_step,
                                                         uint32_t idesc, uint32_t first_accumulate, uint32_t peek_bar,
                                                         uint32_t peek_parity) {
  uint32_t ready;
  const uint64_t b1 = b0 + b_step, b2 = b1 + b_step, b3 = b2 + b_step;
  asm volatile(
      "{\n\t"
      ".reg .pred ready, first, always;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 ready, [%1], %2;\n\t"
      "setp.ne.b32 first, %3, 0;\n\t"
      "setp.eq.b32 always, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%4], [%5], %9, %8, first;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%4], [%6], %10, %8, always;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%4], [%7], %11, %8, always;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%4], [%13], %12, %8, always;\n\t"
      "selp.u32 %0, 1, 0, ready;\n\t"
      "}"
      : "=r"(ready)
      : "r"(peek_bar), "r"(peek_parity), "r"(first_accumulate), "r"(d_tmem), "r"(a_tmem), "r"(a_tmem + 8),
        "r"(a_tmem + 16), "r"(idesc), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(a_tmem + 24)
      : "memory");
  return ready;
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has
// completed; for a CTA pair, on the barrier at that offset in both CTAs.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if (CG == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  } else {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                     "r"(bar),
                 "h"(both)
                 : "memory");
  }
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16-column forms, for code that is short of registers.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_field, uint32_t hi) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (lbo_field << 16);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// --------------------------------------------------------------------------- host
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      sym = nullptr;
    }
    return reinterpret_cast<EncodeTiled>(sym);
  }();
  return fn;
}

// 3-D map over a row-major [batch][rows][cols] bf16 view with 128-byte swizzle.
bool encode_map(CUtensorMap* map, const void* base, int64_t cols, int64_t rows, int64_t batch, int64_t ld,
                int64_t batch_stride, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(batch_stride) * 2};
  const cuuint32_t box[3] = {box_cols, box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-D map over a row-major [batch][rows][cols] bf16 view whose columns are a multiple of 64,
// seen as [batch][cols / 64][rows][64]: one box is `box_chunks` 64-column chunks of
// `box_rows` rows, each chunk a contiguous run of 128-byte rows in shared memory (the layout
// of an M- or N-contiguous UMMA operand), so a whole operand stage is one copy.
bool encode_map_chunked(CUtensorMap* map, const void* base, int64_t cols, int64_t rows, int64_t batch, int64_t ld,
                        int64_t batch_stride, uint32_t box_rows, uint32_t box_chunks) {
  EncodeTiled fn = encode_tiled();
  if (!fn || cols % 64) return false;
  const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 64),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(ld) * 2, 128, static_cast<cuuint64_t>(batch_stride) * 2};
  const cuuint32_t box[4] = {64, box_rows, box_chunks, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 5-D map over a 32x32-blocked bf16 operand [batch][rows/32][cols/32][32][32] (row-major
// blocks), 64-byte swizzle: a box is `box_blocks` row blocks of one column block, i.e.
// 32 * box_blocks rows of 64 bytes, contiguous in shared memory.
bool encode_map_blocked(CUtensorMap* map, const void* base, int64_t row_blocks, int64_t col_blocks, int64_t batch,
                        int64_t batch_stride, uint32_t box_blocks) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[5] = {32, 32, static_cast<cuuint64_t>(col_blocks), static_cast<cuuint64_t>(row_blocks),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[4] = {64, 2048, static_cast<cuuint64_t>(col_blocks) * 2048,
                                 static_cast<cuuint64_t>(batch_stride) * 2};
  const cuuint32_t box[5] = {32, 32, 1, box_blocks, 1};
  const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D map over `rows` rows of `cols` bf16 values, `ld` elements apart, for stores of boxes of
// `box_rows` rows x 64 columns held in shared memory as 128-byte-swizzled rows.
bool encode_store_map(CUtensorMap* map, void* base, int64_t cols, int64_t rows, int64_t ld, uint32_t box_rows) {
  EncodeTiled fn = encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// High word of a matrix descriptor: stride byte offset, version 1, swizzle mode
// (2: 128-byte rows, 4: 64-byte rows).
__host__ __device__ inline uint32_t desc_hi(uint32_t sbo_bytes, uint32_t swizzle_mode = 2) {
  return (sbo_bytes >> 4) | (1u << 14) | (swizzle_mode << 29);
}

}  // namespace
}  // namespace b200
