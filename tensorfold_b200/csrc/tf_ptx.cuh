// Thin wrappers over the sm_100a PTX the kernels use: mbarrier, bulk (TMA) copies, ldmatrix, mma.sync, packed fp32
// fma, programmatic dependent launch.  Every wait is bounded: it gives up after a fixed number of polls and reports it.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tf {

constexpr uint32_t WAIT_POLLS = 1u << 16;      // try_wait polls of up to 20 us each (about a second) before a wait is lost

enum ErrorCode : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,      // a consumer never saw its stage arrive
  ERR_WAIT_EMPTY = 2,     // the producer never got a stage back
  ERR_WAIT_SUMS = 3,      // a consumer never saw the group sums
  ERR_WAIT_PEER = 4,      // a peer flag never arrived (cross-GPU reduce)
  ERR_BAD_ITEM = 5,       // a plan item named an expert outside the table (the item was skipped)
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Adds expected bytes to the barrier's current phase without arriving on it.
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint (nanoseconds): the thread may sleep in hardware that long before it reports "not
// yet", so a waiting warp does not burn issue slots polling.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait by a whole warp (every lane calls it): false, for all lanes alike, when the barrier did not flip within
// WAIT_POLLS polls or another warp already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
  bool ok = false;
  for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
    if (mbar_try_wait_sleep(bar, parity, 20000u)) {
      ok = true;
      break;
    }
    if ((i & 255u) == 255u && *abort_flag) break;
  }
  return __all_sync(0xFFFFFFFFu, ok);
}

// One non-blocking test by a whole warp: true, for all lanes alike, when the phase with this parity is complete.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return __all_sync(0xFFFFFFFFu, ok != 0);
}

// Arrival on the same barrier in block `cta` of this cluster; the arriving thread's (and, through a preceding
// __syncthreads, its block's) earlier writes to that block's shared memory are visible to whoever sees the phase flip.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(bar)), "r"(cta));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// Bounded wait (whole warp, like mbar_wait) that acquires at cluster scope: for barriers other blocks arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
  bool ok = false;
  for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity), "r"(20000u)
        : "memory");
    if (done) {
      ok = true;
      break;
    }
    if ((i & 255u) == 255u && *abort_flag) break;
  }
  return __all_sync(0xFFFFFFFFu, ok);
}

// Bounded wait for a lane that already probed once: loops only if `ready` is false; uniform result across the warp.
__device__ __forceinline__ bool mbar_wait_probed(bool ready, uint64_t* bar, uint32_t parity, const volatile int* abort_flag) {
  if (__all_sync(0xFFFFFFFFu, ready)) return true;
  return mbar_wait(bar, parity, abort_flag);
}

// ---- the same barrier operations on 32-bit shared-memory addresses (no generic-to-shared conversion per call) ----
__device__ __forceinline__ void mbar32_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar32_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar32_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait by a whole warp: polls (each poll may suspend the warp in hardware for a while) until the phase
// completes, WAIT_POLLS polls have passed or another warp of the block has given up (abort word != 0).  `nap` > 0 adds
// that many nanoseconds of sleep between polls, for waits that are not latency-critical (a warp that polls flat out
// takes issue slots from the warps that work).  False (for all lanes alike) when the wait gave up.
#ifdef TF_WAIT_STATS
#define TF_COUNT_POLL(polls) ++(polls)
#else
#define TF_COUNT_POLL(polls) (void)0
#endif
__device__ __forceinline__ bool mbar32_wait(uint32_t bar, uint32_t parity, uint32_t abort_word, uint32_t nap = 0,
                                            uint32_t* polls = nullptr) {
  if (__all_sync(0xFFFFFFFFu, mbar32_try_wait(bar, parity))) return true;
  bool ok = false;
#pragma unroll 1
  for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
    if (polls) TF_COUNT_POLL(*polls);
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity), "r"(20000u)
                 : "memory");
    if (done) {
      ok = true;
      break;
    }
    if (nap) __nanosleep(nap);
    if ((i & 255u) == 255u) {
      uint32_t gone;
      asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(gone) : "r"(abort_word));
      if (gone) break;
    }
  }
  return __all_sync(0xFFFFFFFFu, ok);
}
__device__ __forceinline__ void bulk_load32(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d32(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
               "l"(map), "r"(bar), "r"(x), "r"(y)
               : "memory");
}

// Bulk asynchronous copy global -> shared of `bytes` (a multiple of 16; both addresses 16-byte aligned),
// completing on an mbarrier.  Every CTA fetches its own data.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// 16-byte asynchronous copy global -> shared through the load/store unit (rows of x: any 16-byte aligned placement).
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
// The executing thread's earlier cp.async copies arrive on `bar` when they land (the barrier's count includes them).
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Tensor-map (TMA) copy of one 2-D box global -> shared, completing on an mbarrier; (x, y) = (inner, outer) element
// coordinates of the box's corner.  x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_addr(dst)),
               "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col).  Each D element is the dot of one A row with one B
// column; it does not depend on the other rows or columns of the operands.
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same with a zero accumulator input: D = A * B (the first k-step of a group needs no cleared registers).
__device__ __forceinline__ void mma_bf16_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));      // (a & mask) | orv
  return r;
}

// Loads from a 32-bit shared-memory address (the generic-pointer form costs 64-bit address arithmetic per load).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

// (d0, d1) = (a0, a1) * (b0, b1) + (d0, d1): two IEEE fp32 fused multiply-adds in one instruction (each half rounds
// exactly as fmaf does, so results carry the same bits as two scalar fmas).
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rd, {%0, %1};\n"
      "fma.rn.f32x2 rd, ra, rb, rd;\nmov.b64 {%0, %1}, rd;\n}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// Two fp32 values in one 64-bit register, the operand form of fma.rn.f32x2.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// a * b + c on both halves, each an IEEE fp32 fused multiply-add (the bits of two fmaf calls)
__device__ __forceinline__ uint64_t fma2p(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Programmatic dependent launch: wait for the grid this one depends on (no-op without the launch attribute), and
// let the dependent grid start its own prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace tf
