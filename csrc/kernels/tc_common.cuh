// Blackwell (sm_100a) building blocks written as inline PTX: mbarrier, TMA tiled
// loads (never multicast), tcgen05 MMA / commit / TMEM alloc / TMEM load, and the
// shared-memory matrix descriptor for K-major 128-byte-swizzled bf16 tiles.
//
// Every wait is bounded (clock64 budget).  A wait that runs out returns false; the
// caller records a status word and unwinds to the common tail that frees TMEM.
#pragma once
#include "common.cuh"
#include <cuda.h>  // CUtensorMap (types only; the encode entry point is resolved at run time)

namespace poot {
namespace tc {

constexpr long long kWaitBudgetCycles = 1500000000LL;  // about 0.8 s at 1.9 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// Bounded wait on a barrier that only this CTA's own copies and MMAs complete: false after kWaitBudgetCycles.
// Callers start such a wait only after griddepcontrol.wait, so a predecessor that is itself waiting (on another
// rank, up to its step deadline) cannot make it run out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > kWaitBudgetCycles) return false;
  }
  return true;
}

// Bounded wait on a barrier whose completion depends on something that may legitimately last until the step
// deadline: the kernel before this one (it may be waiting for another rank; this kernel's producer warp sits in
// griddepcontrol.wait meanwhile), or the producer warp's own wait for peers' flags.  Its limit is later than those
// by construction: the step deadline plus kDependentSlackNs, or kLongWaitCycles when the control block carries no
// deadline.  It ends early only when the CTA-local failure flag is raised (the producer gave up on its ring).  It
// deliberately does not end on a recorded failure or on the host's abort word: the waits on other ranks do, their
// kernels then run to the end at once, and this barrier completes in the normal way microseconds later; stopping
// here as well would stall the ring and turn one failure into a slow drain.
constexpr unsigned long long kDependentSlackNs = 250000000ull;   // 0.25 s
constexpr long long kLongWaitCycles = 20000000000LL;              // about 10 s
__device__ __forceinline__ bool mbar_wait_dependent(uint32_t bar, uint32_t parity, const int* status,
                                                    const volatile int* cta_fail) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned tries = 0;
  while (!mbar_try(bar, parity)) {
    if ((++tries & 255u) == 0) {
      if (cta_fail != nullptr && *cta_fail != 0) return false;
      const unsigned long long d = ctl_deadline(status);
      if (d != 0ull && global_ns() > d + kDependentSlackNs) return false;
      if (clock64() - t0 > kLongWaitCycles) return false;
    }
  }
  return true;
}

// 2-D tiled TMA load into this CTA's shared memory, completion on an mbarrier.
// x is the innermost (contiguous) coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM -------------------------------------------------------------------
// Whole-warp calls (.sync.aligned).
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive on an mbarrier when all previously issued tcgen05.mma of this thread are complete.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int M, int N) {
  return (1u << 4)                     // D format f32
         | (1u << 7)                   // A format bf16
         | (1u << 10)                  // B format bf16
         | ((uint32_t)(N >> 3) << 17)  // N / 8
         | ((uint32_t)(M >> 4) << 24); // M / 16
}

// Shared-memory matrix descriptor: K-major tile whose rows are 128 bytes (64 bf16),
// 128-byte swizzle, 8-row groups 1024 bytes apart.  The tile base must be 1024-byte aligned;
// stepping K by 16 elements adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                    // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc

// Host side: bf16 2-D tensor map [rows, cols] row-major with pitch ld (elements),
// box = box_rows x 64 columns, 128-byte swizzle.  Returns 0 on success.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows);

}  // namespace poot
