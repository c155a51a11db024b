// Tensor-parallel plumbing shared by the fused compute+collective kernels.
//
// Ranks are processes, one per GPU.  Each rank owns a block of "symmetric" device memory that every
// peer maps through CUDA IPC; kernels read and write peers' memory with ordinary loads/stores (and
// non-multicast TMA loads) over NVLink.  Synchronisation uses monotone 32-bit flags in that memory:
//
//   flags[ch * 8 + src]   written by rank `src` (st.release.sys on the peer mapping), polled locally
//   ch 0 = "my reduce-scatter contribution for site s has landed in your inbox"
//   ch 1 = "my normalised activation shard for site s is ready to be gathered"
//
// A step of the model has a fixed number of sites per channel; a device-resident epoch counter is
// bumped once per step, so the value to signal / wait for is (epoch-1)*sites + site + 1 and nothing
// is ever reset between CUDA-graph replays.  Buffers are double-buffered on the parity of that value.
//
//   ch 3 = greedy-pick exchange, ch 4 / 5 = expert-parallel dispatch / combine (ep_exchange.cu)
//   ch 2 = poison: flags[2 * 8 + src] != 0 means rank `src` recorded a failure; it is published with the rank's
//          next signal, and every wait on this rank that sees it gives up with kPeerFailed, so one rank's failure
//          reaches all ranks within one site instead of leaving them to compute on stale inboxes
//
// Every wait is bounded, and the waits of one step share one budget: the step's first kernel (tp_begin_step)
// writes a deadline into the control block, and a wait gives up when the deadline has passed, when a failure has
// already been recorded for the step, when a peer's poison word is set, or when the host has set the abort word.
// The kernel then records the first cause in the control block and goes on without further waiting (the step's
// output is invalid, the context stays usable, the host raises a typed error and marks the engine dead).
//
// This replaces the reference's lowering of AllReduce / AllGather to world*(world-1) host-issued peer
// copies per collective plus Add kernels (crates/poot-graph-plan/src/passes/sharding.rs:1165-1357,
// crates/poot-ptx-runtime/src/context.rs:741-785).
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace poot {

constexpr int TP_MAX_WORLD = 8;
constexpr int TP_CH_RS = 0;
constexpr int TP_CH_AG = 1;
constexpr int TP_CH_POISON = 2;
constexpr int TP_CH_AX = 3;       // "my greedy-pick partial table of exchange n has landed in your exchange area"
constexpr int TP_CH_EPD = 4;      // "the rows of exchange n that I route to your experts have landed in your receive area"
constexpr int TP_CH_EPC = 5;      // "your rows of exchange n, through my experts, have landed in your combine area"
constexpr int TP_FLAG_WORDS = 6 * TP_MAX_WORLD;
// Limit of one wait when the control block carries no step deadline (plain kernel tests): about 1 s.
constexpr long long kFlagWaitBudgetCycles = 2000000000LL;

struct TpArgs {
  int world;          // 1 = not tensor parallel (all other fields unused)
  int rank;
  int S;              // token rows per rank (multiple of 8); padded step rows = world * S
  int ag_site;        // >= 0: gather the X operand from the peers' activation shards for this site
  int ag_sites;       // gather sites per step
  int rs_site;        // >= 0: scatter the output rows to their owner ranks' inboxes for this site
  int rs_sites;       // scatter sites per step
  int ld_inbox;       // row pitch (elements) of an inbox slice = hidden size
  int oneshot;        // 1: every rank receives every rank's whole partial (one-shot all-reduce; S = rows per slot)
  const int* epoch;             // device step counter (>= 1 inside a step)
  uint32_t* flags_local;        // this rank's flag block [2 * 8]
  uint32_t* flags_peer[TP_MAX_WORLD];        // every rank's flag block (peer mappings; [rank] = local)
  __nv_bfloat16* inbox_peer[TP_MAX_WORLD];   // every rank's inbox [2][world][S][ld_inbox] bf16
  __nv_bfloat16* xs_peer[TP_MAX_WORLD];      // every rank's gather buffer [2][world*S][ld_inbox] bf16
  int* ticket;                  // local CTA-completion counter (self-resetting)
  int* ax_peer[TP_MAX_WORLD];   // every rank's greedy-pick exchange area [2][world][ax_cap] ints (tp_argmax_exchange only)
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded poll until flags_local[ch][src] >= target (wrap-safe).  Returns 0 when the flag arrived, otherwise the
// Status code that ended the wait; the caller records it with ctl_fail.  A wait that starts after a failure has
// been recorded returns at once, so one lost signal costs one budget, not one per kernel.
__device__ __forceinline__ int tp_wait_flag(const uint32_t* flags_local, int world, int ch, int src, uint32_t target,
                                            const int* status) {
  const uint32_t* flag = flags_local + ch * TP_MAX_WORLD + src;
  if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return 0;
  int why = ctl_stop_reason(status);
  if (why != 0) return why;
  const bool has_deadline = ctl_deadline(status) != 0ull;
  const long long t0 = clock64();
  unsigned spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - target) < 0) {
    if ((++spins & 63u) == 0) {
      for (int r = 0; r < world; ++r)
        if (*reinterpret_cast<const volatile uint32_t*>(flags_local + TP_CH_POISON * TP_MAX_WORLD + r) != 0u)
          return (int)kPeerFailed;
      why = ctl_stop_reason(status);
      if (why != 0) return why;
      if (!has_deadline && clock64() - t0 > kFlagWaitBudgetCycles) return (int)kTimeoutPeerFlag;
    }
    __nanosleep(64);
  }
  return 0;
}

// Waits for every rank's flag of (ch, target).  True when all arrived; otherwise records the first cause (detail =
// site * 16 + the rank that was missing) and returns false.
__device__ __forceinline__ bool tp_wait_all(const uint32_t* flags_local, int world, int ch, uint32_t target, int site,
                                            int* status) {
  // A peer that gave up has run ahead without waiting and has already published every flag of the step: its flags
  // alone would let this rank compute on contributions that are not valid.  Its poison word says so.
  for (int r = 0; r < world; ++r)
    if (ld_acquire_sys(flags_local + TP_CH_POISON * TP_MAX_WORLD + r) != 0u) {
      ctl_fail(status, (int)kPeerFailed, site * 16 + r);
      return false;
    }
  for (int r = 0; r < world; ++r) {
    const int why = tp_wait_flag(flags_local, world, ch, r, target, status);
    if (why != 0) {
      ctl_fail(status, why == (int)kStepDeadline ? (int)kStepDeadline : why, site * 16 + r);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ uint32_t tp_target(const TpArgs& tp, int site, int sites) {
  return (uint32_t)(*tp.epoch - 1) * (uint32_t)sites + (uint32_t)site + 1u;
}

// Called by every CTA after its peer stores; the last CTA to arrive publishes `target` on channel `ch`
// of every rank's flag block.  All threads of the CTA must call it (it contains a barrier).
// Acquire-release fence at system scope.  Deliberately NOT the sequentially consistent fence that
// __threadfence_system() emits: SC fences are totally ordered across the GPU, so one per CTA serialises a few
// hundred CTAs behind one another (measured: about 25 us per kernel); acquire-release fences only order this
// thread's own accesses, which is all the release pattern below needs.
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

__device__ __forceinline__ void tp_signal_all(const TpArgs& tp, int ch, uint32_t target, int num_ctas,
                                              const int* status = nullptr, int* bump = nullptr) {
  __syncthreads();  // every thread's peer stores are ordered before thread 0's fence (CTA-scope barrier)
  if (threadIdx.x == 0) {
    // Release pattern: this CTA's peer stores (ordered before thread 0 by the barrier) -> system-scope fence ->
    // ticket -> observed by the last CTA -> system-scope fence -> flags.  Every CTA issues its own system-scope
    // fence: a device-scope fence per CTA with a single system-scope fence in the last CTA is a few microseconds
    // faster per launch but was never validated beyond two GPUs, so it is not used.
    fence_acq_rel_sys();
    int t = atomicAdd(tp.ticket, 1);
    if (t == num_ctas - 1) {
      fence_acq_rel_sys();  // every CTA's stores (observed through the ticket) come before the flags
      if (ctl_failed(status)) {
        // this rank's step is invalid: say so before the flag that lets the peers go on
        const uint32_t code = (uint32_t)*reinterpret_cast<const volatile int*>(status);
        for (int d = 0; d < tp.world; ++d)
          if (d != tp.rank) st_release_sys(tp.flags_peer[d] + TP_CH_POISON * TP_MAX_WORLD + tp.rank, code);
      }
      for (int d = 0; d < tp.world; ++d) st_release_sys(tp.flags_peer[d] + ch * TP_MAX_WORLD + tp.rank, target);
      if (bump != nullptr) *reinterpret_cast<volatile int*>(bump) = (int)target;  // every CTA read it before its ticket
      atomicExch(tp.ticket, 0);
    }
  }
}

}  // namespace poot
