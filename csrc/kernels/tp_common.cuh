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
// Every wait is bounded: on timeout the kernel records kTimeoutPeerFlag in the status word and goes on
// (the step's output is then invalid, the context stays usable, the host raises a typed error).
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
constexpr long long kFlagWaitBudgetCycles = 2000000000LL;  // about 1 s

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
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded poll until *flag >= target (wrap-safe).  False on timeout.
// `status` is the per-device word that records a wait that ran out: once any wait has failed, every later wait gives
// up at once instead of spending its own budget, so one lost signal costs about a second, not a second per kernel.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t target, const int* status = nullptr) {
  if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return false;
  const long long t0 = clock64();
  unsigned spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - target) < 0) {
    if (clock64() - t0 > kFlagWaitBudgetCycles) return false;
    if (status != nullptr && (++spins & 1023u) == 0 && *reinterpret_cast<const volatile int*>(status) != 0) return false;
    __nanosleep(40);
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

__device__ __forceinline__ void tp_signal_all(const TpArgs& tp, int ch, uint32_t target, int num_ctas) {
  __syncthreads();  // every thread's peer stores are ordered before thread 0's fence (CTA-scope barrier)
  if (threadIdx.x == 0) {
    // Release pattern: this CTA's peer stores (ordered before thread 0 by the barrier) -> system-scope fence ->
    // ticket -> observed by the last CTA -> system-scope fence -> flags.  (A device-scope fence here and a single
    // system-scope fence in the last CTA measured about 5 us faster per launch on one GPU; it is not used because
    // it has only been validated on two GPUs.)
    fence_acq_rel_sys();
    int t = atomicAdd(tp.ticket, 1);
    if (t == num_ctas - 1) {
      fence_acq_rel_sys();  // every CTA's stores (observed through the ticket) come before the flags
      for (int d = 0; d < tp.world; ++d) st_release_sys(tp.flags_peer[d] + ch * TP_MAX_WORLD + tp.rank, target);
      atomicExch(tp.ticket, 0);
    }
  }
}

}  // namespace poot
