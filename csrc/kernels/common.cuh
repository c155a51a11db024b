// Shared device helpers for the sm_100a kernel library.
//
// Every exported launcher in this library has the C ABI
//   extern "C" int poot_<name>(..., cudaStream_t stream)
// and returns the cudaError_t of its launch (0 = success).  Python loads the
// library with ctypes and passes raw device pointers, so no torch headers are
// needed to build it and the build takes seconds.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define POOT_API extern "C" __attribute__((visibility("default")))

#ifndef POOT_SPIN_LIMIT
// Upper bound on polls of any device-side wait (mbarrier, peer flag).  A wait
// that runs out records a status word and returns; nothing spins forever.
#define POOT_SPIN_LIMIT (1u << 24)
#endif

namespace poot {

// Status codes written to a kernel's status word (0 = ok).
enum Status : int {
  kOk = 0,
  kTimeoutProducer = 1,
  kTimeoutMma = 2,
  kTimeoutEpilogue = 3,
  kTimeoutPeerFlag = 4,
  kBadArgument = 5,
  kAborted = 6,        // the host set the abort word while a wait was pending
  kStepDeadline = 7,   // the step's deadline passed while a wait was pending
  kPeerFailed = 8,     // another rank published a failure (poison word) for the current step
};

// ---- control block -----------------------------------------------------------------------------
// Every launcher takes an `int* status`.  It points at a 16-word block in device memory, one per device:
//
//   [0]     first failure of a bounded wait (a Status code); written with compare-and-swap from 0, so the
//           first cause stays and later, consequential failures do not overwrite it
//   [1]     detail of that failure (site index, peer rank or ring slot; -1 when there is none)
//   [2..3]  step deadline: a %globaltimer value (ns).  0 = none.  Set by the step's first kernel; every wait on
//           another rank gives up once it has passed, so the waits of one step share ONE budget
//   [4..5]  device-visible address of a host-mapped abort word (0 = none).  The host sets that word to make every
//           pending and future wait return at once (drain before exit, signal handlers, watchdogs)
//   [6..7]  the budget (ns) that the step's first kernel adds to %globaltimer to form the deadline (0 = none)
//   [8]     number of waits that gave up since the block was last cleared (diagnostic)
//
// A block whose words 1.. are zero behaves like the old single status word.
constexpr int kCtlWords = 16;

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool ctl_failed(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
}
// Record a failure; only the first one of a step is kept.
__device__ __forceinline__ void ctl_fail(int* status, int code, int detail = -1) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) reinterpret_cast<volatile int*>(status)[1] = detail;
  atomicAdd(status + 8, 1);
}
__device__ __forceinline__ unsigned long long ctl_deadline(const int* status) {
  return status == nullptr ? 0ull : *reinterpret_cast<const volatile unsigned long long*>(status + 2);
}
__device__ __forceinline__ bool ctl_host_abort(const int* status) {
  if (status == nullptr) return false;
  const unsigned long long a = *reinterpret_cast<const volatile unsigned long long*>(status + 4);
  return a != 0ull && *reinterpret_cast<const volatile int*>(a) != 0;
}
// Why a pending wait should stop now (0 = keep waiting).  `slack_ns` is added to the step deadline: waits that
// depend on another wait of the same kernel get a later limit than the wait they depend on.
__device__ __forceinline__ int ctl_stop_reason(const int* status, unsigned long long slack_ns = 0ull) {
  if (status == nullptr) return 0;
  if (*reinterpret_cast<const volatile int*>(status) != 0) return *reinterpret_cast<const volatile int*>(status);
  if (ctl_host_abort(status)) return (int)kAborted;
  const unsigned long long d = ctl_deadline(status);
  if (d != 0ull && global_ns() > d + slack_ns) return (int)kStepDeadline;
  return 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// bf16 pair packed in a 32-bit word -> two floats (exact: bf16 is the top half of f32).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// 16-byte streaming load that bypasses L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

template <typename T> struct Vec8;  // 8 elements = one 16-byte access for 2-byte types

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  f[0] = bf16lo(v.x); f[1] = bf16hi(v.x);
  f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  f[4] = bf16lo(v.z); f[5] = bf16hi(v.z);
  f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  v.x = pack_bf16(f[0], f[1]);
  v.y = pack_bf16(f[2], f[3]);
  v.z = pack_bf16(f[4], f[5]);
  v.w = pack_bf16(f[6], f[7]);
  return v;
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of the library starts with pdl_wait() (block until the preceding kernel's memory is
// visible; a no-op for an ordinary launch) and pdl_launch() (let the next kernel's CTAs be scheduled
// while this one still runs).  With the library-wide switch on, launchers add the programmatic stream
// serialization attribute, so launch latency and kernel prologues overlap the predecessor's tail.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_poot_pdl;

template <typename... KArgs, typename... Args>
inline int launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_poot_pdl ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- checked build ---------------------------------------------------------------------------------------------
// With -DPOOT_DEBUG_BOUNDS every data-dependent index a kernel reads from device memory (token ids, K/V slots, block
// ids, expert ids, row maps) is compared with its bound before use.  An index outside it is not trapped on: the
// kernel records {site, source line, index, bound} - the first record wins - substitutes a safe index and carries
// on, so the context stays usable and the host reads the record after the step (poot_debug_bounds_read).  Bounds a
// kernel is not given as an argument (pool slots, pool blocks, recurrent-state rows) are set once from the host
// (poot_debug_bounds_limit).  The record and the limits are per translation unit; each unit registers its accessors
// in one host-side list, which the two entry points walk.  A release build compiles every check away.
enum BoundsSite {
  kSiteTokenId = 1, kSiteKvSlot = 2, kSiteBlockId = 3, kSitePosition = 4, kSiteExpertId = 5, kSiteRowMap = 6,
  kSiteLogitIndex = 7, kSiteSeqRow = 8, kSiteStateRow = 9, kSiteGatherRow = 10,
};
enum BoundsLimit { kLimPoolSlots = 0, kLimPoolBlocks = 1, kLimStateRows = 2, kLimCount = 4 };

#ifdef POOT_DEBUG_BOUNDS
}  // namespace poot
#include <vector>
namespace poot {
namespace dbg {
static __device__ int g_fault[4];
static __device__ long long g_limit[kLimCount];
struct Unit {
  int (*read)(int*);
  int (*clear)();
  int (*limit)(int, long long);
};
inline std::vector<Unit>& units() {
  static std::vector<Unit> u;
  return u;
}
static int unit_read(int* out4) { return (int)cudaMemcpyFromSymbol(out4, g_fault, sizeof(int) * 4); }
static int unit_clear() {
  const int z[4] = {0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_fault, z, sizeof(z));
}
static int unit_limit(int which, long long v) {
  return (int)cudaMemcpyToSymbol(g_limit, &v, sizeof(v), sizeof(long long) * which);
}
static const int unit_registered = (units().push_back(Unit{unit_read, unit_clear, unit_limit}), 0);

__device__ __forceinline__ bool in_range(long long i, long long n, int site, int line) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_fault[0], 0, site) == 0) {
    g_fault[1] = line;
    g_fault[2] = (int)(i < -2147483647LL ? -2147483647LL : (i > 2147483647LL ? 2147483647LL : i));
    g_fault[3] = (int)(n > 2147483647LL ? 2147483647LL : n);
  }
  return false;
}
__device__ __forceinline__ long long limit(int which) {
  const long long v = g_limit[which];
  return v > 0 ? v : 0x7fffffffffffffffLL;
}
}  // namespace dbg
#define POOT_IN_RANGE(i, n, site) (::poot::dbg::in_range((long long)(i), (long long)(n), (site), __LINE__))
#define POOT_LIMIT(which) (::poot::dbg::limit(which))
#else
#define POOT_IN_RANGE(i, n, site) (true)
#define POOT_LIMIT(which) (0x7fffffffffffffffLL)
#endif

}  // namespace poot
