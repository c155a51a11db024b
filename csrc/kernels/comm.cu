// Tensor-parallel communication kernels and the symmetric-memory setup they run on.
//
//  * poot_symm_* / poot_ipc_*: device allocations exported to the peer processes through CUDA IPC
//    (one process per GPU; every rank maps every other rank's block once at start-up).
//  * tp_begin_step: bumps the device-resident epoch once per model step (first node of the step graph) and
//    writes the step's deadline into the control block: the waits of one step share one budget.
//  * tp_argmax_exchange_kernel: the greedy pick over a vocabulary-parallel head without a library collective;
//    every rank pushes its stage-1 table into the peers' exchange areas and combines what it received.
//  * tp_norm_kernel: the consumer side of the fused GEMM + reduce-scatter and the producer side of the
//    fused all-gather + GEMM.  For this rank's S token rows it waits (bounded) for every rank's
//    contribution of the previous projection, adds them in rank order to the residual stream, applies
//    RMSNorm and pushes the normalised rows into every rank's gather buffer (the all-gather), then
//    publishes them with one flag write per peer.
//  * tp_link_probe_kernel: start-up delivery check of every directed link (pattern write, read back),
//    the counterpart of the reference's 256 B / 64 KiB / 4 MiB probe
//    (crates/poot-ptx-runtime/src/context.rs:643-682).
#include "tp_common.cuh"
#include "argmax_common.cuh"
#include <cstring>

namespace poot {

__global__ void tp_begin_step_kernel(int* epoch, int* status) {
  pdl_wait(); pdl_launch();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    *epoch += 1;
    if (status != nullptr) {
      const unsigned long long budget = *reinterpret_cast<const volatile unsigned long long*>(status + 6);
      *reinterpret_cast<volatile unsigned long long*>(status + 2) = budget ? global_ns() + budget : 0ull;
    }
  }
}

// out[b, :] = gathered rows [idx[b], :] of this rank's gather buffer for site ag_site, after every rank's rows have
// landed (the head of a prefill-sized step needs the few sampling rows, not all of them).  grid = rows, 128 threads.
__global__ void __launch_bounds__(128)
tp_gather_rows_kernel(const __nv_bfloat16* __restrict__ xs_local, const long long* __restrict__ idx,
                      __nv_bfloat16* __restrict__ out, int H, int* status, const __grid_constant__ TpArgs tp) {
  __shared__ int s_ok;
  pdl_wait(); pdl_launch();
  const uint32_t target = tp_target(tp, tp.ag_site, tp.ag_sites);
  if (threadIdx.x == 0) s_ok = tp_wait_all(tp.flags_local, tp.world, TP_CH_AG, target, tp.ag_site, status) ? 1 : 0;
  __syncthreads();
  const int R = tp.world * tp.S;
  long long r = idx[blockIdx.x];
  if (!POOT_IN_RANGE(r, R, kSiteGatherRow) || r < 0 || r >= R) r = 0;
  const uint4* src = reinterpret_cast<const uint4*>(xs_local + ((size_t)(target & 1u) * R + (size_t)r) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x)
    dst[c] = s_ok ? __ldcg(src + c) : make_uint4(0u, 0u, 0u, 0u);      // written by peers: never from L1
}

// Last kernel of a tensor-parallel step: the step deadline is cleared, so kernels of steps that do not start with
// tp_begin_step (steps on the library collectives, single-rank work on the same device) never read a stale one.
__global__ void tp_end_step_kernel(int* status) {
  pdl_wait(); pdl_launch();
  if (threadIdx.x == 0 && blockIdx.x == 0 && status != nullptr)
    *reinterpret_cast<volatile unsigned long long*>(status + 2) = 0ull;
}

// Greedy pick over vocabulary shards.  grid = rows, one warp per row.  `part_local` is this rank's stage-1 table
// [rows, groups, 3] (value bits, global index, first non-finite index).  Each CTA copies its row's slice into every
// peer's exchange area, the last CTA to finish publishes the exchange number on channel TP_CH_AX, then each CTA
// waits (bounded) for the peers' tables of the same exchange and reduces all of them for its row.  The exchange
// number lives in `ax_count` (device memory, read by every CTA before its ticket, advanced by the last CTA), the
// areas are double-buffered on its parity: a rank can only reach exchange n + 2 after every peer has signalled
// something later than its own combine of exchange n, because each step in between waits on all peers.
__global__ void __launch_bounds__(32)
tp_argmax_exchange_kernel(const int* __restrict__ part_local, int rows, int groups, int ax_cap, int bad_none,
                          int* __restrict__ out, int* ax_count, int* __restrict__ status,
                          const __grid_constant__ TpArgs tp) {
  __shared__ int s_ok;
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x, l = threadIdx.x;
  const uint32_t target = (uint32_t)*reinterpret_cast<const volatile int*>(ax_count) + 1u;
  const int parity = (int)(target & 1u);
  const int n = groups * 3;
  const int* src = part_local + (size_t)row * n;
  const size_t slot = (size_t)(parity * tp.world + tp.rank) * ax_cap + (size_t)row * n;
  for (int d = 0; d < tp.world; ++d) {
    if (d == tp.rank) continue;
    int* dst = tp.ax_peer[d] + slot;
    for (int e = l; e < n; e += 32) dst[e] = src[e];
  }
  tp_signal_all(tp, TP_CH_AX, target, (int)gridDim.x, status, ax_count);
  if (l == 0) {
    bool ok = true;
    for (int r = 0; r < tp.world && ok; ++r) {
      if (r == tp.rank) continue;
      int why = tp_wait_flag(tp.flags_local, tp.world, TP_CH_AX, r, target, status);
      if (why == 0 && ld_acquire_sys(tp.flags_local + TP_CH_POISON * TP_MAX_WORLD + r) != 0u) why = (int)kPeerFailed;
      if (why != 0) { ctl_fail(status, why, (1 << 20) + r); ok = false; }
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  Cand c{0.f, -1}; int b = bad_none;
  if (s_ok) {
    for (int e = l; e < tp.world * groups; e += 32) {
      const int pt = e / groups, g = e - pt * groups;
      const int* p = (pt == tp.rank) ? src + g * 3
                                     : tp.ax_peer[tp.rank] + (size_t)(parity * tp.world + pt) * ax_cap + (size_t)row * n + g * 3;
      // peers wrote these words: read them past L1
      Cand t{__int_as_float(__ldcg(p)), __ldcg(p + 1)};
      c = better(c, t);
      b = min(b, __ldcg(p + 2));
    }
  }
  c = warp_best(c); b = warp_min_i(b);
  if (l == 0) {
    const bool nf = b < bad_none;
    out[row * 2] = (nf || c.i < 0) ? 0 : c.i;
    out[row * 2 + 1] = nf ? b : -1;
  }
}

template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
tp_norm_kernel(__nv_bfloat16* __restrict__ h_shard,            // [S, H] residual stream rows owned by this rank
               const __nv_bfloat16* __restrict__ inbox_local,  // [2][world][S][H] contributions (or unused)
               const __nv_bfloat16* __restrict__ w,            // [H]
               __nv_bfloat16* __restrict__ x_local,            // one-shot form: normalised rows stay local (no push)
               int H, float eps, int* __restrict__ status, const __grid_constant__ TpArgs tp) {
  __shared__ float red[32];
  __shared__ int s_ok;
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x;
  const int H8 = H >> 3;
  const bool has_in = tp.rs_site >= 0;
  uint32_t rs_target = 0;
  if (has_in) {
    rs_target = tp_target(tp, tp.rs_site, tp.rs_sites);
    if (threadIdx.x == 0)
      s_ok = tp_wait_all(tp.flags_local, tp.world, TP_CH_RS, rs_target, tp.rs_site, status) ? 1 : 0;
    __syncthreads();
  }
  const int in_parity = (int)(rs_target & 1u);
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < H8) {
      unpack8(reinterpret_cast<const uint4*>(h_shard + (size_t)row * H)[c], v[i]);
      if (has_in) {
        for (int r = 0; r < tp.world; ++r) {  // rank order: every rank computes bit-identical sums
          const __nv_bfloat16* src = inbox_local + ((size_t)((in_parity * tp.world + r) * tp.S + row)) * H;
          float f[8];
          unpack8(__ldcg(reinterpret_cast<const uint4*>(src) + c), f);  // written by peers: never from L1
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += f[j];
        }
        uint4 packed = pack8(v[i]);
        unpack8(packed, v[i]);
        reinterpret_cast<uint4*>(h_shard + (size_t)row * H)[c] = packed;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  // block sum
  ss = warp_sum(ss);
  const int wid = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[wid] = ss;
  __syncthreads();
  float tot = (l < THREADS / 32) ? red[l] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / (float)H + eps);
  if (x_local != nullptr) {
    const uint4* wr2 = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(x_local + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < H8) {
        float wf[8], o[8];
        unpack8(wr2[c], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * wf[j];
        yr[c] = pack8(o);
      }
    }
    return;
  }
  const uint32_t ag_target = tp_target(tp, tp.ag_site, tp.ag_sites);
  const int out_parity = (int)(ag_target & 1u);
  // all-gather by push: this rank's rows go into every rank's gather buffer (16-byte peer stores, whole rows)
  const size_t xoff = ((size_t)(out_parity * tp.world * tp.S + tp.rank * tp.S + row)) * H;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < H8) {
      float wf[8], o[8];
      unpack8(wr[c], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * wf[j];
      const uint4 pk = pack8(o);
      for (int d = 0; d < tp.world; ++d) reinterpret_cast<uint4*>(tp.xs_peer[d] + xoff)[c] = pk;
    }
  }
  tp_signal_all(tp, TP_CH_AG, ag_target, (int)gridDim.x, status);
}

// Writes a pattern of n 32-bit words into `dst` (a peer mapping) / checks it in local memory.
__global__ void tp_probe_write_kernel(uint32_t* dst, size_t n, uint32_t seed) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = seed ^ (uint32_t)(i * 2654435761u);
}
__global__ void tp_probe_check_kernel(const uint32_t* src, size_t n, uint32_t seed, int* bad) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    if (src[i] != (seed ^ (uint32_t)(i * 2654435761u))) atomicAdd(bad, 1);
}

}  // namespace poot

using namespace poot;

POOT_API int poot_symm_alloc(size_t bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
POOT_API int poot_symm_free(void* p) { return (int)cudaFree(p); }
POOT_API int poot_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
POOT_API int poot_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
POOT_API int poot_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
POOT_API int poot_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// First kernel of a tensor-parallel step: epoch += 1, control block deadline = now + the block's step budget.
POOT_API int poot_tp_begin_step(int* epoch, int* status, cudaStream_t s) {
  return launch_k(tp_begin_step_kernel, dim3(1), dim3(32), 0, s, epoch, status);
}

POOT_API int poot_tp_gather_rows(const void* xs_local, const long long* idx, void* out, int rows, int H, int world, int rank,
                                 int S, int ag_site, int ag_sites, const int* epoch, void* flags_local, int* status,
                                 cudaStream_t s) {
  if (rows == 0) return 0;
  if (H % 8 || world < 1 || world > TP_MAX_WORLD || ag_site < 0 || status == nullptr) return (int)cudaErrorInvalidValue;
  TpArgs tp = {};
  tp.world = world; tp.rank = rank; tp.S = S; tp.ag_site = ag_site; tp.ag_sites = ag_sites; tp.rs_site = -1; tp.epoch = epoch;
  tp.flags_local = (uint32_t*)flags_local;
  return launch_k(tp_gather_rows_kernel, dim3(rows), dim3(128), 0, s, (const __nv_bfloat16*)xs_local, idx,
                  (__nv_bfloat16*)out, H, status, tp);
}

POOT_API int poot_tp_end_step(int* status, cudaStream_t s) {
  return launch_k(tp_end_step_kernel, dim3(1), dim3(32), 0, s, status);
}

// Greedy pick over `world` vocabulary shards through the symmetric block (no library collective).
//   part_local [rows, groups, 3] int32, ax_peer[r] = rank r's exchange area [2][world][ax_cap] int32 with
//   rows * groups * 3 <= ax_cap, ax_count = device counter of exchanges done, out [rows, 2] int32.
POOT_API int poot_tp_argmax_exchange(const int* part_local, int rows, int groups, int ax_cap, int vocab_total, int* out,
                                     int* ax_count, int world, int rank, void* flags_local, void* const* flags_peer,
                                     void* const* ax_peer, int* ticket, int* status, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (world < 2 || world > TP_MAX_WORLD || groups < 1 || (long long)rows * groups * 3 > (long long)ax_cap)
    return (int)cudaErrorInvalidValue;
  if (status == nullptr || ax_count == nullptr || ticket == nullptr) return (int)cudaErrorInvalidValue;
  TpArgs tp = {};
  tp.world = world; tp.rank = rank; tp.ag_site = -1; tp.rs_site = -1;
  tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
  for (int r = 0; r < world; ++r) { tp.flags_peer[r] = (uint32_t*)flags_peer[r]; tp.ax_peer[r] = (int*)ax_peer[r]; }
  return launch_k(tp_argmax_exchange_kernel, dim3(rows), dim3(32), 0, s, part_local, rows, groups, ax_cap, vocab_total,
                  out, ax_count, status, tp);
}

// ---- control block: host-mapped abort word -------------------------------------------------------------------
// The abort word lives in pinned host memory that the device reads through its mapped address, so the host can
// set it while kernels are running (a store to device memory from the host would need a stream).
POOT_API int poot_abort_word_alloc(int** host_ptr_out, void** device_ptr_out) {
  int* h = nullptr;
  cudaError_t e = cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return (int)e;
  *h = 0;
  void* d = nullptr;
  e = cudaHostGetDevicePointer(&d, h, 0);
  if (e != cudaSuccess) { cudaFreeHost(h); return (int)e; }
  *host_ptr_out = h;
  *device_ptr_out = d;
  return 0;
}
POOT_API void poot_abort_word_set(int* host_ptr, int value) {
  __atomic_store_n(host_ptr, value, __ATOMIC_SEQ_CST);
}
POOT_API int poot_abort_word_free(int* host_ptr) { return (int)cudaFreeHost(host_ptr); }

static void fill_tp(TpArgs& tp, int world, int rank, int S, int ag_site, int ag_sites, int rs_site, int rs_sites,
                    const int* epoch, void* flags_local, void* const* flags_peer, int* ticket) {
  tp.world = world; tp.rank = rank; tp.S = S;
  tp.ag_site = ag_site; tp.ag_sites = ag_sites; tp.rs_site = rs_site; tp.rs_sites = rs_sites;
  tp.epoch = epoch; tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
  for (int r = 0; r < world; ++r) tp.flags_peer[r] = (uint32_t*)flags_peer[r];
}

// h_shard [S,H] += sum over ranks of inbox (when rs_site >= 0); xs_local[parity] = rmsnorm(h_shard) * w; signal ag_site.
// x_local != null selects the one-shot form: `rows` token rows, inbox slots of S rows, output stays local.
POOT_API int poot_tp_norm(void* h_shard, const void* inbox_local, const void* w, void* const* xs_peer, void* x_local,
                          int rows, int H, float eps, int world, int rank, int S, int ag_site, int ag_sites, int rs_site, int rs_sites,
                          const int* epoch, void* flags_local, void* const* flags_peer, int* ticket, int* status,
                          cudaStream_t s) {
  if (H % 8 || world < 2 || world > TP_MAX_WORLD) return (int)cudaErrorInvalidValue;
  TpArgs tp = {};
  fill_tp(tp, world, rank, S, ag_site, ag_sites, rs_site, rs_sites, epoch, flags_local, flags_peer, ticket);
  for (int r = 0; r < world; ++r) tp.xs_peer[r] = xs_peer ? (__nv_bfloat16*)xs_peer[r] : nullptr;
  __nv_bfloat16* xl = (__nv_bfloat16*)x_local;
  const int grid = x_local ? rows : S;
  __nv_bfloat16* hb = (__nv_bfloat16*)h_shard;
  const __nv_bfloat16* ib = (const __nv_bfloat16*)inbox_local;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
  const int H8 = H / 8;
  if (H8 <= 128) return launch_k(tp_norm_kernel<128, 1>, dim3(grid), dim3(128), 0, s, hb, ib, wb, xl, H, eps, status, tp);
  if (H8 <= 256) return launch_k(tp_norm_kernel<256, 1>, dim3(grid), dim3(256), 0, s, hb, ib, wb, xl, H, eps, status, tp);
  if (H8 <= 512) return launch_k(tp_norm_kernel<512, 1>, dim3(grid), dim3(512), 0, s, hb, ib, wb, xl, H, eps, status, tp);
  if (H8 <= 1024) return launch_k(tp_norm_kernel<512, 2>, dim3(grid), dim3(512), 0, s, hb, ib, wb, xl, H, eps, status, tp);
  if (H8 <= 2048) return launch_k(tp_norm_kernel<512, 4>, dim3(grid), dim3(512), 0, s, hb, ib, wb, xl, H, eps, status, tp);
  return (int)cudaErrorInvalidValue;
}

POOT_API int poot_tp_probe_write(void* dst, long long n_words, unsigned seed, cudaStream_t s) {
  tp_probe_write_kernel<<<64, 256, 0, s>>>((uint32_t*)dst, (size_t)n_words, seed);
  return (int)cudaGetLastError();
}
POOT_API int poot_tp_probe_check(const void* src, long long n_words, unsigned seed, int* bad, cudaStream_t s) {
  tp_probe_check_kernel<<<64, 256, 0, s>>>((const uint32_t*)src, (size_t)n_words, seed, bad);
  return (int)cudaGetLastError();
}
