// Tensor-parallel communication kernels and the symmetric-memory setup they run on.
//
//  * poot_symm_* / poot_ipc_*: device allocations exported to the peer processes through CUDA IPC
//    (one process per GPU; every rank maps every other rank's block once at start-up).
//  * tp_begin_step: bumps the device-resident epoch once per model step (first node of the step graph).
//  * tp_norm_kernel: the consumer side of the fused GEMM + reduce-scatter and the producer side of the
//    fused all-gather + GEMM.  For this rank's S token rows it waits (bounded) for every rank's
//    contribution of the previous projection, adds them in rank order to the residual stream, applies
//    RMSNorm and pushes the normalised rows into every rank's gather buffer (the all-gather), then
//    publishes them with one flag write per peer.
//  * tp_link_probe_kernel: start-up delivery check of every directed link (pattern write, read back),
//    the counterpart of the reference's 256 B / 64 KiB / 4 MiB probe
//    (crates/poot-ptx-runtime/src/context.rs:643-682).
#include "tp_common.cuh"
#include <cstring>

namespace poot {

__global__ void tp_begin_step_kernel(int* epoch) {
  pdl_wait(); pdl_launch();
  if (threadIdx.x == 0 && blockIdx.x == 0) *epoch += 1;
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
    if (threadIdx.x == 0) {
      bool ok = true;
      for (int r = 0; r < tp.world; ++r)
        if (!wait_flag_ge(tp.flags_local + TP_CH_RS * TP_MAX_WORLD + r, rs_target, status)) ok = false;
      if (!ok) atomicExch(status, (int)kTimeoutPeerFlag);
      s_ok = ok ? 1 : 0;
    }
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
  tp_signal_all(tp, TP_CH_AG, ag_target, (int)gridDim.x);
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

POOT_API int poot_tp_begin_step(int* epoch, cudaStream_t s) {
  return launch_k(tp_begin_step_kernel, dim3(1), dim3(32), 0, s, epoch);
}

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
