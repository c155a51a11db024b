// Expert parallelism over a token-sharded residual stream: dispatch and combine as all-to-all exchanges through the
// symmetric block, fused with the router's output on one side and the grouped expert GEMMs on the other.
//
// Each rank owns S token rows of the step (the reduce-scatter form of tensor parallelism) and E / world experts.
//
//   ep_plan      (owner)   from the router's ids [S * k]: destination rank and position of every (token, slot) row in
//                          that rank's receive area, in row order (deterministic), and the row count per destination
//   ep_dispatch  (owner)   each row's activation goes into ITS expert's rank only - recv[dst][src = me][pos] - with
//                          (expert id, source row, gate); counts are published, then channel EPD is signalled
//   ep_mask      (expert)  waits for every source's EPD flag, then marks which receive slots hold rows of this exchange
//                          (expert id, or -1) and reads their gates; moe_align groups them by local expert
//   ep_gather    (expert)  received rows into the grouped order the expert GEMMs walk (peer-written: read past L1)
//   ep_combine   (expert)  each result row (gate-scaled by the down projection) goes back to its source rank's combine
//                          area at (token, slot); channel EPC is signalled
//   ep_finish    (owner)   waits for every rank's EPC flag, then h[t] += sum over the token's k slots, in slot order
//
// A token's row crosses NVLink to at most k ranks and its k results come back once: (world - 1) / world of 2 k rows per
// token instead of the (world - 1) rows an all-gather of the activations moves.  Plain peer stores and monotone flags,
// double-buffered on the exchange's parity; every wait is bounded by the step deadline like the other channels'.
#include "tp_common.cuh"

namespace poot {

struct EpArgs {
  TpArgs tp;          // world, rank, epoch, flags_local, flags_peer, ticket (the other fields are unused here)
  int S, k, cap, H, e_local;
  int site, sites;
  __nv_bfloat16* recv_peer[TP_MAX_WORLD];   // every rank's receive area [2][world][cap][H]
  int* meta_peer[TP_MAX_WORLD];             // [2][world][cap][4]: expert id, source row, gate bits, 0
  int* count_peer[TP_MAX_WORLD];            // [2][world]
  __nv_bfloat16* back_peer[TP_MAX_WORLD];   // every rank's combine area [2][S * k][H]
};

__device__ __forceinline__ uint32_t ep_target(const EpArgs& a) {
  return (uint32_t)(*a.tp.epoch - 1) * (uint32_t)a.sites + (uint32_t)a.site + 1u;
}

constexpr int EP_PLAN_THREADS = 1024;

// One CTA.  dest[i] = rank of row i's expert, dpos[i] = how many earlier rows go to the same rank, counts[d] = rows for d.
__global__ void __launch_bounds__(EP_PLAN_THREADS)
ep_plan_kernel(const int* __restrict__ ids, int n, int e_local, int world, int* __restrict__ dest, int* __restrict__ dpos,
               int* __restrict__ counts) {
  __shared__ int part[EP_PLAN_THREADS][TP_MAX_WORLD];
  pdl_wait(); pdl_launch();
  const int t = threadIdx.x;
  const int chunk = (n + EP_PLAN_THREADS - 1) / EP_PLAN_THREADS;
  const int a = min(n, t * chunk), b = min(n, a + chunk);
  int mine[TP_MAX_WORLD];
#pragma unroll
  for (int d = 0; d < TP_MAX_WORLD; ++d) mine[d] = 0;
  for (int i = a; i < b; ++i) {
    int d = ids[i] / e_local;
    if (!POOT_IN_RANGE(d, world, kSiteExpertId) || d < 0 || d >= world) d = 0;
#pragma unroll
    for (int x = 0; x < TP_MAX_WORLD; ++x) mine[x] += (x == d);
  }
#pragma unroll
  for (int d = 0; d < TP_MAX_WORLD; ++d) part[t][d] = mine[d];
  __syncthreads();
  if (t < world) {                       // exclusive scan over the threads' chunks, one destination per thread
    int run = 0;
    for (int x = 0; x < EP_PLAN_THREADS; ++x) {
      const int v = part[x][t];
      part[x][t] = run;
      run += v;
    }
    counts[t] = run;
  }
  __syncthreads();
  int at[TP_MAX_WORLD];
#pragma unroll
  for (int d = 0; d < TP_MAX_WORLD; ++d) at[d] = part[t][d];
  for (int i = a; i < b; ++i) {
    int d = ids[i] / e_local;
    if (d < 0 || d >= world) d = 0;
    dest[i] = d;
    int p = 0;
#pragma unroll
    for (int x = 0; x < TP_MAX_WORLD; ++x)
      if (x == d) p = at[x]++;
    dpos[i] = p;
  }
}

// grid = S * k rows, 128 threads.
__global__ void __launch_bounds__(128)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ ids, const float* __restrict__ gates,
                   const int* __restrict__ dest, const int* __restrict__ dpos, const int* __restrict__ counts,
                   const __grid_constant__ EpArgs a, int* status) {
  pdl_wait(); pdl_launch();
  const int i = blockIdx.x;
  const uint32_t target = ep_target(a);
  const int parity = (int)(target & 1u);
  const int d = dest[i], p = dpos[i];
  if (p < a.cap) {
    const size_t slot = (size_t)(parity * a.tp.world + a.tp.rank) * a.cap + p;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / a.k) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(a.recv_peer[d] + slot * a.H);
    for (int c = threadIdx.x; c < a.H / 8; c += blockDim.x) dst[c] = src[c];
    if (threadIdx.x == 0) {
      int4 m = make_int4(ids[i], i, __float_as_int(gates[i]), 0);
      *reinterpret_cast<int4*>(a.meta_peer[d] + slot * 4) = m;
    }
  }
  if (i == 0 && threadIdx.x < a.tp.world)
    a.count_peer[threadIdx.x][parity * a.tp.world + a.tp.rank] = counts[threadIdx.x];
  tp_signal_all(a.tp, TP_CH_EPD, target, (int)gridDim.x, status);
}

// grid over world * cap receive slots.  ids_out / gate_out are indexed like the receive area of this exchange.
__global__ void __launch_bounds__(256)
ep_mask_kernel(const int* __restrict__ meta_local, const int* __restrict__ count_local, int* __restrict__ ids_out,
               float* __restrict__ gate_out, const __grid_constant__ EpArgs a, int* status) {
  __shared__ int s_ok;
  pdl_wait(); pdl_launch();
  const uint32_t target = ep_target(a);
  const int parity = (int)(target & 1u);
  if (threadIdx.x == 0) s_ok = tp_wait_all(a.tp.flags_local, a.tp.world, TP_CH_EPD, target, a.site, status) ? 1 : 0;
  __syncthreads();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.tp.world * a.cap) return;
  const int src = idx / a.cap, pos = idx - src * a.cap;
  int id = -1;
  float g = 0.f;
  if (s_ok && pos < __ldcg(count_local + parity * a.tp.world + src)) {
    const int4 m = __ldcg(reinterpret_cast<const int4*>(meta_local + ((size_t)(parity * a.tp.world) * a.cap + idx) * 4));
    id = m.x;
    g = __int_as_float(m.z);
  }
  ids_out[idx] = id;
  gate_out[idx] = g;
}

// xs[p, :] = received row sorted_rows[p] (zeros for padding rows); gate_sorted[p] = its gate.  grid = max_tiles * block.
__global__ void __launch_bounds__(128)
ep_gather_kernel(const __nv_bfloat16* __restrict__ recv_local, const int* __restrict__ sorted_rows,
                 const float* __restrict__ gate_flat, const int* __restrict__ n_tiles, int block, int H,
                 __nv_bfloat16* __restrict__ xs, float* __restrict__ gate_sorted, const __grid_constant__ EpArgs a) {
  pdl_wait(); pdl_launch();
  const int p = blockIdx.x;
  if (p >= *n_tiles * block) return;
  const int parity = (int)(ep_target(a) & 1u);
  const int i = sorted_rows[p];
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * H);
  if (i < 0) {
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x == 0) gate_sorted[p] = 0.f;
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(recv_local + ((size_t)(parity * a.tp.world) * a.cap + i) * H);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = __ldcg(src + c);      // written by peers: never from L1
  if (threadIdx.x == 0) gate_sorted[p] = gate_flat[i];
}

// grid over world * cap receive slots: slot idx's result row y[pos[idx]] goes back to its source.
__global__ void __launch_bounds__(128)
ep_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, const int* __restrict__ meta_local,
                  const __grid_constant__ EpArgs a, int* status) {
  pdl_wait(); pdl_launch();
  const int idx = blockIdx.x;
  const uint32_t target = ep_target(a);
  const int parity = (int)(target & 1u);
  const int p = pos[idx];
  if (p >= 0) {
    const int src = idx / a.cap;
    const int row = __ldcg(meta_local + ((size_t)(parity * a.tp.world) * a.cap + idx) * 4 + 1);
    if (POOT_IN_RANGE(row, a.S * a.k, kSiteRowMap) && row >= 0 && row < a.S * a.k) {
      const uint4* s = reinterpret_cast<const uint4*>(y + (size_t)p * a.H);
      uint4* d = reinterpret_cast<uint4*>(a.back_peer[src] + ((size_t)parity * a.S * a.k + row) * a.H);
      for (int c = threadIdx.x; c < a.H / 8; c += blockDim.x) d[c] = s[c];
    }
  }
  tp_signal_all(a.tp, TP_CH_EPC, target, (int)gridDim.x, status);
}

// grid = S token rows.  h[t] += sum_j back[t * k + j], slots in order.
__global__ void __launch_bounds__(256)
ep_finish_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ back_local,
                 const __grid_constant__ EpArgs a, int* status) {
  __shared__ int s_ok;
  pdl_wait(); pdl_launch();
  const uint32_t target = ep_target(a);
  const int parity = (int)(target & 1u);
  if (threadIdx.x == 0) s_ok = tp_wait_all(a.tp.flags_local, a.tp.world, TP_CH_EPC, target, a.site, status) ? 1 : 0;
  __syncthreads();
  if (!s_ok) return;                      // the step is invalid already; the residual stream is left as it was
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < a.H / 8; c += blockDim.x) {
    float acc[8];
    unpack8(reinterpret_cast<const uint4*>(h + (size_t)t * a.H)[c], acc);
    for (int j = 0; j < a.k; ++j) {
      float f[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(back_local + ((size_t)parity * a.S * a.k + (size_t)t * a.k + j) * a.H) + c), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    reinterpret_cast<uint4*>(h + (size_t)t * a.H)[c] = pack8(acc);
  }
}

static int ep_fill(EpArgs& a, int world, int rank, int S, int k, int cap, int H, int e_local, int site, int sites,
                   const int* epoch, void* flags_local, void* const* flags_peer, void* const* recv_peer,
                   void* const* meta_peer, void* const* count_peer, void* const* back_peer, int* ticket) {
  if (world < 1 || world > TP_MAX_WORLD || rank < 0 || rank >= world || S < 1 || k < 1 || cap < S * k || H % 8 || e_local < 1 ||
      site < 0 || site >= sites || epoch == nullptr || flags_local == nullptr || ticket == nullptr)
    return (int)cudaErrorInvalidValue;
  a = EpArgs{};
  a.tp.world = world; a.tp.rank = rank; a.tp.epoch = epoch; a.tp.flags_local = (uint32_t*)flags_local; a.tp.ticket = ticket;
  a.tp.ag_site = -1; a.tp.rs_site = -1;
  a.S = S; a.k = k; a.cap = cap; a.H = H; a.e_local = e_local; a.site = site; a.sites = sites;
  for (int r = 0; r < world; ++r) {
    a.tp.flags_peer[r] = (uint32_t*)flags_peer[r];
    a.recv_peer[r] = recv_peer ? (__nv_bfloat16*)recv_peer[r] : nullptr;
    a.meta_peer[r] = meta_peer ? (int*)meta_peer[r] : nullptr;
    a.count_peer[r] = count_peer ? (int*)count_peer[r] : nullptr;
    a.back_peer[r] = back_peer ? (__nv_bfloat16*)back_peer[r] : nullptr;
  }
  return 0;
}

}  // namespace poot

using namespace poot;

POOT_API int poot_ep_plan(const int* ids, int n, int e_local, int world, int* dest, int* dpos, int* counts, cudaStream_t s) {
  if (n < 1 || e_local < 1 || world < 1 || world > TP_MAX_WORLD) return (int)cudaErrorInvalidValue;
  return launch_k(ep_plan_kernel, dim3(1), dim3(EP_PLAN_THREADS), 0, s, ids, n, e_local, world, dest, dpos, counts);
}

#define EP_COMMON_PARAMS                                                                                              \
  int world, int rank, int S, int k, int cap, int H, int e_local, int site, int sites, const int *epoch,              \
      void *flags_local, void *const *flags_peer, void *const *recv_peer, void *const *meta_peer,                     \
      void *const *count_peer, void *const *back_peer, int *ticket, int *status, cudaStream_t s
#define EP_FILL()                                                                                                     \
  EpArgs a;                                                                                                           \
  if (status == nullptr) return (int)cudaErrorInvalidValue;                                                           \
  {                                                                                                                   \
    int e = ep_fill(a, world, rank, S, k, cap, H, e_local, site, sites, epoch, flags_local, flags_peer, recv_peer,    \
                    meta_peer, count_peer, back_peer, ticket);                                                        \
    if (e) return e;                                                                                                  \
  }

POOT_API int poot_ep_dispatch(const void* x, int ldx, const int* ids, const float* gates, const int* dest, const int* dpos,
                              const int* counts, EP_COMMON_PARAMS) {
  EP_FILL();
  if (ldx % 8) return (int)cudaErrorInvalidValue;
  return launch_k(ep_dispatch_kernel, dim3(S * k), dim3(128), 0, s, (const __nv_bfloat16*)x, ldx, ids, gates, dest, dpos,
                  counts, a, status);
}

POOT_API int poot_ep_mask(const int* meta_local, const int* count_local, int* ids_out, float* gate_out, EP_COMMON_PARAMS) {
  EP_FILL();
  const int n = world * cap;
  return launch_k(ep_mask_kernel, dim3((n + 255) / 256), dim3(256), 0, s, meta_local, count_local, ids_out, gate_out, a, status);
}

POOT_API int poot_ep_gather(const void* recv_local, const int* sorted_rows, const float* gate_flat, const int* n_tiles,
                            int block, int max_tiles, void* xs, float* gate_sorted, EP_COMMON_PARAMS) {
  EP_FILL();
  if (block < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
  return launch_k(ep_gather_kernel, dim3(max_tiles * block), dim3(128), 0, s, (const __nv_bfloat16*)recv_local, sorted_rows,
                  gate_flat, n_tiles, block, H, (__nv_bfloat16*)xs, gate_sorted, a);
}

POOT_API int poot_ep_combine(const void* y, const int* pos, const int* meta_local, EP_COMMON_PARAMS) {
  EP_FILL();
  return launch_k(ep_combine_kernel, dim3(world * cap), dim3(128), 0, s, (const __nv_bfloat16*)y, pos, meta_local, a, status);
}

POOT_API int poot_ep_finish(void* h, const void* back_local, EP_COMMON_PARAMS) {
  EP_FILL();
  return launch_k(ep_finish_kernel, dim3(S), dim3(256), 0, s, (__nv_bfloat16*)h, (const __nv_bfloat16*)back_local, a, status);
}
