// Mixture-of-experts routing and combine.
//
//  * moe_route: per token, canonical router scores (NaN / -inf -> f32::MIN, +inf -> f32::MAX), stable descending
//    top-k (ties go to the lower expert index), gate weights by softmax over the selected k (Mixtral) or softmax over
//    all experts without renormalisation; writes ids [T,k], gates [T,k] and the dense gate matrix [E,T] (0 for an
//    unselected expert) that the grouped expert GEMM applies per row
//    (crates/poot-graph-ir/src/ops/moe.rs:9-431, router kinds crates/poot-models/src/components/router.rs).
//  * moe_combine: h[t] += sum over groups of the (already gate-scaled) expert outputs.
//  * moe_align / moe_gather_rows / moe_scatter_combine: row grouping by expert.  The (token, slot) rows routed to
//    one expert are made contiguous and every expert's run is padded to a whole row tile, so a grouped GEMM walks
//    tiles that each belong to exactly one expert and every expert multiplies only its own rows at any token count
//    (the reference's group_expert_rows pass and grouped indexed contraction:
//    crates/poot-graph-plan/src/passes/group_expert_rows.rs:1-8, crates/poot-kernelgen/src/contraction/indexed.rs:1-6).
//    With an expert-parallel shard (experts [e0, e0 + e_local) on this rank) rows routed elsewhere are left out.
#include "common.cuh"
#include "tp_common.cuh"
#include <float.h>

namespace poot {

constexpr int MOE_MAX_K = 16;
constexpr int MOE_MAX_GROUPS = 32;

// mode 0: softmax gates (over the k selected logits when renorm, else over all experts, not renormalised).
// mode 1: sigmoid scores; experts are ranked by score + select_bias[e] (the bias does not enter the gate), gates are
//         the selected scores, divided by their sum (+1e-20) when renorm.  Both: gates are multiplied by `scale`.
__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int k, int renorm, int mode,
                                 const float* __restrict__ select_bias, float scale, int n_group, int topk_group,
                                 int* __restrict__ ids, float* __restrict__ gates, float* __restrict__ dense) {
  pdl_wait(); pdl_launch();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* lr = logits + (size_t)t * E;
  // Group-limited routing (mode 1): experts form n_group groups; a group's score is the sum of its two best selection
  // values; only the topk_group best groups (lower index first on ties) stay eligible, the others rank as 0.
  unsigned keep_groups = 0xffffffffu;
  const int per = n_group > 1 ? E / n_group : E;
  if (n_group > 1) {
    float gs[MOE_MAX_GROUPS];
    for (int g = 0; g < n_group; ++g) {
      float b1 = -FLT_MAX, b2 = -FLT_MAX;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        float s = lr[e];
        if (!(s >= -FLT_MAX)) s = -FLT_MAX;
        if (s > FLT_MAX) s = FLT_MAX;
        const float v = 1.f / (1.f + expf(-s)) + (select_bias ? select_bias[e] : 0.f);
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      gs[g] = b1 + b2;
    }
    keep_groups = 0u;
    for (int n = 0; n < topk_group; ++n) {
      int bg = -1; float bvv = -FLT_MAX;
      for (int g = 0; g < n_group; ++g)
        if (!((keep_groups >> g) & 1u) && (bg < 0 || gs[g] > bvv)) { bg = g; bvv = gs[g]; }
      if (bg >= 0) keep_groups |= 1u << bg;
    }
  }
  int best[MOE_MAX_K];
  float bv[MOE_MAX_K];      // the value experts are ranked by
  float sv[MOE_MAX_K];      // the score that becomes the gate (mode 1)
  for (int j = 0; j < k; ++j) { best[j] = -1; bv[j] = -FLT_MAX; sv[j] = 0.f; }
  float all_max = -FLT_MAX;
  for (int e = 0; e < E; ++e) {
    float s = lr[e];
    if (!(s >= -FLT_MAX)) s = -FLT_MAX;      // NaN and -inf
    if (s > FLT_MAX) s = FLT_MAX;
    all_max = fmaxf(all_max, s);
    float score = s, rankv = s;
    if (mode == 1) {
      score = 1.f / (1.f + expf(-s));
      rankv = score + (select_bias ? select_bias[e] : 0.f);
      if (n_group > 1 && !((keep_groups >> (e / per)) & 1u)) rankv = 0.f;
    }
    // insertion into the sorted top-k; strict '>' keeps the lower index first on ties
    int pos = k;
    for (int j = k - 1; j >= 0; --j) if (best[j] < 0 || rankv > bv[j]) pos = j;
    if (pos < k) {
      for (int j = k - 1; j > pos; --j) { best[j] = best[j - 1]; bv[j] = bv[j - 1]; sv[j] = sv[j - 1]; }
      best[pos] = e; bv[pos] = rankv; sv[pos] = score;
    }
  }
  float w[MOE_MAX_K], sum = 0.f;
  if (mode == 1) {
    for (int j = 0; j < k; ++j) { w[j] = sv[j]; sum += sv[j]; }
    sum = renorm ? sum + 1e-20f : 1.f;
  } else if (renorm) {
    for (int j = 0; j < k; ++j) { w[j] = expf(bv[j] - bv[0]); sum += w[j]; }
  } else {
    for (int e = 0; e < E; ++e) {
      float s = lr[e];
      if (!(s >= -FLT_MAX)) s = -FLT_MAX;
      if (s > FLT_MAX) s = FLT_MAX;
      sum += expf(s - all_max);
    }
    for (int j = 0; j < k; ++j) w[j] = expf(bv[j] - all_max);
  }
  for (int e = 0; e < E; ++e) dense[(size_t)e * T + t] = 0.f;
  for (int j = 0; j < k; ++j) {
    const float g = w[j] / sum * scale;
    ids[(size_t)t * k + j] = best[j];
    gates[(size_t)t * k + j] = g;
    if (best[j] >= 0) dense[(size_t)best[j] * T + t] = g;
  }
}

// out[t, :] = (h ? h[t, :] : 0) + sum_{j < n} parts[(g0(t) + j) * gstride + row(t) * H + :]
//   dense form (per_token == 0): g0 = 0, row = t, n = groups         parts [groups, T, H]
//   slot form  (per_token  > 0): g0 = t * per_token, row = 0, n = per_token   parts [T * per_token, 1, H]
__global__ void moe_combine_kernel(const __nv_bfloat16* h, const __nv_bfloat16* __restrict__ parts,
                                   __nv_bfloat16* out, int T, int H, int groups, long long gstride, int per_token) {
  pdl_wait(); pdl_launch();
  const int t = blockIdx.x;
  const int n = per_token > 0 ? per_token : groups;
  const int g0 = per_token > 0 ? t * per_token : 0;
  const size_t row_off = per_token > 0 ? 0 : (size_t)t * H;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8];
    if (h != nullptr) unpack8(reinterpret_cast<const uint4*>(h + (size_t)t * H)[c], acc);
    else { for (int i = 0; i < 8; ++i) acc[i] = 0.f; }
    for (int j = 0; j < n; ++j) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(parts + (size_t)(g0 + j) * gstride + row_off)[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = pack8(acc);
  }
}

// Block-aligned grouping of (token, slot) rows by expert.  One CTA.
//   ids [n]            expert of every flat row (token * k + slot); ids outside [e0, e0 + e_local) are skipped
//   pos [n]            out: position of the row in the grouped order, -1 when skipped
//   sorted_rows [cap]  out: flat row at each grouped position, -1 for padding (cap = max_tiles * block)
//   tile_expert [max_tiles]  out: local expert of each row tile, -1 for tiles beyond the last used one
//   n_tiles            out: tiles in use
// The order of rows inside one expert's run follows the arrival of the atomics; every row's result is independent
// of its position inside the tile, so the step's output does not depend on that order.
constexpr int MOE_ALIGN_THREADS = 1024;
constexpr int MOE_ALIGN_MAX_E = 1024;

__global__ void __launch_bounds__(MOE_ALIGN_THREADS)
moe_align_kernel(const int* __restrict__ ids, int n, int e0, int e_local, int block, int max_tiles,
                 int* __restrict__ pos, int* __restrict__ sorted_rows, int* __restrict__ tile_expert,
                 int* __restrict__ n_tiles) {
  __shared__ int counts[MOE_ALIGN_MAX_E];
  __shared__ int starts[MOE_ALIGN_MAX_E];
  __shared__ int cursor[MOE_ALIGN_MAX_E];
  __shared__ int s_tiles;
  pdl_wait(); pdl_launch();
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i] - e0;
    if (e >= 0 && e < e_local) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < e_local; ++e) {
      starts[e] = tiles * block;
      int t = (counts[e] + block - 1) / block;
      if (tiles + t > max_tiles) t = max_tiles - tiles;   // cannot happen when max_tiles >= ceil(n / block) + e_local
      for (int j = 0; j < t; ++j) tile_expert[tiles + j] = e;
      tiles += t;
    }
    for (int j = tiles; j < max_tiles; ++j) tile_expert[j] = -1;
    s_tiles = tiles;
    *n_tiles = tiles;
  }
  for (int p = threadIdx.x; p < max_tiles * block; p += blockDim.x) sorted_rows[p] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i] - e0;
    int p = -1;
    if (e >= 0 && e < e_local) {
      const int slot = atomicAdd(&cursor[e], 1);
      p = starts[e] + slot;
      if (p < s_tiles * block) sorted_rows[p] = i; else p = -1;
    }
    pos[i] = p;
  }
}

// xs[p, :] = x[sorted_rows[p] / k, :] (zeros for padding rows), gate_sorted[p] = gates[sorted_rows[p]] (0 for padding).
// One CTA per grouped row; rows of tiles that are not in use are left alone.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ sorted_rows,
                                       const float* __restrict__ gates, const int* __restrict__ n_tiles, int block, int k,
                                       int H, __nv_bfloat16* __restrict__ xs, float* __restrict__ gate_sorted) {
  pdl_wait(); pdl_launch();
  const int p = blockIdx.x;
  if (p >= *n_tiles * block) return;
  const int i = sorted_rows[p];
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * H);
  if (i < 0) {
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x == 0) gate_sorted[p] = 0.f;
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * ldx);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = src[c];
  if (threadIdx.x == 0) gate_sorted[p] = gates[i];
}

// out[t, :] = (h ? h[t, :] : 0) + sum over the token's k slots of y[pos[t * k + j], :] (slots with pos < 0 are other
// ranks' experts).  y rows are already gate-scaled by the down projection's epilogue.  Slots add in slot order.
__global__ void moe_scatter_combine_kernel(const __nv_bfloat16* h, const __nv_bfloat16* __restrict__ y,
                                           const int* __restrict__ pos, __nv_bfloat16* out, int T, int H, int k) {
  pdl_wait(); pdl_launch();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8];
    if (h != nullptr) unpack8(reinterpret_cast<const uint4*>(h + (size_t)t * H)[c], acc);
    else { for (int i = 0; i < 8; ++i) acc[i] = 0.f; }
    for (int j = 0; j < k; ++j) {
      const int p = pos[(size_t)t * k + j];
      if (p < 0) continue;
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(y + (size_t)p * H)[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = pack8(acc);
  }
}

// Expert-parallel combine for decode-sized steps, fused with the one-shot all-reduce: this rank's share of every token
// (the gate-scaled outputs of its own experts, summed in slot order; zero for a token none of them serves) is written
// straight into every rank's inbox slot for this rank, then the reduce-scatter channel is signalled.  The consumer is
// the same reduce + norm kernel that follows a row-parallel GEMM.  One CTA per token row; every CTA signals.
__global__ void moe_scatter_combine_push_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, int T, int H,
                                                int k, TpArgs tp, int* status) {
  pdl_wait(); pdl_launch();
  const int t = blockIdx.x;
  const uint32_t target = tp_target(tp, tp.rs_site, tp.rs_sites);
  const int parity = (int)(target & 1u);
  const size_t row = ((size_t)((parity * tp.world + tp.rank) * tp.S + t)) * tp.ld_inbox;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int p = pos[(size_t)t * k + j];
      if (p < 0) continue;
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(y + (size_t)p * H)[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    const uint4 pk = pack8(acc);
    for (int d = 0; d < tp.world; ++d) *reinterpret_cast<uint4*>(tp.inbox_peer[d] + row + (size_t)c * 8) = pk;
  }
  tp_signal_all(tp, TP_CH_RS, target, gridDim.x, status);
}

}  // namespace poot

using namespace poot;

// Row grouping: see moe_align_kernel.  max_tiles must be at least ceil(n / block) + e_local.
POOT_API int poot_moe_align(const int* ids, int n, int e0, int e_local, int block, int max_tiles, int* pos,
                            int* sorted_rows, int* tile_expert, int* n_tiles, cudaStream_t s) {
  if (n < 0 || e_local < 1 || e_local > MOE_ALIGN_MAX_E || block < 1 || max_tiles < 1) return (int)cudaErrorInvalidValue;
  if ((long long)max_tiles < ((long long)n + block - 1) / block + e_local) return (int)cudaErrorInvalidValue;
  return launch_k(moe_align_kernel, dim3(1), dim3(MOE_ALIGN_THREADS), 0, s, ids, n, e0, e_local, block, max_tiles, pos,
                  sorted_rows, tile_expert, n_tiles);
}

POOT_API int poot_moe_gather_rows(const void* x, int ldx, const int* sorted_rows, const float* gates, const int* n_tiles,
                                  int block, int max_tiles, int k, int H, void* xs, float* gate_sorted, cudaStream_t s) {
  if (H % 8 || ldx % 8 || k < 1) return (int)cudaErrorInvalidValue;
  return launch_k(moe_gather_rows_kernel, dim3(max_tiles * block), dim3(128), 0, s, (const __nv_bfloat16*)x, ldx,
                  sorted_rows, gates, n_tiles, block, k, H, (__nv_bfloat16*)xs, gate_sorted);
}

POOT_API int poot_moe_scatter_combine(const void* h, const void* y, const int* pos, void* out, int T, int H, int k,
                                      cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8 || k < 1) return (int)cudaErrorInvalidValue;
  return launch_k(moe_scatter_combine_kernel, dim3(T), dim3(256), 0, s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)y,
                  pos, (__nv_bfloat16*)out, T, H, k);
}

POOT_API int poot_moe_route(const float* logits, int T, int E, int k, int renorm, int* ids, float* gates, float* dense,
                            cudaStream_t s) {
  if (T == 0) return 0;
  if (k < 1 || k > MOE_MAX_K || k > E) return (int)cudaErrorInvalidValue;
  return launch_k(moe_route_kernel, dim3((T + 63) / 64), dim3(64), 0, s, logits, T, E, k, renorm, 0,
                  (const float*)nullptr, 1.f, 1, 1, ids, gates, dense);
}

// Router variants: mode 1 = sigmoid scores with an optional selection-only bias [E]; gates times `scale`.
POOT_API int poot_moe_route_ex(const float* logits, int T, int E, int k, int renorm, int mode, const float* select_bias,
                               float scale, int n_group, int topk_group, int* ids, float* gates, float* dense, cudaStream_t s) {
  if (T == 0) return 0;
  if (k < 1 || k > MOE_MAX_K || k > E || mode < 0 || mode > 1) return (int)cudaErrorInvalidValue;
  if (mode == 0 && (select_bias != nullptr || n_group > 1)) return (int)cudaErrorInvalidValue;
  if (n_group < 1 || n_group > MOE_MAX_GROUPS || E % n_group || topk_group < 1 || topk_group > n_group ||
      (n_group > 1 && E / n_group < 2))
    return (int)cudaErrorInvalidValue;
  return launch_k(moe_route_kernel, dim3((T + 63) / 64), dim3(64), 0, s, logits, T, E, k, renorm, mode, select_bias, scale,
                  n_group, topk_group, ids, gates, dense);
}

POOT_API int poot_moe_combine(const void* h, const void* parts, void* out, int T, int H, int groups, long long gstride,
                              int per_token, cudaStream_t s) {
  if (T == 0) return 0;
  if (H % 8) return (int)cudaErrorInvalidValue;
  return launch_k(moe_combine_kernel, dim3(T), dim3(256), 0, s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)parts,
                  (__nv_bfloat16*)out, T, H, groups, gstride, per_token);
}

// Combine + one-shot push (see moe_scatter_combine_push_kernel).  slot_rows: rows of one inbox slot; T <= slot_rows.
POOT_API int poot_moe_scatter_combine_push(const void* y, const int* pos, int T, int H, int k, int tp_world, int tp_rank,
                                           int slot_rows, int rs_site, int rs_sites, const int* epoch, void* flags_local,
                                           void* const* flags_peer, void* const* inbox_peer, int ld_inbox, int* ticket,
                                           int* status, cudaStream_t s) {
  if (T <= 0) return (int)cudaErrorInvalidValue;      // every rank must signal: an empty step has no push to skip
  if (H % 8 || ld_inbox % 8 || ld_inbox < H || k < 1 || T > slot_rows) return (int)cudaErrorInvalidValue;
  if (tp_world < 2 || tp_world > TP_MAX_WORLD || tp_rank < 0 || tp_rank >= tp_world || rs_site < 0 || status == nullptr)
    return (int)cudaErrorInvalidValue;
  TpArgs tp = {};
  tp.world = tp_world; tp.rank = tp_rank; tp.S = slot_rows; tp.oneshot = 1; tp.ag_site = -1; tp.rs_site = rs_site;
  tp.rs_sites = rs_sites; tp.ld_inbox = ld_inbox; tp.epoch = epoch; tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
  for (int r = 0; r < tp_world; ++r) {
    tp.flags_peer[r] = (uint32_t*)flags_peer[r];
    tp.inbox_peer[r] = (__nv_bfloat16*)inbox_peer[r];
  }
  return launch_k(moe_scatter_combine_push_kernel, dim3(T), dim3(256), 0, s, (const __nv_bfloat16*)y, pos, T, H, k, tp, status);
}
