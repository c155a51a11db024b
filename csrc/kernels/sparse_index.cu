// Sparse attention indexer (DeepSeek-V3.2 / GLM-MoE-DSA): a light multi-head scorer over its own cached keys ranks the
// visible keys of every query, and only the `topk` best stay visible to the main attention.
//
//   index_k_write   k = LayerNorm(x . Wk) with the rotary on its leading `dr` channels (half-split), written to the
//                   index pool [blocks, 16, Di] at the token's slot
//   index_q_rope    the rotary on the leading `dr` channels of each of the `ni` query heads, in place
//   index_scores    score[r, j] = sum_h w[r, h] * relu(q[r, h] . k[j]) * Di^-0.5 over the row's visible keys j < ctx,
//                   keys read through the row's block table
//   index_select    per row, the `topk` best scores by an exact radix select over the order-preserving key of each
//                   score; the kept positions come out in ascending order, -1 after the last.  Ties at the cut keep
//                   the lowest positions first, which is the stable descending rank the graph states.
//
// The attention over the kept positions is attn_general with its selection list.  These kernels use no tensor cores
// and wait on nothing: the score kernel is the one GEMM-shaped piece (queries x keys x heads x Di) and the candidate
// for a tcgen05 version.
#include "common.cuh"
#include <float.h>

namespace poot {

constexpr int IDX_MAX_D = 256;     // indexer head width
constexpr int IDX_MAX_HEADS = 64;
constexpr int IDX_BLOCK = 16;      // positions per pool block

// One warp per token.  kraw [T, Di] bf16; norm weight / bias [Di] bf16; cos / sin [max_pos, dr / 2] f32.
__global__ void __launch_bounds__(128)
index_k_write_kernel(const __nv_bfloat16* __restrict__ kraw, const __nv_bfloat16* __restrict__ nw,
                     const __nv_bfloat16* __restrict__ nb, float eps, const int* __restrict__ positions,
                     const int* __restrict__ slots, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                     __nv_bfloat16* __restrict__ pool, int T, int Di, int dr, int max_pos) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;
  if (!POOT_IN_RANGE(slot, POOT_LIMIT(kLimPoolSlots), kSiteKvSlot)) return;
  int pos = positions[t];
  POOT_IN_RANGE(pos, max_pos, kSitePosition);
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const __nv_bfloat16* src = kraw + (size_t)t * Di;
  float v[IDX_MAX_D / 32];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < IDX_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    v[i] = d < Di ? __bfloat162float(src[d]) : 0.f;
    sum += v[i];
  }
  const float mean = warp_sum(sum) / (float)Di;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < IDX_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    const float c = d < Di ? v[i] - mean : 0.f;
    var += c * c;
  }
  const float inv = rsqrtf(warp_sum(var) / (float)Di + eps);
  __nv_bfloat16* dst = pool + (size_t)slot * Di;
  // normalised values go through the pool row so the rotary can pair channel j with j + dr / 2 whatever lane holds them
#pragma unroll
  for (int i = 0; i < IDX_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < Di) dst[d] = __float2bfloat16((v[i] - mean) * inv * __bfloat162float(nw[d]) + (nb ? __bfloat162float(nb[d]) : 0.f));
  }
  __syncwarp();
  const int half = dr >> 1;
  const float* cr = cos_t + (size_t)pos * half;
  const float* sr = sin_t + (size_t)pos * half;
  for (int j = lane; j < half; j += 32) {
    const float x1 = __bfloat162float(dst[j]), x2 = __bfloat162float(dst[j + half]);
    dst[j] = __float2bfloat16(x1 * cr[j] - x2 * sr[j]);
    dst[j + half] = __float2bfloat16(x2 * cr[j] + x1 * sr[j]);
  }
}

// One warp per (token, head): q [T, ni * Di] in place.
__global__ void __launch_bounds__(256)
index_q_rope_kernel(__nv_bfloat16* __restrict__ q, const int* __restrict__ positions, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int T, int ni, int Di, int dr, int max_pos) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= T * ni) return;
  const int t = item / ni;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const int half = dr >> 1;
  const float* cr = cos_t + (size_t)pos * half;
  const float* sr = sin_t + (size_t)pos * half;
  __nv_bfloat16* row = q + (size_t)item * Di;
  for (int j = lane; j < half; j += 32) {
    const float x1 = __bfloat162float(row[j]), x2 = __bfloat162float(row[j + half]);
    row[j] = __float2bfloat16(x1 * cr[j] - x2 * sr[j]);
    row[j + half] = __float2bfloat16(x2 * cr[j] + x1 * sr[j]);
  }
}

// grid (rows, key chunks of IDX_KEYS_PER_CTA); 4 warps.  The row's query heads sit in shared memory (rows padded by two
// elements so lanes that own different heads hit different banks); each warp takes keys one at a time, stages the key in
// its own shared row, and every lane accumulates the heads it owns (lane, lane + 32) over the whole key.
constexpr int IDX_KEYS_PER_CTA = 256;

__global__ void __launch_bounds__(128)
index_scores_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ w, int ldw,
                    const __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ row_seq, const int* __restrict__ row_ctx, float* __restrict__ scores,
                    int ld_scores, int ni, int Di, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_wait(); pdl_launch();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = row_ctx[r];
  const int j0 = blockIdx.y * IDX_KEYS_PER_CTA;
  if (ctx <= 0 || j0 >= ctx) return;
  const int ldq = Di + 2;
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [ni][ldq]
  float* sk = reinterpret_cast<float*>(smem_raw + (((size_t)ni * ldq * 2 + 15) / 16) * 16);   // [4][Di]
  const __nv_bfloat16* qrow = q + (size_t)r * ni * Di;
  for (int i = threadIdx.x; i < ni * Di; i += blockDim.x) sq[(i / Di) * ldq + (i % Di)] = qrow[i];
  __syncthreads();
  const int seq = row_seq ? row_seq[r] : r;
  const int* bt = block_tables + (size_t)seq * max_blocks;
  float wh[2];
  wh[0] = lane < ni ? w[(size_t)r * ldw + lane] : 0.f;
  wh[1] = lane + 32 < ni ? w[(size_t)r * ldw + lane + 32] : 0.f;
  float* kw = sk + (size_t)warp * Di;
  const int j1 = min(ctx, j0 + IDX_KEYS_PER_CTA);
  for (int j = j0 + warp; j < j1; j += 4) {
    int blk = bt[j >> 4];
    if (!POOT_IN_RANGE(j >> 4, max_blocks, kSitePosition) || !POOT_IN_RANGE(blk, POOT_LIMIT(kLimPoolBlocks), kSiteBlockId)) blk = 0;
    const __nv_bfloat16* kr = pool + ((size_t)blk * IDX_BLOCK + (j & 15)) * Di;
    for (int d = lane; d < Di; d += 32) kw[d] = __bfloat162float(kr[d]);
    __syncwarp();
    float acc = 0.f;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int h = lane + 32 * x;
      if (h < ni) {
        const __nv_bfloat16* qh = sq + (size_t)h * ldq;
        float dot = 0.f;
        for (int d = 0; d < Di; ++d) dot += __bfloat162float(qh[d]) * kw[d];
        acc += wh[x] * fmaxf(dot * scale, 0.f);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) scores[(size_t)r * ld_scores + j] = acc;
    __syncwarp();
  }
}

// Order-preserving 32-bit key of a score: NaN and -inf are the lowest key, -0.0 is +0.0.
__device__ __forceinline__ uint32_t score_key(float s) {
  if (!(s == s) || s == -INFINITY) s = -FLT_MAX;
  if (s == INFINITY) s = FLT_MAX;
  if (s == 0.f) s = 0.f;
  const uint32_t u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA of 256 threads per row.  sel [rows, topk]: kept positions ascending, -1 after the last kept.
__global__ void __launch_bounds__(256)
index_select_kernel(const float* __restrict__ scores, int ld_scores, const int* __restrict__ row_ctx, int* __restrict__ sel,
                    int topk) {
  __shared__ unsigned int hist[256];
  __shared__ unsigned int s_prefix, s_need;
  __shared__ int scan_gt[256], scan_eq[256];
  pdl_wait(); pdl_launch();
  const int r = blockIdx.x, tid = threadIdx.x;
  const int n = max(row_ctx[r], 0);
  int* out = sel + (size_t)r * topk;
  const float* sc = scores + (size_t)r * ld_scores;
  if (n <= topk) {                      // everything visible is kept
    for (int i = tid; i < topk; i += 256) out[i] = i < n ? i : -1;
    return;
  }
  // radix select, most significant byte first: after pass p the top (p + 1) bytes of the cut key are known
  unsigned int prefix = 0, need = (unsigned int)topk;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    hist[tid] = 0;
    __syncthreads();
    const unsigned int mask_hi = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < n; i += 256) {
      const uint32_t k = score_key(sc[i]);
      if ((k & mask_hi) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int run = 0, digit = 0, left = need;
      for (int d = 255; d >= 0; --d) {
        if (run + hist[d] >= need) { digit = (unsigned int)d; left = need - run; break; }
        run += hist[d];
      }
      s_prefix = prefix | (digit << shift);
      s_need = left;
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    __syncthreads();
  }
  // prefix = the key of the topk-th largest score; need = how many positions equal to it are kept (lowest first)
  const int chunk = (n + 255) / 256;
  const int a = min(n, tid * chunk), b = min(n, a + chunk);
  int gt = 0, eq = 0;
  for (int i = a; i < b; ++i) {
    const uint32_t k = score_key(sc[i]);
    gt += k > prefix;
    eq += k == prefix;
  }
  scan_gt[tid] = gt;
  scan_eq[tid] = eq;
  __syncthreads();
  if (tid == 0) {                        // 256 entries: a serial exclusive scan is a few hundred cycles
    int g = 0, e = 0;
    for (int i = 0; i < 256; ++i) {
      const int tg = scan_gt[i], te = scan_eq[i];
      scan_gt[i] = g;
      scan_eq[i] = e;
      g += tg;
      e += te;
    }
  }
  __syncthreads();
  int eq_before = scan_eq[tid];
  int at = scan_gt[tid] + min(eq_before, (int)need);
  for (int i = a; i < b; ++i) {
    const uint32_t k = score_key(sc[i]);
    bool keep = k > prefix;
    if (k == prefix) { keep = eq_before < (int)need; ++eq_before; }
    if (keep && at < topk) out[at++] = i;
  }
}

}  // namespace poot

using namespace poot;

POOT_API int poot_index_k_write(const void* kraw, const void* norm_w, const void* norm_b, float eps, const int* positions,
                                const int* slots, const float* cos_t, const float* sin_t, void* pool, int T, int Di, int dr,
                                int max_pos, cudaStream_t s) {
  if (T == 0) return 0;
  if (Di < 2 || Di > IDX_MAX_D || dr < 0 || dr > Di || (dr & 1)) return (int)cudaErrorInvalidValue;
  return launch_k(index_k_write_kernel, dim3((T + 3) / 4), dim3(128), 0, s, (const __nv_bfloat16*)kraw,
                  (const __nv_bfloat16*)norm_w, (const __nv_bfloat16*)norm_b, eps, positions, slots, cos_t, sin_t,
                  (__nv_bfloat16*)pool, T, Di, dr, max_pos);
}

POOT_API int poot_index_q_rope(void* q, const int* positions, const float* cos_t, const float* sin_t, int T, int ni, int Di,
                               int dr, int max_pos, cudaStream_t s) {
  if (T == 0 || dr == 0) return 0;
  if (Di < 2 || dr > Di || (dr & 1) || ni < 1) return (int)cudaErrorInvalidValue;
  const int items = T * ni;
  return launch_k(index_q_rope_kernel, dim3((items + 7) / 8), dim3(256), 0, s, (__nv_bfloat16*)q, positions, cos_t, sin_t, T,
                  ni, Di, dr, max_pos);
}

POOT_API int poot_index_scores(const void* q, const float* w, int ldw, const void* pool, const int* block_tables,
                               int max_blocks, const int* row_seq, const int* row_ctx, float* scores, int ld_scores, int R,
                               int ni, int Di, int max_ctx, float scale, cudaStream_t s) {
  if (R == 0 || max_ctx <= 0) return 0;
  if (ni < 1 || ni > IDX_MAX_HEADS || Di < 1 || Di > IDX_MAX_D || ld_scores < max_ctx) return (int)cudaErrorInvalidValue;
  const size_t smem = (((size_t)ni * (Di + 2) * 2 + 15) / 16) * 16 + (size_t)4 * Di * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(index_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_k(index_scores_kernel, dim3(R, (max_ctx + IDX_KEYS_PER_CTA - 1) / IDX_KEYS_PER_CTA), dim3(128), smem, s,
                  (const __nv_bfloat16*)q, w, ldw, (const __nv_bfloat16*)pool, block_tables, max_blocks, row_seq, row_ctx,
                  scores, ld_scores, ni, Di, scale);
}

POOT_API int poot_index_select(const float* scores, int ld_scores, const int* row_ctx, int* sel, int R, int topk,
                               cudaStream_t s) {
  if (R == 0) return 0;
  if (topk < 1) return (int)cudaErrorInvalidValue;
  return launch_k(index_select_kernel, dim3(R), dim3(256), 0, s, scores, ld_scores, row_ctx, sel, topk);
}
