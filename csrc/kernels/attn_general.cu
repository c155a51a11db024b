// General paged attention: any head widths (query / key width Dk and value width Dv, multiples of 32 up to 512, which need
// not be equal), causal window, score soft cap, per-head ALiBi slopes, per-head sink logits.  It serves the shapes the
// tuned kernels do not (head_dim 256, split key / value widths): one CTA of four warps per (query row, head); the warps
// take every fourth key and keep online-softmax partials that are merged through shared memory.  Correctness path, not
// a fast one: no split over the keys across CTAs, no tensor cores.  With a selection list (the output of the sparse
// attention indexer) a row attends to the listed key positions only.
//
// K / V pools are [blocks, kv heads, 16, pool_d]; a row holds the key (Dk used) or the value (Dv used).
#include "common.cuh"
#include <float.h>

namespace poot {

constexpr int AG_WARPS = 4;
constexpr int AG_MAXD = 512;

__global__ void __launch_bounds__(AG_WARPS * 32)
attn_general_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ kpool,
                    const __nv_bfloat16* __restrict__ vpool, int pool_d, const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ row_seq, const int* __restrict__ row_ctx, __nv_bfloat16* __restrict__ out,
                    int out_stride, int Hq, int Hkv, int Dk, int Dv, float scale, float softcap, int window,
                    const float* __restrict__ alibi, const float* __restrict__ sinks, const int* __restrict__ sel, int sel_k) {
  __shared__ float sm_m[AG_WARPS], sm_l[AG_WARPS];
  __shared__ float sm_o[AG_WARPS][AG_MAXD];
  pdl_wait(); pdl_launch();
  const int r = blockIdx.x, h = blockIdx.y, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = row_ctx[r];
  if (ctx <= 0) return;                                   // a padding row, or a row another kernel covers
  const int seq = row_seq ? row_seq[r] : r;
  const int kvh = h / (Hq / Hkv);
  const int first = (window > 0 && ctx > window) ? ctx - window : 0;
  const int nk = Dk >> 5, nv = Dv >> 5;                   // elements per lane
  float qr[AG_MAXD / 32], o[AG_MAXD / 32];
  const __nv_bfloat16* qrow = q + (size_t)r * q_stride + (size_t)h * Dk;
#pragma unroll
  for (int i = 0; i < AG_MAXD / 32; ++i) {
    qr[i] = i < nk ? __bfloat162float(qrow[lane + 32 * i]) : 0.f;
    o[i] = 0.f;
  }
  const float slope = alibi ? alibi[h] : 0.f;
  float m = -FLT_MAX, l = 0.f;
  // with a selection list the row attends to the listed positions only (ascending, -1 after the last kept)
  const int n_iter = sel ? sel_k : ctx - first;
  for (int it = w; it < n_iter; it += AG_WARPS) {
    const int j = sel ? sel[(size_t)r * sel_k + it] : first + it;
    if (j < 0 || j >= ctx) continue;
    int blk = block_tables[(size_t)seq * max_blocks + (j >> 4)];
    if (!POOT_IN_RANGE(j >> 4, max_blocks, kSitePosition) || !POOT_IN_RANGE(blk, POOT_LIMIT(kLimPoolBlocks), kSiteBlockId)) blk = 0;
    const size_t base = (((size_t)blk * Hkv + kvh) * 16 + (j & 15)) * pool_d;
    const __nv_bfloat16* kr = kpool + base;
    const __nv_bfloat16* vr = vpool + base;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < AG_MAXD / 32; ++i)
      if (i < nk) s += qr[i] * __bfloat162float(kr[lane + 32 * i]);
    s = warp_sum(s) * scale;
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    s += slope * (float)(j - (ctx - 1));
    const float mn = fmaxf(m, s);
    const float corr = __expf(m - mn), p = __expf(s - mn);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < AG_MAXD / 32; ++i)
      if (i < nv) o[i] = o[i] * corr + p * __bfloat162float(vr[lane + 32 * i]);
    m = mn;
  }
  if (lane == 0) { sm_m[w] = m; sm_l[w] = l; }
#pragma unroll
  for (int i = 0; i < AG_MAXD / 32; ++i)
    if (i < nv) sm_o[w][lane + 32 * i] = o[i];
  __syncthreads();
  if (w != 0) return;
  float M = sinks ? sinks[h] : -FLT_MAX;
  for (int x = 0; x < AG_WARPS; ++x) M = fmaxf(M, sm_m[x]);
  float L = sinks ? __expf(sinks[h] - M) : 0.f;           // the sink joins the denominator and carries no value
  float f[AG_WARPS];
  for (int x = 0; x < AG_WARPS; ++x) {
    f[x] = sm_l[x] > 0.f ? __expf(sm_m[x] - M) : 0.f;
    L += sm_l[x] * f[x];
  }
  __nv_bfloat16* orow = out + (size_t)r * out_stride + (size_t)h * Dv;
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int i = 0; i < nv; ++i) {
    float acc = 0.f;
    for (int x = 0; x < AG_WARPS; ++x) acc += sm_o[x][lane + 32 * i] * f[x];
    orow[lane + 32 * i] = __float2bfloat16(acc * inv);
  }
}

}  // namespace poot

using namespace poot;

POOT_API int poot_attn_general(const void* q, int q_stride, const void* kpool, const void* vpool, int pool_d,
                               const int* block_tables, int max_blocks, const int* row_seq, const int* row_ctx, void* out,
                               int out_stride, int R, int Hq, int Hkv, int Dk, int Dv, float scale, float softcap, int window,
                               const float* alibi, const float* sinks, const int* sel, int sel_k, cudaStream_t s) {
  if (R == 0) return 0;
  if (Dk % 32 || Dv % 32 || Dk < 32 || Dv < 32 || Dk > AG_MAXD || Dv > AG_MAXD || pool_d < Dk || pool_d < Dv || Hkv < 1 || Hq % Hkv)
    return (int)cudaErrorInvalidValue;
  if (sel != nullptr && sel_k < 1) return (int)cudaErrorInvalidValue;
  return launch_k(attn_general_kernel, dim3(R, Hq), dim3(AG_WARPS * 32), 0, s, (const __nv_bfloat16*)q, q_stride,
                  (const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, pool_d, block_tables, max_blocks, row_seq, row_ctx,
                  (__nv_bfloat16*)out, out_stride, Hq, Hkv, Dk, Dv, scale, softcap, window, alibi, sinks, sel, sel_k);
}
