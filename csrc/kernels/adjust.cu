// Sampler-suffix helpers on the device: sparse logit adjustments and the log-probability record.
//
// adjust: for each row a short list of (token, bias, mul_pos, mul_neg, add) entries applied in the reference's order
//   +bias, repetition (divide if > 0 else multiply), -presence, -frequency*count
// folded per token as  l += bias; l = (l > 0 ? l * mul_pos : l * mul_neg) + add, followed by an optional dense additive
// guided-decoding mask (0 for an allowed token, f32::MIN for an excluded one)
// (crates/poot-graph-ir/src/ops/sampling.rs:365-440).
// logprob: log softmax of the picked token, log p = l[tok] - max - ln(sum exp(l - max)).
#include "common.cuh"
#include <float.h>

namespace poot {

__global__ void adjust_logits_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ idx,
                                     const float* __restrict__ val, int max_adj, const float* __restrict__ guided) {
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x;
  float* lr = logits + (size_t)row * vocab;
  // entries of a row name distinct tokens, so the sparse pass has no write conflicts
  for (int i = threadIdx.x; i < max_adj; i += blockDim.x) {
    const int t = idx[(size_t)row * max_adj + i];
    if (t >= 0) POOT_IN_RANGE(t, vocab, kSiteLogitIndex);      // a negative id ends the row's list
    if (t < 0 || t >= vocab) continue;
    const float* v = val + ((size_t)row * max_adj + i) * 4;
    float l = lr[t] + v[0];
    l = (l > 0.f ? l * v[1] : l * v[2]) + v[3];
    lr[t] = l;
  }
  if (guided != nullptr) {
    __syncthreads();
    const float* g = guided + (size_t)row * vocab;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
      const float m = g[j];
      if (m != 0.f) lr[j] = (m <= -FLT_MAX) ? -FLT_MAX : lr[j] + m;
    }
  }
}

__global__ void token_logprob_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ picked,
                                     float* __restrict__ out) {
  __shared__ float red[32];
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * vocab;
  float mx = -FLT_MAX;
  for (int j = threadIdx.x; j < vocab; j += blockDim.x) mx = fmaxf(mx, lr[j]);
  mx = warp_max(mx);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = mx;
  __syncthreads();
  mx = warp_max(l < (blockDim.x >> 5) ? red[l] : -FLT_MAX);
  __syncthreads();
  float s = 0.f;
  for (int j = threadIdx.x; j < vocab; j += blockDim.x) s += __expf(lr[j] - mx);
  s = warp_sum(s);
  if (l == 0) red[w] = s;
  __syncthreads();
  s = warp_sum(l < (blockDim.x >> 5) ? red[l] : 0.f);
  if (threadIdx.x == 0) {
    const int t = picked[row * 2];
    POOT_IN_RANGE(t, vocab, kSiteTokenId);
    out[row] = (t >= 0 && t < vocab) ? lr[t] - mx - logf(s) : 0.f;
  }
}

}  // namespace poot

using namespace poot;

POOT_API int poot_adjust_logits(float* logits, int rows, int vocab, const int* idx, const float* val, int max_adj,
                                const float* guided, cudaStream_t s) {
  if (rows == 0) return 0;
  return launch_k(adjust_logits_kernel, dim3(rows), dim3(256), 0, s, logits, vocab, idx, val, max_adj, guided);
}

POOT_API int poot_token_logprob(const float* logits, int rows, int vocab, const int* picked, float* out, cudaStream_t s) {
  if (rows == 0) return 0;
  return launch_k(token_logprob_kernel, dim3(rows), dim3(512), 0, s, logits, vocab, picked, out);
}
