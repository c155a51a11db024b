// On-device token sampling: two-stage greedy argmax and the Gumbel-max family
// (temperature + min-p, + top-k value bisection, + top-p integer-mass bisection).
// Output per row is (token, non_finite_index): token is forced to 0 and the index of
// the first non-finite logit is reported when any logit is NaN/Inf; otherwise -1.
//
// The rules are bit-compatible with the CPU oracle: maximum of
//   logit*inv_temp + noise_scale*noise   (two roundings, no FMA; first index wins ties)
// over the kept set  logit >= floor,  floor = max(t_k, max+floor_offset, t_p), with
// t_k from a 30-step bisection on the count of logits >= mid and t_p from a 30-step
// bisection over exact integer masses round(exp((l-max)*inv_temp)*2^24).
// Noise is Gumbel(-ln(-ln u)) of u = (2*(fmix32(seed ^ idx*0x9E3779B9)>>9)+1)*2^-24.
//
// Reference behaviour covered: crates/pootc/kernels/sampling/{argmax_chunk,argmax_combine,
// random_uniform,sample_gumbel_argmax_batched,sample_truncated_gumbel_argmax_batched,
// sample_topp_gumbel_argmax_batched}.rs and crates/poot-eval/src/ops/sampling.rs:40-183.
#include "common.cuh"
#include "argmax_common.cuh"
#include <float.h>

namespace poot {

__device__ __forceinline__ bool finite_f32(float v) { return v >= -FLT_MAX && v <= FLT_MAX; }

__device__ __forceinline__ uint32_t fmix32(uint32_t x) {
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform_at(uint32_t seed, uint32_t idx) {
  uint32_t x = fmix32(seed ^ (idx * 0x9E3779B9u));
  int mant = (int)(x >> 9);
  return __fmul_rn(__fadd_rn(__fmul_rn(2.0f, (float)mant), 1.0f), 5.9604645e-8f);
}

constexpr int SAMP_THREADS = 256;

// Stage 1: part[(row*groups+g)*3 ..] = (bits of best_val, best_idx, bad_idx) over one chunk of a row of
// `vocab` logits (row pitch ld).  Indices are global: idx_offset is added (vocabulary-sharded logits), and
// `bad_none` (the total vocabulary) stands for "no non-finite logit".
__global__ void __launch_bounds__(SAMP_THREADS)
argmax_chunk_kernel(const float* __restrict__ logits, int vocab, int ld, int idx_offset, int bad_none, int chunk,
                    int groups, int* __restrict__ part) {
  __shared__ float sv[SAMP_THREADS / 32];
  __shared__ int si[SAMP_THREADS / 32], sb[SAMP_THREADS / 32];
  pdl_wait(); pdl_launch();
  const int row = blockIdx.y, g = blockIdx.x;
  const int start = g * chunk;
  const int end = min(start + chunk, vocab);
  const float* lr = logits + (size_t)row * ld;
  Cand best{0.f, -1};
  int bad = bad_none;
  for (int j = start + threadIdx.x; j < end; j += SAMP_THREADS) {
    float v = lr[j];
    if (finite_f32(v)) { if (best.i < 0 || v > best.v) { best.v = v; best.i = j + idx_offset; } }
    else if (j + idx_offset < bad) bad = j + idx_offset;
  }
  best = warp_best(best);
  bad = warp_min_i(bad);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best.v; si[w] = best.i; sb[w] = bad; }
  __syncthreads();
  if (w == 0) {
    Cand c{0.f, -1}; int b = bad_none;
    if (l < SAMP_THREADS / 32) { c.v = sv[l]; c.i = si[l]; b = sb[l]; }
    c = warp_best(c); b = warp_min_i(b);
    if (l == 0) {
      size_t p = ((size_t)row * groups + g) * 3;
      part[p] = __float_as_int(c.v); part[p + 1] = c.i; part[p + 2] = b;
    }
  }
}

// Stage 2 over `nparts` partial tables (one per vocabulary shard), each [rows, groups, 3], part_stride ints apart.
__global__ void argmax_combine_kernel(const int* __restrict__ part, int nparts, long long part_stride, int groups,
                                      int bad_none, int* __restrict__ out) {
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x, l = threadIdx.x;  // one warp
  Cand c{0.f, -1}; int b = bad_none;
  for (int e = l; e < nparts * groups; e += 32) {
    const int pt = e / groups, g = e - pt * groups;
    const int* p = part + (size_t)pt * part_stride + ((size_t)row * groups + g) * 3;
    Cand t{__int_as_float(p[0]), p[1]};
    c = better(c, t);
    b = min(b, p[2]);
  }
  c = warp_best(c); b = warp_min_i(b);
  if (l == 0) {
    bool nf = b < bad_none;
    out[row * 2] = (nf || c.i < 0) ? 0 : c.i;
    out[row * 2 + 1] = nf ? b : -1;
  }
}

// Block-wide helpers over SAMP_BIG threads.
constexpr int SAMP_BIG = 1024;
__device__ __forceinline__ float block_red_f(float v, bool is_max, float* sh) {
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  v = is_max ? warp_max(v) : -warp_max(-v);
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = sh[l];  // SAMP_BIG/32 == 32 entries
  r = is_max ? warp_max(r) : -warp_max(-r);
  __syncthreads();
  return r;
}
__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sh) {
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (l == 0) sh[w] = v;
  __syncthreads();
  unsigned long long r = sh[l];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// rule: 1 = Gumbel (temperature+min-p), 2 = +top-k, 3 = +top-k+top-p.
// params [rows,4] = (inv_temp, floor_offset, noise_scale, top_p); top_k [rows]; seeds [rows] (u32 bits).
__global__ void __launch_bounds__(SAMP_BIG)
sample_gumbel_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ params,
                     const int* __restrict__ top_k, const int* __restrict__ seeds, int rule,
                     int* __restrict__ out) {
  __shared__ float shf[32];
  __shared__ unsigned long long shu[32];
  __shared__ int shi[32];
  __shared__ float shv[32];
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * vocab;
  const float inv_temp = params[row * 4 + 0], floor_offset = params[row * 4 + 1];
  const float noise_scale = params[row * 4 + 2], top_p = params[row * 4 + 3];
  const uint32_t seed = (uint32_t)seeds[row];
  const float MASKED = -FLT_MAX;

  float mx = -FLT_MAX, mn = FLT_MAX;
  int bad = vocab;
  for (int j = threadIdx.x; j < vocab; j += SAMP_BIG) {
    float v = lr[j];
    if (finite_f32(v)) { mx = fmaxf(mx, v); if (v < mn && v != MASKED) mn = v; }
    else if (j < bad) bad = j;
  }
  mx = block_red_f(mx, true, shf);
  mn = block_red_f(mn, false, shf);
  {
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    bad = warp_min_i(bad);
    if (l == 0) shi[w] = bad;
    __syncthreads();
    bad = warp_min_i(shi[l]);
    __syncthreads();
  }

  float lo = mn;
  if (rule >= 2) {
    int k = top_k[row];
    if ((float)k > 0.f) {
      float hi = mx;
      for (int it = 0; it < 30; ++it) {
        float mid = __fmul_rn(__fadd_rn(lo, hi), 0.5f);
        unsigned long long cnt = 0;
        for (int j = threadIdx.x; j < vocab; j += SAMP_BIG) cnt += (lr[j] >= mid) ? 1ull : 0ull;
        cnt = block_sum_u64(cnt, shu);
        if ((float)cnt >= (float)k) lo = mid; else hi = mid;
      }
    }
  }
  const float t_k = lo;
  const float min_p_floor = __fadd_rn(mx, floor_offset);
  float floor_v = min_p_floor > t_k ? min_p_floor : t_k;
  if (rule >= 3) {
    const float floor1 = floor_v;
    if (top_p <= 0.f) {
      floor_v = mx;
    } else if (top_p < 1.f) {
      auto mass_at = [&](float th) -> unsigned long long {
        unsigned long long m = 0;
        for (int j = threadIdx.x; j < vocab; j += SAMP_BIG) {
          float v = lr[j];
          if (v >= th) m += (unsigned long long)(unsigned int)roundf(expf(__fmul_rn(__fsub_rn(v, mx), inv_temp)) * 16777216.0f);
        }
        return block_sum_u64(m, shu);
      };
      unsigned long long total = mass_at(floor1);
      unsigned long long thresh = (unsigned long long)roundf(__fmul_rn(top_p, (float)total));
      float tlo = floor1, thi = mx;
      for (int it = 0; it < 30; ++it) {
        float mid = __fmul_rn(__fadd_rn(tlo, thi), 0.5f);
        if (mass_at(mid) >= thresh) tlo = mid; else thi = mid;
      }
      floor_v = floor1 > tlo ? floor1 : tlo;
    }
  }

  Cand best{0.f, -1};
  for (int j = threadIdx.x; j < vocab; j += SAMP_BIG) {
    float v = lr[j];
    if (v >= floor_v) {
      float u = uniform_at(seed, (uint32_t)j);
      float noise = -logf(-logf(u));
      float pert = __fadd_rn(__fmul_rn(v, inv_temp), __fmul_rn(noise_scale, noise));
      if (best.i < 0 || pert > best.v) { best.v = pert; best.i = j; }
    }
  }
  best = warp_best(best);
  {
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { shv[w] = best.v; shi[w] = best.i; }
    __syncthreads();
    if (w == 0) {
      Cand c{shv[l], shi[l]};
      c = warp_best(c);
      if (l == 0) {
        bool nf = bad < vocab;
        out[row * 2] = (nf || c.i < 0) ? 0 : c.i;
        out[row * 2 + 1] = nf ? bad : -1;
      }
    }
  }
}

__global__ void random_uniform_kernel(const int* __restrict__ seeds, int cols, float* __restrict__ out, size_t n) {
  pdl_wait(); pdl_launch();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  size_t r = i / cols;
  out[i] = uniform_at((uint32_t)seeds[r], (uint32_t)(i - r * cols));
}

}  // namespace poot

using namespace poot;

// part: int32 scratch [rows, groups, 3]; groups = ceil(vocab / chunk).
POOT_API int poot_argmax_partials(const float* logits, int rows, int vocab, int ld, int idx_offset, int vocab_total,
                                  int chunk, int* part, cudaStream_t s) {
  if (rows == 0) return 0;
  int groups = (vocab + chunk - 1) / chunk;
  if (groups < 1) groups = 1;
  return launch_k(argmax_chunk_kernel, dim3(groups, rows), dim3(SAMP_THREADS), 0, s, logits, vocab, ld, idx_offset,
                  vocab_total, chunk, groups, part);
}

POOT_API int poot_argmax_combine(const int* part, int nparts, long long part_stride, int rows, int groups,
                                 int vocab_total, int* out, cudaStream_t s) {
  if (rows == 0) return 0;
  return launch_k(argmax_combine_kernel, dim3(rows), dim3(32), 0, s, part, nparts, part_stride, groups, vocab_total,
                  out);
}

POOT_API int poot_argmax(const float* logits, int rows, int vocab, int chunk, int* part, int* out, cudaStream_t s) {
  int e = poot_argmax_partials(logits, rows, vocab, vocab, 0, vocab, chunk, part, s);
  if (e) return e;
  int groups = (vocab + chunk - 1) / chunk;
  if (groups < 1) groups = 1;
  return poot_argmax_combine(part, 1, 0, rows, groups, vocab, out, s);
}

POOT_API int poot_sample_gumbel(const float* logits, int rows, int vocab, const float* params, const int* top_k,
                                const int* seeds, int rule, int* out, cudaStream_t s) {
  if (rows == 0) return 0;
  if (rule < 1 || rule > 3) return (int)cudaErrorInvalidValue;
  return launch_k(sample_gumbel_kernel, dim3(rows), dim3(SAMP_BIG), 0, s, logits, vocab, params, top_k, seeds, rule, out);
}

POOT_API int poot_random_uniform(const int* seeds, int rows, int cols, float* out, cudaStream_t s) {
  size_t n = (size_t)rows * cols;
  if (n == 0) return 0;
  return launch_k(random_uniform_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, seeds, cols, out, n);
}
