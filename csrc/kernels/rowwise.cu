// Row-wise and element-wise kernels: embedding gather, RMSNorm (with fused
// residual add and split-K / cross-rank partial reduction), SwiGLU, casts.
//
// Reference behaviour covered: the fused row family (RMSNorm, crates/poot-kernelgen
// fused.rs; op definition crates/poot-graph-ir/src/ops/norm.rs:4-29), the pointwise
// family (SwiGLU, residual add; ops/activation.rs:94-143) and the packed bf16 row
// gather (crates/pootc/kernels/packed/packed_bf16_row_gather.rs).
#include "common.cuh"

namespace poot {

int g_poot_pdl = 0;

// ---------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :]   (bf16 rows, D % 8 == 0)
// ---------------------------------------------------------------------------
__global__ void embed_gather_kernel(const int* __restrict__ ids, const uint4* __restrict__ table,
                                    uint4* __restrict__ out, int T, int D8, int vocab) {
  pdl_wait(); pdl_launch();
  int t = blockIdx.x;
  int id = ids[t];
  if (!POOT_IN_RANGE(id, vocab, kSiteTokenId) || id < 0 || id >= vocab) id = 0;
  const uint4* src = table + (size_t)id * D8;
  uint4* dst = out + (size_t)t * D8;
  for (int i = threadIdx.x; i < D8; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------
// RMSNorm family.  One CTA per row.
//   h_new = h (+ sum_p partial_p)             (optional residual update, written back)
//   y     = h_new / sqrt(mean(h_new^2)+eps) * w
// Partials are fp32 [P, T, D] (split-K slices of the producing GEMM) or bf16.
// ---------------------------------------------------------------------------
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// MAXV: 16-byte vectors per thread held in registers (D <= THREADS*8*MAXV).
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,      // [T,D] input / residual stream
               __nv_bfloat16* __restrict__ h_out,        // [T,D] updated residual (may alias x) or null
               const float* __restrict__ partials,       // [P,T,D] fp32 or null
               int P, size_t partial_stride,             // elements between partial slices
               const __nv_bfloat16* __restrict__ w,      // [D]
               __nv_bfloat16* __restrict__ y,            // [T,D] normalized output (or null)
               int D, float eps) {
  __shared__ float red[32];
  pdl_wait(); pdl_launch();
  const int row = blockIdx.x;
  const int D8 = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int c = threadIdx.x + i * THREADS;
    if (c < D8) {
      uint4 raw = xr[c];
      unpack8(raw, v[i]);
      if (partials != nullptr) {
        for (int p = 0; p < P; ++p) {
          const float4* pr = reinterpret_cast<const float4*>(partials + p * partial_stride + (size_t)row * D) + 2 * c;
          float4 a = pr[0], b = pr[1];
          v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
          v[i][4] += b.x; v[i][5] += b.y; v[i][6] += b.z; v[i][7] += b.w;
        }
        // The residual stream is stored in bf16: normalise what is stored.
        uint4 packed = pack8(v[i]);
        unpack8(packed, v[i]);
        if (h_out != nullptr) reinterpret_cast<uint4*>(h_out + (size_t)row * D)[c] = packed;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  float tot = block_sum<THREADS>(ss, red);
  float inv = rsqrtf(tot / (float)D + eps);
  if (y == nullptr) return;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * D);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int c = threadIdx.x + i * THREADS;
    if (c < D8) {
      float wf[8], o[8];
      unpack8(wr[c], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * wf[j];
      yr[c] = pack8(o);
    }
  }
}

// out[t, j] = silu(gate) * up over an interleaved or split gate/up buffer.
//   split layout:       gu[t, 0:F] = gate, gu[t, F:2F] = up
//   interleaved layout: gu[t, 2j] = gate_j, gu[t, 2j+1] = up_j
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                              int T, int F, int interleaved) {
  pdl_wait(); pdl_launch();
  size_t n = (size_t)T * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t t = i / F;
    int j = (int)(i - t * F);
    float g, u;
    if (interleaved) {
      __nv_bfloat162 p = reinterpret_cast<const __nv_bfloat162*>(gu + t * 2 * F)[j];
      g = __low2float(p); u = __high2float(p);
    } else {
      g = __bfloat162float(gu[t * 2 * F + j]);
      u = __bfloat162float(gu[t * 2 * F + F + j]);
    }
    out[i] = __float2bfloat16(silu(g) * u);
  }
}

// act(gate) * up for gated FFNs whose activation is not plain SiLU: act 0 = SiLU, 1 = GELU (tanh form), 2 = GELU (erf),
// 3 = clamped SwiGLU.
__global__ void gated_act_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                 int T, int F, int interleaved, int act, float limit, float alpha) {
  pdl_wait(); pdl_launch();
  size_t n = (size_t)T * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t t = i / F;
    int j = (int)(i - t * F);
    float g, u;
    if (interleaved) {
      __nv_bfloat162 p = reinterpret_cast<const __nv_bfloat162*>(gu + t * 2 * F)[j];
      g = __low2float(p); u = __high2float(p);
    } else {
      g = __bfloat162float(gu[t * 2 * F + j]);
      u = __bfloat162float(gu[t * 2 * F + F + j]);
    }
    float a;
    if (act == 1) {
      const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      a = g / (1.f + __expf(-2.f * z));
    } else if (act == 2) {
      a = 0.5f * g * (1.f + erff(g * 0.7071067811865475f));
    } else if (act == 3) {          // clamped SwiGLU: gate <= limit, |up| <= limit, (up + 1) * gate * sigmoid(alpha * gate)
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit) + 1.f;
      a = g / (1.f + __expf(-alpha * g));
    } else {
      a = silu(g);
    }
    out[i] = __float2bfloat16(a * u);
  }
}

// LayerNorm over the last axis: (x - mean) * rsqrt(var + eps) * w (+ b).  One CTA of 256 threads per row.
__global__ void __launch_bounds__(256)
layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                 float eps, __nv_bfloat16* __restrict__ out, int D) {
  __shared__ float red[2][8];
  pdl_wait(); pdl_launch();
  const __nv_bfloat16* xr = x + (size_t)blockIdx.x * D;
  __nv_bfloat16* o = out + (size_t)blockIdx.x * D;
  float s = 0.f, ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) { const float v = __bfloat162float(xr[i]); s += v; ss += v * v; }
  s = warp_sum(s); ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = ss; }
  __syncthreads();
  s = 0.f; ss = 0.f;
  for (int i = 0; i < 8; ++i) { s += red[0][i]; ss += red[1][i]; }
  const float mean = s / (float)D;
  const float var = fmaxf(ss / (float)D - mean * mean, 0.f);
  const float inv = rsqrtf(var + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = (__bfloat162float(xr[i]) - mean) * inv * __bfloat162float(w[i]);
    if (b != nullptr) v += __bfloat162float(b[i]);
    o[i] = __float2bfloat16(v);
  }
}

// x = act(x) in place over bf16: 1 = GELU (tanh form), 2 = GELU (erf), 4 = squared ReLU, 0 = SiLU
__global__ void act_bf16_kernel(__nv_bfloat16* __restrict__ x, size_t n, int act) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float g = __bfloat162float(x[i]);
    float a;
    if (act == 1) {
      const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      a = g / (1.f + __expf(-2.f * z));
    } else if (act == 2) {
      a = 0.5f * g * (1.f + erff(g * 0.7071067811865475f));
    } else if (act == 4) {
      const float r = fmaxf(g, 0.f);
      a = r * r;
    } else {
      a = silu(g);
    }
    x[i] = __float2bfloat16(a);
  }
}

// h[t, :] = rows[t, :] for the rows whose flag is set (rows of another modality in place of token embeddings);
// 16-byte chunks, D a multiple of 8
__global__ void replace_rows_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ rows,
                                    const int* __restrict__ flags, int T, int D) {
  pdl_wait(); pdl_launch();
  const int chunks = D / 8;
  const size_t total = (size_t)T * chunks;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks);
    if (flags[t] == 0) continue;
    reinterpret_cast<uint4*>(h)[i] = reinterpret_cast<const uint4*>(rows)[i];
  }
}

// x = cap * tanh(x / cap) in place over fp32 logits
__global__ void softcap_f32_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv_cap);
}

__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, size_t n) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}

// h[t,:] += sum_p partial[p,t,:]   (split-K reduction without a following norm)
__global__ void reduce_partials_kernel(const __nv_bfloat16* h, const float* partials, int P,
                                       size_t partial_stride, __nv_bfloat16* out, size_t n) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = h ? __bfloat162float(h[i]) : 0.f;
    for (int p = 0; p < P; ++p) v += partials[p * partial_stride + i];
    out[i] = __float2bfloat16(v);
  }
}

__global__ void cast_f32_bf16_kernel(const float* in, __nv_bfloat16* out, size_t n) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* in, float* out, size_t n) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

// Device-side step advance for chained decode: feed the sampled token back as the next input and move
// every row one position forward (position, visible context, write slot), so consecutive graph replays
// need no host round trip (the reference's step chain, crates/poot-executor/src/lib.rs:532-540).
__global__ void decode_advance_kernel(const int* __restrict__ picked, int* __restrict__ tokens,
                                      int* __restrict__ positions, int* __restrict__ slots, int* __restrict__ ctx,
                                      const int* __restrict__ block_tables, int max_blocks,
                                      const int* __restrict__ row_seq, int B) {
  pdl_wait(); pdl_launch();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  if (slots[i] < 0) return;  // padding row
  tokens[i] = picked[2 * i];
  int pos = positions[i] + 1;
  positions[i] = pos;
  ctx[i] = pos + 1;
  int seq = row_seq ? row_seq[i] : i;
  int b = pos / 16;
  POOT_IN_RANGE(b, max_blocks, kSitePosition);      // a row that outgrew its block table: release writes slot -1
  int blk = b < max_blocks ? block_tables[(size_t)seq * max_blocks + b] : 0;
  if (!POOT_IN_RANGE(blk, POOT_LIMIT(kLimPoolBlocks), kSiteBlockId)) blk = 0;
  slots[i] = b < max_blocks ? blk * 16 + (pos % 16) : -1;
}

// ---- small pointwise and movement kernels the layer programs need between the large ones ------------------------
// x[t, :] += bias[:]   (bf16 rows with pitch ldx, bf16 or f32 bias; also the f32 form for router logits)
template <typename XT, typename BT>
__global__ void bias_add_kernel(XT* __restrict__ x, const BT* __restrict__ bias, int T, int N, int ldx) {
  pdl_wait(); pdl_launch();
  const size_t total = (size_t)T * N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / N), n = (int)(i - (size_t)t * N);
    XT* p = x + (size_t)t * ldx + n;
    *p = (XT)((float)*p + (float)bias[n]);
  }
}

// x *= s
__global__ void scale_bf16_kernel(__nv_bfloat16* __restrict__ x, size_t n, float s) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

// out[b, :] = src[idx[b], :]  moved in chunks of type C (16, 4 or 2 bytes: the widest that divides the row and both
// pitches); idx is int64.  An index outside [0, rows) copies row 0 (the step is refused on the host before it can
// name one).
template <typename C>
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, int rows,
                                   const long long* __restrict__ idx, uint8_t* __restrict__ out, long long out_pitch,
                                   int row_bytes) {
  pdl_wait(); pdl_launch();
  long long r = idx[blockIdx.x];
  if (!POOT_IN_RANGE(r, rows, kSiteGatherRow) || r < 0 || r >= rows) r = 0;
  const C* s = reinterpret_cast<const C*>(src + (size_t)r * src_pitch);
  C* d = reinterpret_cast<C*>(out + (size_t)blockIdx.x * out_pitch);
  for (int c = threadIdx.x; c < row_bytes / (int)sizeof(C); c += blockDim.x) d[c] = s[c];
}

// x[t, :] *= sigmoid(g[t * ldg])   (the per-token gate of a shared expert)
__global__ void sigmoid_gate_rows_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ g, int ldg, int T, int N) {
  pdl_wait(); pdl_launch();
  const size_t total = (size_t)T * N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / N);
    const float s = 1.f / (1.f + __expf(-g[(size_t)t * ldg]));
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
  }
}

// x[r, :] += table[idx[r / div] + e0, :] * (gate ? gate[r] : 1): the bias of each row's expert.  Rows of a padding
// tile (idx < 0) are left alone.
__global__ void bias_add_indexed_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ table,
                                        const int* __restrict__ idx, int div, int e0, int experts,
                                        const float* __restrict__ gate, int R, int N) {
  pdl_wait(); pdl_launch();
  const size_t total = (size_t)R * N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / N), n = (int)(i - (size_t)r * N);
    const int e = idx[r / div];
    if (e >= 0) POOT_IN_RANGE(e + e0, experts, kSiteExpertId);      // a negative id marks a padding tile
    if (e < 0 || e + e0 >= experts) continue;
    const float b = __bfloat162float(table[(size_t)(e + e0) * N + n]) * (gate ? gate[r] : 1.f);
    x[i] = __float2bfloat16(__bfloat162float(x[i]) + b);
  }
}

}  // namespace poot

using namespace poot;

POOT_API void poot_set_pdl(int on) { g_poot_pdl = on; }
POOT_API int poot_get_pdl() { return g_poot_pdl; }

POOT_API int poot_decode_advance(const int* picked, int* tokens, int* positions, int* slots, int* ctx,
                                 const int* block_tables, int max_blocks, const int* row_seq, int B, cudaStream_t s) {
  if (B == 0) return 0;
  return launch_k(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, picked, tokens, positions, slots, ctx, block_tables,
                                                        max_blocks, row_seq, B);
  return (int)cudaGetLastError();
}

POOT_API int poot_embed_gather(const int* ids, const void* table, void* out, int T, int D, int vocab,
                               cudaStream_t s) {
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  return launch_k(embed_gather_kernel, dim3(T), dim3(128), 0, s, ids, (const uint4*)table, (uint4*)out, T, D / 8, vocab);
  return (int)cudaGetLastError();
}

// x: [T,D] bf16.  partials: fp32 [P,T,D] or null.  h_out: where x+sum(partials) is stored (may equal x)
// or null.  y: normalized output or null (reduce only).
POOT_API int poot_rmsnorm(const void* x, void* h_out, const float* partials, int P, long long partial_stride,
                          const void* w, void* y, int T, int D, float eps, cudaStream_t s) {
  if (D % 8) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  __nv_bfloat16* hb = (__nv_bfloat16*)h_out;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
  __nv_bfloat16* yb = (__nv_bfloat16*)y;
  int D8 = D / 8;
  if (D8 <= 128) return launch_k(rmsnorm_kernel<128, 1>, dim3(T), dim3(128), 0, s, xb, hb, partials, P, (size_t)partial_stride, wb, yb, D, eps);
  else if (D8 <= 256) return launch_k(rmsnorm_kernel<256, 1>, dim3(T), dim3(256), 0, s, xb, hb, partials, P, (size_t)partial_stride, wb, yb, D, eps);
  else if (D8 <= 512) return launch_k(rmsnorm_kernel<512, 1>, dim3(T), dim3(512), 0, s, xb, hb, partials, P, (size_t)partial_stride, wb, yb, D, eps);
  else if (D8 <= 1024) return launch_k(rmsnorm_kernel<512, 2>, dim3(T), dim3(512), 0, s, xb, hb, partials, P, (size_t)partial_stride, wb, yb, D, eps);
  else if (D8 <= 2048) return launch_k(rmsnorm_kernel<512, 4>, dim3(T), dim3(512), 0, s, xb, hb, partials, P, (size_t)partial_stride, wb, yb, D, eps);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

POOT_API int poot_swiglu(const void* gu, void* out, int T, int F, int interleaved, cudaStream_t s) {
  size_t n = (size_t)T * F;
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(swiglu_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F, interleaved);
  return (int)cudaGetLastError();
}

POOT_API int poot_gated_act(const void* gu, void* out, int T, int F, int interleaved, int act, float limit, float alpha,
                            cudaStream_t s) {
  size_t n = (size_t)T * F;
  if (n == 0) return 0;
  if (act < 0 || act > 3 || (act == 3 && !(limit > 0.f))) return (int)cudaErrorInvalidValue;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(gated_act_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F,
                  interleaved, act, limit, alpha);
}

POOT_API int poot_layernorm(const void* x, const void* w, const void* b, float eps, void* out, int T, int D, cudaStream_t s) {
  if (T == 0) return 0;
  if (D < 1) return (int)cudaErrorInvalidValue;
  return launch_k(layernorm_kernel, dim3(T), dim3(256), 0, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                  (const __nv_bfloat16*)b, eps, (__nv_bfloat16*)out, D);
}

POOT_API int poot_act_bf16(void* x, long long n, int act, cudaStream_t s) {
  if (n == 0) return 0;
  if (act != 0 && act != 1 && act != 2 && act != 4) return (int)cudaErrorInvalidValue;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(act_bf16_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, (size_t)n, act);
}

POOT_API int poot_replace_rows(void* h, const void* rows, const int* flags, int T, int D, cudaStream_t s) {
  if (T == 0) return 0;
  if (D < 8 || D % 8 != 0) return (int)cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(rows)) & 15) return (int)cudaErrorInvalidValue;
  size_t total = (size_t)T * (D / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(replace_rows_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)h, (const __nv_bfloat16*)rows, flags, T, D);
}

POOT_API int poot_softcap_f32(void* x, long long n, float cap, cudaStream_t s) {
  if (n == 0) return 0;
  if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(softcap_f32_kernel, dim3(blocks), dim3(256), 0, s, (float*)x, (size_t)n, cap, 1.f / cap);
}

POOT_API int poot_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(add_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, (size_t)n);
  return (int)cudaGetLastError();
}

POOT_API int poot_reduce_partials(const void* h, const float* partials, int P, long long partial_stride,
                                  void* out, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(reduce_partials_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)h, partials, P, (size_t)partial_stride,
                                                (__nv_bfloat16*)out, (size_t)n);
  return (int)cudaGetLastError();
}

POOT_API int poot_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(cast_f32_bf16_kernel, dim3(blocks), dim3(256), 0, s, in, (__nv_bfloat16*)out, (size_t)n);
  return (int)cudaGetLastError();
}
POOT_API int poot_cast_bf16_f32(const void* in, float* out, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(cast_bf16_f32_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)in, out, (size_t)n);
  return (int)cudaGetLastError();
}

// bias dtype: 0 bf16, 1 f32.  x dtype: 0 bf16, 1 f32 (the f32 form takes an f32 bias only).
POOT_API int poot_bias_add(void* x, const void* bias, int T, int N, int ldx, int x_f32, int bias_f32, cudaStream_t s) {
  if (T == 0 || N == 0) return 0;
  size_t total = (size_t)T * N;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (x_f32) {
    if (!bias_f32) return (int)cudaErrorInvalidValue;
    return launch_k(bias_add_kernel<float, float>, dim3(blocks), dim3(256), 0, s, (float*)x, (const float*)bias, T, N, ldx);
  }
  if (bias_f32)
    return launch_k(bias_add_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, (const float*)bias, T, N, ldx);
  return launch_k(bias_add_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)bias, T, N, ldx);
}

POOT_API int poot_scale_bf16(void* x, long long n, float scale, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(scale_bf16_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, (size_t)n, scale);
}

POOT_API int poot_gather_rows(const void* src, long long src_pitch, int rows, const long long* idx, void* out,
                              long long out_pitch, int n_out, int row_bytes, cudaStream_t s) {
  if (n_out == 0) return 0;
  const uintptr_t all = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out) | (uintptr_t)src_pitch |
                        (uintptr_t)out_pitch | (uintptr_t)row_bytes;
  const dim3 g(n_out), b(128);
  if (all % 16 == 0)
    return launch_k(gather_rows_kernel<uint4>, g, b, 0, s, (const uint8_t*)src, src_pitch, rows, idx, (uint8_t*)out,
                    out_pitch, row_bytes);
  if (all % 4 == 0)
    return launch_k(gather_rows_kernel<uint32_t>, g, b, 0, s, (const uint8_t*)src, src_pitch, rows, idx, (uint8_t*)out,
                    out_pitch, row_bytes);
  if (all % 2 == 0)
    return launch_k(gather_rows_kernel<uint16_t>, g, b, 0, s, (const uint8_t*)src, src_pitch, rows, idx, (uint8_t*)out,
                    out_pitch, row_bytes);
  return (int)cudaErrorInvalidValue;
}

POOT_API int poot_sigmoid_gate_rows(void* x, const float* g, int ldg, int T, int N, cudaStream_t s) {
  if (T == 0 || N == 0) return 0;
  size_t total = (size_t)T * N;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(sigmoid_gate_rows_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, g, ldg, T, N);
}

POOT_API int poot_bias_add_indexed(void* x, const void* table, const int* idx, int div, int e0, int experts,
                                   const float* gate, int R, int N, cudaStream_t s) {
  if (R == 0 || N == 0) return 0;
  if (div <= 0) return (int)cudaErrorInvalidValue;
  size_t total = (size_t)R * N;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(bias_add_indexed_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, (const __nv_bfloat16*)table,
                  idx, div, e0, experts, gate, R, N);
}
