// Paged flash attention for decode and chunked prefill rows (online softmax,
// GQA heads of one KV head share every K/V load, split-KV with a combine pass).
//
// A "row" is one query token: row r belongs to sequence row_seq[r] and sees the
// first row_ctx[r] keys of that sequence (causal: position + 1), optionally
// limited to the last `window` keys.  K/V live in pools
//   [num_blocks, Hkv, 16, D] bf16
// addressed through the per-sequence block table [nseq, max_blocks].
//
// Work split: grid (Hkv * head_groups, rows, splits); 4 warps per CTA; a warp
// consumes one 16-key block per step: D/8 lanes cover one key row with 16-byte
// loads, the partial dot products of (keys x heads) are folded across lanes by
// a transposed butterfly, scores/probabilities pass through a warp-private
// shared tile, and P.V accumulates in registers.
//
// Reference behaviour covered: Attention Streaming / SplitKv + AttentionCombine
// (crates/poot-kernelgen/src/attention.rs:7-29,283-300; planner split rule
// crates/poot-graph-plan/src/planner/attention.rs:305-347), paged keys through a
// slot map, live length, causal window, softcap
// (crates/poot-graph-ir/src/op.rs:1013-1112).
#include "common.cuh"

namespace poot {

constexpr int ATT_WARPS = 4;
constexpr int ATT_BLOCK = 16;  // keys per pool block

template <int D, int NREP>
__global__ void __launch_bounds__(ATT_WARPS * 32, 4)   // four CTAs per SM: 592 slots, so 512 (64 rows x 8 KV heads) run as one wave
attn_paged_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,  // row stride in elements
                  const __nv_bfloat16* __restrict__ kpool, const __nv_bfloat16* __restrict__ vpool,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ row_seq,
                  const int* __restrict__ row_ctx, __nv_bfloat16* __restrict__ out, int out_stride,
                  float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv, int head_groups,
                  float scale, float softcap, int window, int splits) {
  constexpr int LPP = D / 8;           // lanes per key row
  constexpr int GROUPS = 32 / LPP;     // key rows loaded per warp instruction
  constexpr int PPG = ATT_BLOCK / GROUPS;  // keys per lane group per block
  constexpr int NS = PPG * NREP;       // partial dot products per lane
  constexpr float LOG2E = 1.4426950408889634f;

  __shared__ float s_sc[ATT_WARPS][ATT_BLOCK * NREP];
  __shared__ float s_alpha[ATT_WARPS][NREP];
  __shared__ float s_o[ATT_WARPS][NREP][D];
  __shared__ float s_m[ATT_WARPS][NREP];
  __shared__ float s_l[ATT_WARPS][NREP];

  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = lane % LPP, g = lane / LPP;
  const int kvh = blockIdx.x / head_groups;
  const int hg = blockIdx.x - kvh * head_groups;
  const int n_rep = NREP * head_groups;
  const int h0 = kvh * n_rep + hg * NREP;  // first query head of this CTA
  const int row = blockIdx.y;
  const int split = blockIdx.z;
  const int ctx = row_ctx[row];
  const int seq = row_seq ? row_seq[row] : row;
  const int* bt = block_tables + (size_t)seq * max_blocks;

  int first_key = (window > 0 && ctx > window) ? ctx - window : 0;
  int nb_begin = first_key / ATT_BLOCK;
  int nb_end = (ctx + ATT_BLOCK - 1) / ATT_BLOCK;
  {
    int nb = nb_end - nb_begin;
    int per = (nb + splits - 1) / splits;
    int b0 = nb_begin + split * per;
    int b1 = b0 + per;
    nb_begin = b0 < nb_end ? b0 : nb_end;
    nb_end = b1 < nb_end ? b1 : nb_end;
  }

  // queries of the NREP heads, this lane's 8 channels, pre-scaled
  float qf[NREP][8];
#pragma unroll
  for (int h = 0; h < NREP; ++h) {
    uint4 raw = *reinterpret_cast<const uint4*>(q + (size_t)row * q_stride + (size_t)(h0 + h) * D + c * 8);
    unpack8(raw, qf[h]);
#pragma unroll
    for (int j = 0; j < 8; ++j) qf[h][j] *= scale;
  }

  float o[NREP][8];
#pragma unroll
  for (int h = 0; h < NREP; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j) o[h][j] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;  // statistics of head (lane % NREP), replicated
  const int hl = lane % NREP;

  for (int b = nb_begin + warp; b < nb_end; b += ATT_WARPS) {
    int blk = bt[b];
    if (!POOT_IN_RANGE(blk, POOT_LIMIT(kLimPoolBlocks), kSiteBlockId)) blk = 0;
    const int pbase = b * ATT_BLOCK;
    const size_t boff = ((size_t)blk * Hkv + kvh) * ATT_BLOCK * D;
    const uint4* kb = reinterpret_cast<const uint4*>(kpool + boff);
    const uint4* vb = reinterpret_cast<const uint4*>(vpool + boff);
    uint4 kr[PPG], vr[PPG];
#pragma unroll
    for (int i = 0; i < PPG; ++i) {
      int p = g * PPG + i;
      bool ok = (pbase + p) < ctx;
      kr[i] = ok ? kb[p * LPP + c] : make_uint4(0, 0, 0, 0);
      vr[i] = ok ? vb[p * LPP + c] : make_uint4(0, 0, 0, 0);
    }
    float s[NS];
#pragma unroll
    for (int i = 0; i < PPG; ++i) {
      float kf[8];
      unpack8(kr[i], kf);
#pragma unroll
      for (int h = 0; h < NREP; ++h) {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) a += qf[h][j] * kf[j];
        s[i * NREP + h] = a;
      }
    }
    // transposed butterfly over the LPP lanes of a key row
    int cnt = NS, base = 0;
#pragma unroll
    for (int off = LPP / 2; off >= 1; off >>= 1) {
      if (cnt > 1) {
        const int n = cnt / 2;
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < NS / 2; ++i) {
          if (i < n) {
            float send = up ? s[i] : s[i + n];
            float keep = up ? s[i + n] : s[i];
            s[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
          }
        }
        if (up) base += n;
        cnt = n;
      } else {
        s[0] += __shfl_xor_sync(0xffffffffu, s[0], off);
      }
    }
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (i < cnt) {
        int idx = base + i;                 // = key_in_group * NREP + head
        int p = g * PPG + idx / NREP;       // key within the block
        float v = s[i];
        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
        v *= LOG2E;
        int pos = pbase + p;
        if (pos >= ctx || pos < first_key) v = -INFINITY;
        s_sc[warp][p * NREP + (idx % NREP)] = v;
      }
    }
    __syncwarp();
    // online softmax over the 16 x NREP tile: lane owns entries lane, lane+32, ...
    constexpr int ITEMS = ATT_BLOCK * NREP;
    constexpr int PER = (ITEMS + 31) / 32;
    float e[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      int idx = lane + 32 * t;
      e[t] = idx < ITEMS ? s_sc[warp][idx] : -INFINITY;
      mx = fmaxf(mx, e[t]);
    }
#pragma unroll
    for (int off = 16; off >= NREP; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float m_new = fmaxf(m_run, mx);
    float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
    float ls = 0.f;
#pragma unroll
    for (int t = 0; t < PER; ++t) {
      int idx = lane + 32 * t;
      float p = (m_new == -INFINITY) ? 0.f : exp2f(e[t] - m_new);
      if (idx < ITEMS) s_sc[warp][idx] = p;
      ls += (idx < ITEMS) ? p : 0.f;
    }
#pragma unroll
    for (int off = 16; off >= NREP; off >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, off);
    l_run = l_run * alpha + ls;
    m_run = m_new;
    if (lane < NREP) s_alpha[warp][lane] = alpha;
    __syncwarp();
    // P.V
    float al[NREP];
#pragma unroll
    for (int h = 0; h < NREP; ++h) al[h] = s_alpha[warp][h];
#pragma unroll
    for (int h = 0; h < NREP; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) o[h][j] *= al[h];
#pragma unroll
    for (int i = 0; i < PPG; ++i) {
      float vf[8];
      unpack8(vr[i], vf);
      int p = g * PPG + i;
#pragma unroll
      for (int h = 0; h < NREP; ++h) {
        float pv = s_sc[warp][p * NREP + h];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[h][j] += pv * vf[j];
      }
    }
    __syncwarp();
  }

  // fold the lane groups (they saw different keys of the same blocks, same m)
#pragma unroll
  for (int off = LPP; off < 32; off <<= 1)
#pragma unroll
    for (int h = 0; h < NREP; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) o[h][j] += __shfl_xor_sync(0xffffffffu, o[h][j], off);

  if (g == 0) {
#pragma unroll
    for (int h = 0; h < NREP; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) s_o[warp][h][c * 8 + j] = o[h][j];
  }
  if (lane < NREP) { s_m[warp][lane] = m_run; s_l[warp][lane] = l_run; }
  __syncthreads();

  // cross-warp combine: thread handles (head, dim) pairs
  for (int e = threadIdx.x; e < NREP * D; e += ATT_WARPS * 32) {
    int h = e / D, d = e - h * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, s_m[w][h]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      float wgt = (s_m[w][h] == -INFINITY) ? 0.f : exp2f(s_m[w][h] - M);
      acc += s_o[w][h][d] * wgt;
      L += s_l[w][h] * wgt;
    }
    int head = h0 + h;
    if (splits == 1) {
      float r = L > 0.f ? acc / L : 0.f;
      out[(size_t)row * out_stride + (size_t)head * D + d] = __float2bfloat16(r);
    } else {
      size_t pi = ((size_t)row * Hq + head) * splits + split;
      part_o[pi * D + d] = acc;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
  }
}

// out[row, head, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int out_stride, int Hq, int D, int splits) {
  pdl_wait(); pdl_launch();
  const int row = blockIdx.y, head = blockIdx.x;
  size_t pi = ((size_t)row * Hq + head) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(pi + s) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < splits; ++s) {
      float m = part_ml[(pi + s) * 2];
      float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
      acc += part_o[(pi + s) * D + d] * w;
      L += part_ml[(pi + s) * 2 + 1] * w;
    }
    out[(size_t)row * out_stride + (size_t)head * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
  }
}

template <int D>
static int launch_attn(const void* q, int q_stride, const void* kpool, const void* vpool, const int* bt,
                       int max_blocks, const int* row_seq, const int* row_ctx, void* out, int out_stride,
                       float* part_o, float* part_ml, int R, int Hq, int Hkv, float scale, float softcap,
                       int window, int splits, cudaStream_t s) {
  int n_rep = Hq / Hkv;
  int nrep_t = n_rep >= 4 ? 4 : n_rep;
  if (n_rep % nrep_t) return (int)cudaErrorInvalidValue;
  int hgs = n_rep / nrep_t;
  dim3 grid(Hkv * hgs, R, splits), block(ATT_WARPS * 32);
#define POOT_ATT(NR)                                                                                        \
  err = launch_k(attn_paged_kernel<D, NR>, grid, block, 0, s, (const __nv_bfloat16*)q, q_stride,            \
      (const __nv_bfloat16*)kpool, (const __nv_bfloat16*)vpool, bt, max_blocks, row_seq, row_ctx,            \
      (__nv_bfloat16*)out, out_stride, part_o, part_ml, Hq, Hkv, hgs, scale, softcap, window, splits)
  int err = 0;
  switch (nrep_t) {
    case 1: POOT_ATT(1); break;
    case 2: POOT_ATT(2); break;
    case 4: POOT_ATT(4); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef POOT_ATT
  if (err) return err;
  if (splits > 1) {
    err = launch_k(attn_combine_kernel, dim3(Hq, R), dim3(D <= 128 ? D : 128), 0, s, (const float*)part_o,
                   (const float*)part_ml, (__nv_bfloat16*)out, out_stride, Hq, D, splits);
  }
  return err;
}

}  // namespace poot

using namespace poot;

// Scratch (only read/written when splits > 1): part_o fp32 [R, Hq, splits, D], part_ml fp32 [R, Hq, splits, 2].
POOT_API int poot_attn_paged(const void* q, int q_stride, const void* kpool, const void* vpool, const int* block_tables,
                             int max_blocks, const int* row_seq, const int* row_ctx, void* out, int out_stride,
                             float* part_o, float* part_ml, int R, int Hq, int Hkv, int D, float scale, float softcap,
                             int window, int splits, cudaStream_t s) {
  if (R == 0) return 0;
  if (R < 0 || Hq <= 0 || Hkv <= 0) return (int)cudaErrorInvalidValue;   // before the modulo: Hkv == 0 must not trap the host
  if (splits < 1 || Hq % Hkv) return (int)cudaErrorInvalidValue;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return (int)cudaErrorInvalidValue;
  if (D == 128)
    return launch_attn<128>(q, q_stride, kpool, vpool, block_tables, max_blocks, row_seq, row_ctx, out, out_stride,
                            part_o, part_ml, R, Hq, Hkv, scale, softcap, window, splits, s);
  if (D == 64)
    return launch_attn<64>(q, q_stride, kpool, vpool, block_tables, max_blocks, row_seq, row_ctx, out, out_stride,
                           part_o, part_ml, R, Hq, Hkv, scale, softcap, window, splits, s);
  return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared in poot_noalloc.h).  The split-KV partials go to a file-scope
// device array instead of caller-provided scratch.  In host code `g_noalloc_scratch` is only a
// stand-in for the symbol, not a device address: the address handed to the kernels is resolved
// once per device with cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------------------------
#include "poot_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[POOT_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

POOT_API int poot_attn_paged_noalloc(const void* q, int q_stride, const void* kpool, const void* vpool,
                                     const int* block_tables, int max_blocks, const int* row_seq, const int* row_ctx,
                                     void* out, int out_stride, int R, int Hq, int Hkv, int D, float scale,
                                     float softcap, int window, int splits, cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || D <= 0 || splits < 1) return (int)cudaErrorInvalidValue;
  const unsigned long long need = (unsigned long long)R * Hq * splits * (unsigned long long)(D + 2);
  if (need > (unsigned long long)POOT_NOALLOC_SCRATCH_FLOATS) return (int)cudaErrorInvalidValue;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (g_noalloc_ptr[dev] == nullptr) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = p;
  }
  float* part_o = g_noalloc_ptr[dev];
  float* part_ml = part_o + (size_t)R * Hq * splits * D;
  return poot_attn_paged(q, q_stride, kpool, vpool, block_tables, max_blocks, row_seq, row_ctx, out, out_stride,
                         part_o, part_ml, R, Hq, Hkv, D, scale, softcap, window, splits, stream);
}
