// Dequant-fused kernels for the planar (safetensors) quantised formats: the weight stays in its checkpoint tensors
// (codes, scales, zero points each a tensor of its own) and is decoded inside the matrix-vector product.
//
//   fmt 0  E4M3_CHANNEL   weight [N, K] fp8 e4m3, scale [N] f32                       w = dec(code) * scale[n]
//   fmt 1  E4M3_BLOCK128  weight [N, K] fp8 e4m3, scale [ceil(N/128), ceil(K/128)]    w = dec(code) * scale[n/128][k/128]
//   fmt 2  E2M1_ROW32     weight [N, K/2] two fp4 e2m1 per byte (low nibble first),
//                         scale [N, K/32] e8m0                                       w = e2m1(code) * 2^(scale - 127)
//   fmt 3  GPTQ           qweight [K/8, N] int32 (eight k per word), qzeros [K/g, N/8] int32 (stored zero - 1),
//                         scales [K/g, N] f32, optional g_idx [K]                    w = (q - (z + 1)) * s
//   fmt 4  AWQ            qweight [K, N/8] int32 (eight n per word, nibble i holds column [0,4,1,5,2,6,3,7][i]),
//                         qzeros [K/g, N/8] same order, scales [K/g, N] f32          w = (q - z) * s
//
// planar_gemv: y[m, n] = sum_k x[m, k] * w[n, k] for m < M <= 4 (decode), epilogues store / f32 / residual.
// planar_dequant: the whole weight as bf16 [N, K] (larger steps multiply with the tiled GEMM over it).
// planar_gemv_grouped: routed experts that stay packed (formats 0-2): one activation row per group against the
// group's expert of a stack, optionally the gated activation of two stacks, biases and a per-group scale fused.
// Row-major formats (0-2) take one warp per output row; the K-major int4 formats (3, 4) take one thread per output
// column (GPTQ) or per word of eight columns (AWQ) with the K range cut over the warps of the CTA and summed in shared
// memory in a fixed order, so results do not depend on scheduling.
#include "common.cuh"

namespace poot {

enum PlanarFmt { PF_E4M3_CHANNEL = 0, PF_E4M3_BLOCK128 = 1, PF_E2M1_ROW32 = 2, PF_GPTQ = 3, PF_AWQ = 4 };
enum PlanarEpi { PEPI_STORE = 0, PEPI_F32 = 1, PEPI_RESID = 2 };
constexpr int PG_MAX_M = 4;

struct PlanarOps {
  const void* w;          // codes
  const void* scale;      // f32 (formats 0, 1, 3, 4) or e8m0 bytes (format 2)
  const void* zeros;      // int32 words (formats 3, 4)
  const int* g_idx;       // GPTQ act-order group of every k, or null (k / group)
  int group;              // int4 group size along K
};

__host__ __device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
  const uint32_t s = (c & 0x80u) << 24, e = (c >> 3) & 0xFu, m = c & 7u;
  if (e == 0u) {
    const float v = (float)m * 0.001953125f;                 // subnormal: m * 2^-9
#ifdef __CUDA_ARCH__
    return __uint_as_float(__float_as_uint(v) | s);
#else
    return s ? -v : v;
#endif
  }
  if (e == 15u && m == 7u) c = 0x7FC00000u;                   // NaN (the FN format has no infinity)
  else c = s | ((e + 120u) << 23) | (m << 20);
#ifdef __CUDA_ARCH__
  return __uint_as_float(c);
#else
  float f;
  memcpy(&f, &c, 4);
  return f;
#endif
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6 with the sign in bit 3
  const uint32_t m = c & 7u;
  const float v = m < 2u ? 0.5f * (float)m : (float)(2u + (m & 1u)) * (float)(1u << ((m >> 1) - 1u)) * 0.5f;
  return (c & 8u) ? -v : v;
}

__device__ __forceinline__ float e8m0_to_f32(uint32_t e) { return e == 255u ? __uint_as_float(0x7FC00000u) : exp2f((float)e - 127.f); }

__device__ __forceinline__ void store_epi(int epi, void* out, const void* resid, int ldo, int m, int n, float v) {
  const size_t o = (size_t)m * ldo + n;
  if (epi == PEPI_F32) { reinterpret_cast<float*>(out)[o] = v; return; }
  if (epi == PEPI_RESID) v += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(resid)[o]);
  reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16(v);
}

// ---- row-major formats: one warp per output row -------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256)
planar_gemv_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx, PlanarOps ops, void* out, const void* resid, int ldo,
                        int epi, int M, int N, int K) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  float acc[PG_MAX_M] = {0.f, 0.f, 0.f, 0.f};
  if (FMT == PF_E2M1_ROW32) {
    const uint8_t* wr = reinterpret_cast<const uint8_t*>(ops.w) + (size_t)n * (K / 2);
    const uint8_t* sr = reinterpret_cast<const uint8_t*>(ops.scale) + (size_t)n * (K / 32);
    for (int b = lane; b < K / 32; b += 32) {                 // one block of 32 values (16 bytes) per lane and turn
      const float s = e8m0_to_f32(sr[b]);
      const uint4 pk = *reinterpret_cast<const uint4*>(wr + (size_t)b * 16);
      const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float wv = e2m1_to_f32((wd[i >> 3] >> (4 * (i & 7))) & 0xFu) * s;
#pragma unroll
        for (int m = 0; m < PG_MAX_M; ++m)
          if (m < M) acc[m] += wv * __bfloat162float(x[(size_t)m * ldx + b * 32 + i]);
      }
    }
  } else {
    const uint8_t* wr = reinterpret_cast<const uint8_t*>(ops.w) + (size_t)n * K;
    const float* sc = reinterpret_cast<const float*>(ops.scale);
    const int kb = (K + 127) / 128;
    const float row_scale = FMT == PF_E4M3_CHANNEL ? sc[n] : 1.f;
    for (int k0 = lane * 16; k0 < K; k0 += 32 * 16) {         // K is a multiple of 16: one 16-byte load per lane and turn
      const uint4 pk = *reinterpret_cast<const uint4*>(wr + k0);
      const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
      const float s = FMT == PF_E4M3_BLOCK128 ? sc[(size_t)(n >> 7) * kb + (k0 >> 7)] : row_scale;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float wv = e4m3_to_f32((wd[i >> 2] >> (8 * (i & 3))) & 0xFFu) * s;
#pragma unroll
        for (int m = 0; m < PG_MAX_M; ++m)
          if (m < M) acc[m] += wv * __bfloat162float(x[(size_t)m * ldx + k0 + i]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < PG_MAX_M; ++m) {
    if (m >= M) break;
    const float v = warp_sum(acc[m]);
    if (lane == 0) store_epi(epi, out, resid, ldo, m, n, v);
  }
}

// ---- routed experts kept packed: one activation row per group, the group's expert read from stacked operands -------------
// Group g multiplies activation row g / x_row_div (x_row_div > 0) or g with expert ids[g] (or g) of weights stacked as
// [E, N, ...] per operand.  One warp per (group, output row).  With a second weight set the warp computes the gate row
// and the up row of the same index and writes act(gate + b1, up + b2):
//   act 1: silu(gate) * up          act 2: (clamp(up, -limit, limit) + 1) * g * sigmoid(alpha * g), g = min(gate, limit)
// without one it writes (w x + b) * row_scale[g].  Biases are f32 [E, N].  A negative expert id leaves the group's row zero.
struct GroupedOps {
  const uint8_t* w;  const uint8_t* scale;       // gate (or the only) weight set
  const uint8_t* w2; const uint8_t* scale2;      // up weight set, or null
  const float* bias; const float* bias2;
  size_t w_stride, scale_stride;                 // bytes per expert
};

template <int FMT>
__device__ __forceinline__ float packed_row_dot(const uint8_t* wbase, const uint8_t* sbase, int n, int N, int K,
                                                const __nv_bfloat16* __restrict__ xr, int lane) {
  float acc = 0.f;
  if (FMT == PF_E2M1_ROW32) {
    const uint8_t* wr = wbase + (size_t)n * (K / 2);
    const uint8_t* sr = sbase + (size_t)n * (K / 32);
    for (int b = lane; b < K / 32; b += 32) {
      const float s = e8m0_to_f32(sr[b]);
      const uint4 pk = *reinterpret_cast<const uint4*>(wr + (size_t)b * 16);
      const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        part += e2m1_to_f32((wd[i >> 3] >> (4 * (i & 7))) & 0xFu) * __bfloat162float(xr[b * 32 + i]);
      acc += part * s;
    }
  } else {
    const uint8_t* wr = wbase + (size_t)n * K;
    const float* sc = reinterpret_cast<const float*>(sbase);
    const int kb = (K + 127) / 128;
    const float row_scale = FMT == PF_E4M3_CHANNEL ? sc[n] : 1.f;
    for (int k0 = lane * 16; k0 < K; k0 += 32 * 16) {
      const uint4 pk = *reinterpret_cast<const uint4*>(wr + k0);
      const uint32_t wd[4] = {pk.x, pk.y, pk.z, pk.w};
      const float s = FMT == PF_E4M3_BLOCK128 ? sc[(size_t)(n >> 7) * kb + (k0 >> 7)] : row_scale;
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        part += e4m3_to_f32((wd[i >> 2] >> (8 * (i & 3))) & 0xFFu) * __bfloat162float(xr[k0 + i]);
      acc += part * s;
    }
  }
  return warp_sum(acc);
}

template <int FMT>
__global__ void __launch_bounds__(256)
planar_gemv_grouped_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int x_row_div, GroupedOps ops, int act, float alpha,
                           float limit, const int* __restrict__ ids, const float* __restrict__ row_scale,
                           __nv_bfloat16* __restrict__ out, int ldo, int E, int N, int K) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int g = blockIdx.y;
  if (n >= N) return;
  const int e = ids ? ids[g] : g;
  if (e < 0 || e >= E) {                      // an unused slot (or an id outside the stack): the row reads as zero
    if (lane == 0) out[(size_t)g * ldo + n] = __float2bfloat16(0.f);
    return;
  }
  const __nv_bfloat16* xr = x + (size_t)(x_row_div > 0 ? g / x_row_div : g) * ldx;
  float v = packed_row_dot<FMT>(ops.w + (size_t)e * ops.w_stride, ops.scale + (size_t)e * ops.scale_stride, n, N, K, xr, lane);
  if (ops.bias) v += ops.bias[(size_t)e * N + n];
  if (ops.w2) {
    float u = packed_row_dot<FMT>(ops.w2 + (size_t)e * ops.w_stride, ops.scale2 + (size_t)e * ops.scale_stride, n, N, K, xr, lane);
    if (ops.bias2) u += ops.bias2[(size_t)e * N + n];
    if (act == 2) {
      const float gt = fminf(v, limit);
      u = fminf(fmaxf(u, -limit), limit);
      v = (u + 1.f) * gt / (1.f + __expf(-alpha * gt));
    } else {
      v = silu(v) * u;
    }
  }
  if (row_scale) v *= row_scale[g];
  if (lane == 0) out[(size_t)g * ldo + n] = __float2bfloat16(v);
}

// ---- K-major int4 formats -------------------------------------------------------------------------------------------
// CTA: 64 column slots x 4 K-slices (256 threads).  GPTQ: a slot is one output column.  AWQ: a slot is one word of
// eight columns.  Slice s covers k in [s * K / 4, (s + 1) * K / 4) (a multiple of 8); partial sums meet in shared memory.
constexpr int PI_SLOTS = 64, PI_SLICES = 4;
// nibble i of an AWQ word holds column [0, 4, 1, 5, 2, 6, 3, 7][i] of its eight
__host__ __device__ constexpr int awq_col(int i) { return (int)((0x73625140u >> (4 * i)) & 0xFu); }

template <int FMT>
__global__ void __launch_bounds__(PI_SLOTS * PI_SLICES)
planar_gemv_int4_kernel(const __nv_bfloat16* __restrict__ x, int ldx, PlanarOps ops, void* out, const void* resid, int ldo,
                        int epi, int M, int N, int K) {
  constexpr int COLS = FMT == PF_AWQ ? 8 : 1;
  __shared__ float part[PI_SLICES][PI_SLOTS][COLS * PG_MAX_M];
  pdl_wait(); pdl_launch();
  const int slot = threadIdx.x % PI_SLOTS, slice = threadIdx.x / PI_SLOTS;
  const int unit = blockIdx.x * PI_SLOTS + slot;             // column (GPTQ) or word of eight columns (AWQ)
  const int units = N / COLS;
  const int klen = (K / PI_SLICES) & ~7;
  const int k_begin = slice * klen, k_end = slice == PI_SLICES - 1 ? K : k_begin + klen;
  float acc[COLS * PG_MAX_M];
#pragma unroll
  for (int i = 0; i < COLS * PG_MAX_M; ++i) acc[i] = 0.f;
  const uint32_t* qw = reinterpret_cast<const uint32_t*>(ops.w);
  const uint32_t* qz = reinterpret_cast<const uint32_t*>(ops.zeros);
  const float* sc = reinterpret_cast<const float*>(ops.scale);
  if (unit < units) {
    if (FMT == PF_GPTQ) {
      const int n = unit;
      int g_prev = -1;
      float s = 0.f, z = 0.f;
      for (int k8 = k_begin / 8; k8 < k_end / 8; ++k8) {
        const uint32_t word = qw[(size_t)k8 * N + n];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int k = k8 * 8 + i;
          const int g = ops.g_idx ? ops.g_idx[k] : k / ops.group;
          if (g != g_prev) {
            g_prev = g;
            s = sc[(size_t)g * N + n];
            z = (float)(((qz[(size_t)g * (N / 8) + (n >> 3)] >> (4 * (n & 7))) & 0xFu) + 1u);
          }
          const float wv = ((float)((word >> (4 * i)) & 0xFu) - z) * s;
#pragma unroll
          for (int m = 0; m < PG_MAX_M; ++m)
            if (m < M) acc[m] += wv * __bfloat162float(x[(size_t)m * ldx + k]);
        }
      }
    } else {
      const int w8 = unit;
      int g_prev = -1;
      float s[8], z[8];
      for (int k = k_begin; k < k_end; ++k) {
        const int g = k / ops.group;
        if (g != g_prev) {
          g_prev = g;
          const uint32_t zw = qz[(size_t)g * units + w8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            s[awq_col(i)] = sc[(size_t)g * N + w8 * 8 + awq_col(i)];
            z[awq_col(i)] = (float)((zw >> (4 * i)) & 0xFu);
          }
        }
        const uint32_t word = qw[(size_t)k * units + w8];
        float xv[PG_MAX_M];
#pragma unroll
        for (int m = 0; m < PG_MAX_M; ++m) xv[m] = m < M ? __bfloat162float(x[(size_t)m * ldx + k]) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = awq_col(i);
          const float wv = ((float)((word >> (4 * i)) & 0xFu) - z[c]) * s[c];
#pragma unroll
          for (int m = 0; m < PG_MAX_M; ++m) acc[c * PG_MAX_M + m] += wv * xv[m];
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < COLS * PG_MAX_M; ++i) part[slice][slot][i] = acc[i];
  __syncthreads();
  if (slice != 0 || unit >= units) return;
#pragma unroll
  for (int c = 0; c < COLS; ++c)
#pragma unroll
    for (int m = 0; m < PG_MAX_M; ++m) {
      if (m >= M) break;
      float v = 0.f;
      for (int sl = 0; sl < PI_SLICES; ++sl) v += part[sl][slot][c * PG_MAX_M + m];
      store_epi(epi, out, resid, ldo, m, unit * COLS + c, v);
    }
}

// ---- whole-weight decode to bf16 [N, K] -----------------------------------------------------------------------------
template <int FMT>
__global__ void planar_dequant_kernel(PlanarOps ops, __nv_bfloat16* __restrict__ out, int N, int K) {
  pdl_wait(); pdl_launch();
  const size_t total = (size_t)N * K;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(i / K), k = (int)(i - (size_t)n * K);
    float v;
    if (FMT == PF_E4M3_CHANNEL) {
      v = e4m3_to_f32(reinterpret_cast<const uint8_t*>(ops.w)[i]) * reinterpret_cast<const float*>(ops.scale)[n];
    } else if (FMT == PF_E4M3_BLOCK128) {
      const int kb = (K + 127) / 128;
      v = e4m3_to_f32(reinterpret_cast<const uint8_t*>(ops.w)[i]) *
          reinterpret_cast<const float*>(ops.scale)[(size_t)(n >> 7) * kb + (k >> 7)];
    } else if (FMT == PF_E2M1_ROW32) {
      const uint32_t byte = reinterpret_cast<const uint8_t*>(ops.w)[(size_t)n * (K / 2) + (k >> 1)];
      v = e2m1_to_f32((byte >> (4 * (k & 1))) & 0xFu) *
          e8m0_to_f32(reinterpret_cast<const uint8_t*>(ops.scale)[(size_t)n * (K / 32) + (k >> 5)]);
    } else if (FMT == PF_GPTQ) {
      const int g = ops.g_idx ? ops.g_idx[k] : k / ops.group;
      const uint32_t q = (reinterpret_cast<const uint32_t*>(ops.w)[(size_t)(k >> 3) * N + n] >> (4 * (k & 7))) & 0xFu;
      const uint32_t z = ((reinterpret_cast<const uint32_t*>(ops.zeros)[(size_t)g * (N / 8) + (n >> 3)] >> (4 * (n & 7))) & 0xFu) + 1u;
      v = ((float)q - (float)z) * reinterpret_cast<const float*>(ops.scale)[(size_t)g * N + n];
    } else {
      const int g = k / ops.group, w8 = n >> 3, c = n & 7;
      int nib = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (awq_col(j) == c) nib = j;
      const uint32_t q = (reinterpret_cast<const uint32_t*>(ops.w)[(size_t)k * (N / 8) + w8] >> (4 * nib)) & 0xFu;
      const uint32_t z = (reinterpret_cast<const uint32_t*>(ops.zeros)[(size_t)g * (N / 8) + w8] >> (4 * nib)) & 0xFu;
      v = ((float)q - (float)z) * reinterpret_cast<const float*>(ops.scale)[(size_t)g * N + n];
    }
    out[i] = __float2bfloat16(v);
  }
}

static int planar_check(int fmt, const PlanarOps& ops, int N, int K) {
  if (fmt < 0 || fmt > 4 || N < 1 || K < 1 || ops.w == nullptr || ops.scale == nullptr) return (int)cudaErrorInvalidValue;
  if ((fmt == PF_E4M3_CHANNEL || fmt == PF_E4M3_BLOCK128) && (K % 16 || (reinterpret_cast<uintptr_t>(ops.w) & 15)))
    return (int)cudaErrorInvalidValue;
  if (fmt == PF_E2M1_ROW32 && (K % 32 || (reinterpret_cast<uintptr_t>(ops.w) & 15))) return (int)cudaErrorInvalidValue;
  if (fmt == PF_GPTQ || fmt == PF_AWQ) {
    if (ops.zeros == nullptr || ops.group < 8 || ops.group % 8 || K % ops.group || N % 8 || K % 32) return (int)cudaErrorInvalidValue;
    if (fmt == PF_AWQ && ops.g_idx != nullptr) return (int)cudaErrorInvalidValue;
  }
  return 0;
}

}  // namespace poot

using namespace poot;

POOT_API int poot_planar_gemv(int fmt, int epi, const void* x, int ldx, const void* w, const void* scale, const void* zeros,
                              const int* g_idx, int group, void* out, const void* resid, int ldo, int M, int N, int K,
                              cudaStream_t s) {
  if (M == 0) return 0;
  PlanarOps ops{w, scale, zeros, g_idx, group};
  int e = planar_check(fmt, ops, N, K);
  if (e) return e;
  if (M < 1 || M > PG_MAX_M || epi < 0 || epi > 2 || (epi == PEPI_RESID && resid == nullptr)) return (int)cudaErrorInvalidValue;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
#define ROWS(F) launch_k(planar_gemv_rows_kernel<F>, dim3((N + 7) / 8), dim3(256), 0, s, xb, ldx, ops, out, resid, ldo, epi, M, N, K)
#define INT4(F, COLS) launch_k(planar_gemv_int4_kernel<F>, dim3((N / COLS + PI_SLOTS - 1) / PI_SLOTS), dim3(PI_SLOTS * PI_SLICES), 0, s, xb, ldx, ops, out, resid, ldo, epi, M, N, K)
  switch (fmt) {
    case PF_E4M3_CHANNEL: return ROWS(PF_E4M3_CHANNEL);
    case PF_E4M3_BLOCK128: return ROWS(PF_E4M3_BLOCK128);
    case PF_E2M1_ROW32: return ROWS(PF_E2M1_ROW32);
    case PF_GPTQ: return INT4(PF_GPTQ, 1);
    default: return INT4(PF_AWQ, 8);
  }
#undef ROWS
#undef INT4
}

POOT_API int poot_planar_gemv_grouped(int fmt, const void* x, int ldx, int x_row_div, const void* w, const void* scale, const void* w2,
                                      const void* scale2, const float* bias, const float* bias2, int act, float alpha, float limit,
                                      const int* ids, const float* row_scale, void* out, int ldo, int groups, int E, int N, int K,
                                      cudaStream_t s) {
  if (groups == 0) return 0;
  if (fmt < PF_E4M3_CHANNEL || fmt > PF_E2M1_ROW32 || w == nullptr || scale == nullptr || (w2 != nullptr) != (scale2 != nullptr))
    return (int)cudaErrorInvalidValue;
  if (N < 1 || E < 1 || x_row_div < 0 || (fmt == PF_E2M1_ROW32 ? K % 32 : K % 16) || (w2 != nullptr && (act < 1 || act > 2)) ||
      (w2 == nullptr && bias2 != nullptr) || groups > 65535)
    return (int)cudaErrorInvalidValue;
  GroupedOps ops{(const uint8_t*)w, (const uint8_t*)scale, (const uint8_t*)w2, (const uint8_t*)scale2, bias, bias2, 0, 0};
  const size_t kb = (size_t)(K + 127) / 128, nb = (size_t)(N + 127) / 128;
  ops.w_stride = fmt == PF_E2M1_ROW32 ? (size_t)N * (K / 2) : (size_t)N * K;
  ops.scale_stride = fmt == PF_E2M1_ROW32 ? (size_t)N * (K / 32) : fmt == PF_E4M3_CHANNEL ? (size_t)N * 4 : nb * kb * 4;
  const dim3 grid((N + 7) / 8, groups), block(256);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
#define GR(F) launch_k(planar_gemv_grouped_kernel<F>, grid, block, 0, s, xb, ldx, x_row_div, ops, act, alpha, limit, ids, row_scale, (__nv_bfloat16*)out, ldo, E, N, K)
  switch (fmt) {
    case PF_E4M3_CHANNEL: return GR(PF_E4M3_CHANNEL);
    case PF_E4M3_BLOCK128: return GR(PF_E4M3_BLOCK128);
    default: return GR(PF_E2M1_ROW32);
  }
#undef GR
}

POOT_API int poot_planar_dequant(int fmt, const void* w, const void* scale, const void* zeros, const int* g_idx, int group,
                                 void* out, int N, int K, cudaStream_t s) {
  PlanarOps ops{w, scale, zeros, g_idx, group};
  int e = planar_check(fmt, ops, N, K);
  if (e) return e;
  size_t total = (size_t)N * K;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 32) blocks = 148 * 32;
#define DQ(F) launch_k(planar_dequant_kernel<F>, dim3(blocks), dim3(256), 0, s, ops, (__nv_bfloat16*)out, N, K)
  switch (fmt) {
    case PF_E4M3_CHANNEL: return DQ(PF_E4M3_CHANNEL);
    case PF_E4M3_BLOCK128: return DQ(PF_E4M3_BLOCK128);
    case PF_E2M1_ROW32: return DQ(PF_E2M1_ROW32);
    case PF_GPTQ: return DQ(PF_GPTQ);
    default: return DQ(PF_AWQ);
  }
#undef DQ
}

// Host check of the fp8 decoder against the table the host codec uses: out[256] = every code's value.
POOT_API void poot_planar_e4m3_table(float* out256) {
  for (uint32_t c = 0; c < 256; ++c) out256[c] = e4m3_to_f32(c);
}
