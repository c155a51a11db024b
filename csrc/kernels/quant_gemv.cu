// Dequant-fused decode GEMV over GGUF block-quantised weights (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K,
// Q6_K, IQ4_NL, IQ4_XS, MXFP4) and packed embedding-row gather:
//     out[m, n] = sum_k x[m, k] * dequant(W)[n, k]          1 <= m <= 4, bf16 activations, fp32 accumulate
// The packed blocks are read once from HBM in their checkpoint layout; decoding happens in registers.  A warp
// walks a weight row 256 values at a time: every lane owns 8 consecutive values, so scale/min lookups are per
// lane and the per-block sums factor as  (d*sc) * sum(q*x) - (dmin*m) * sum(x)  in the ggml product order.
//
// Reference behaviour covered: Contraction::Packed (crates/poot-kernelgen/src/packed/mod.rs:1-7,
// packed/decode_plan.rs), packed row gathers (crates/pootc/kernels/packed/*.rs) and standalone dequant
// (crates/poot-kernelgen/src/packed/kernel.rs:1-5); block layouts crates/poot-quant/src/blocks.rs:174-346.
#include "quant_decode.cuh"

namespace poot {

constexpr int QG_WARPS = 4;
enum { QEPI_STORE = 0, QEPI_F32 = 1, QEPI_RESID = 2, QEPI_SWIGLU = 3 };

template <int FMT, int M, int EPI>
__global__ void __launch_bounds__(QG_WARPS * 32)
quant_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ W, void* __restrict__ out,
                  const __nv_bfloat16* __restrict__ resid, int N, int K, int ldx, int ldo) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * QG_WARPS + warp, nwarps = gridDim.x * QG_WARPS;
  const size_t row_bytes = (size_t)(K / QGeom<FMT>::ELEMS) * QGeom<FMT>::BYTES;
  for (int pair = gwarp; pair * 2 < N; pair += nwarps) {
    const int n0 = pair * 2;
    const uint8_t* r0 = W + (size_t)n0 * row_bytes;
    const uint8_t* r1 = W + (size_t)(n0 + 1 < N ? n0 + 1 : n0) * row_bytes;
    float acc[M][2];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
    for (int k = lane * 8; k < K; k += 256) {
      float q0[8], q1[8], s0, o0, s1, o1;
      decode8<FMT>(r0, k, q0, s0, o0);
      decode8<FMT>(r1, k, q1, s1, o1);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xf[8];
        unpack8(*reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k), xf);
        float d0 = 0.f, d1 = 0.f, sx = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { d0 += q0[i] * xf[i]; d1 += q1[i] * xf[i]; sx += xf[i]; }
        acc[m][0] += s0 * d0 - o0 * sx;
        acc[m][1] += s1 * d1 - o1 * sx;
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m][0] = warp_sum(acc[m][0]); acc[m][1] = warp_sum(acc[m][1]); }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (EPI == QEPI_SWIGLU) {
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + (n0 >> 1)] = __float2bfloat16(silu(acc[m][0]) * acc[m][1]);
        } else {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int n = n0 + r;
            if (n >= N) break;
            float v = acc[m][r];
            if (EPI == QEPI_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
            else {
              if (EPI == QEPI_RESID) v += __bfloat162float(resid[(size_t)m * ldo + n]);
              reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
  }
}

// out[t, :] = dequant(table[ids[t], :]) as bf16   (packed embedding rows)
template <int FMT>
__global__ void quant_row_gather_kernel(const int* __restrict__ ids, const uint8_t* __restrict__ table,
                                        __nv_bfloat16* __restrict__ out, int D, int vocab) {
  pdl_wait(); pdl_launch();
  int id = ids[blockIdx.x];
  if (!POOT_IN_RANGE(id, vocab, kSiteTokenId) || id < 0 || id >= vocab) id = 0;
  const size_t row_bytes = (size_t)(D / QGeom<FMT>::ELEMS) * QGeom<FMT>::BYTES;
  const uint8_t* row = table + (size_t)id * row_bytes;
  for (int k = threadIdx.x * 8; k < D; k += blockDim.x * 8) {
    float q[8], s, o, v[8];
    decode8<FMT>(row, k, q, s, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = s * q[i] - o;
    *reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * D + k) = pack8(v);
  }
}

// Whole-tensor dequantisation to bf16 (formats without a fused GEMM are expanded once at load time).
template <int FMT>
__global__ void quant_dequant_kernel(const uint8_t* __restrict__ W, __nv_bfloat16* __restrict__ out, int N, int K) {
  const size_t row_bytes = (size_t)(K / QGeom<FMT>::ELEMS) * QGeom<FMT>::BYTES;
  const size_t chunks = (size_t)N * (K / 8);
  for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (size_t)gridDim.x * blockDim.x) {
    const size_t n = c / (K / 8);
    const int k = (int)(c - n * (K / 8)) * 8;
    float q[8], s, o, v[8];
    decode8<FMT>(W + n * row_bytes, k, q, s, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = s * q[i] - o;
    *reinterpret_cast<uint4*>(out + n * K + k) = pack8(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Wide-load variants for the two formats of the quantised decode benchmark (Q4_K projections, Q8_0 embeddings).
// One CTA of four warps owns one pair of weight rows and its warps split K; every lane fetches its weight bytes
// with 16-byte streaming loads issued BEFORE the dependency wait (weights do not depend on the previous kernel),
// so a whole row pair is in flight at once.  Integer levels become floats without a convert instruction: a byte
// permute drops the level into the mantissa of a constant (128.0 as bf16<<16 for nibbles, 2^23 for bytes).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float nib_to_f128(uint32_t masked, int i) {   // 128 + nibble (byte i of `masked`)
  return __uint_as_float(__byte_perm(masked, 0x4300u, 0x5044u | (uint32_t)(i << 8)));
}
__device__ __forceinline__ float byte_to_f(uint32_t biased, int i) {     // signed level of byte i (bytes ^ 0x80)
  return __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7440u | (uint32_t)i)) - 8388736.f;
}

template <int M, int EPI>
__device__ __forceinline__ void qg_block_epilogue(float (&acc)[M][2], float (*red)[M][2], void* out,
                                                  const __nv_bfloat16* resid, int n0, int N, int ldo) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < M; ++m) { acc[m][0] = warp_sum(acc[m][0]); acc[m][1] = warp_sum(acc[m][1]); }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < M; ++m) { red[warp][m][0] = acc[m][0]; red[warp][m][1] = acc[m][1]; }
  }
  __syncthreads();
  if (threadIdx.x < M) {
    const int m = threadIdx.x;
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int w = 0; w < QG_WARPS; ++w) { v0 += red[w][m][0]; v1 += red[w][m][1]; }
    if (EPI == QEPI_SWIGLU) {
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + (n0 >> 1)] = __float2bfloat16(silu(v0) * v1);
    } else {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int n = n0 + r;
        if (n >= N) break;
        float v = r ? v1 : v0;
        if (EPI == QEPI_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
        else {
          if (EPI == QEPI_RESID) v += __bfloat162float(resid[(size_t)m * ldo + n]);
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16(v);
        }
      }
    }
  }
}

// Q4_K: a warp pass covers four 144-byte super-blocks of each row; lane = (block of the pass, 16-byte slice of its
// 128 nibble bytes).  Slice `seg` holds values [seg*16 .. +16) of sub-block 2j in its low nibbles and the same
// positions of sub-block 2j+1 in its high nibbles (j = seg / 2).
struct Q4kLane { uint4 head, qs; };
__device__ __forceinline__ void q4k_scales(const uint4& head, int j, float& a0, float& b0, float& a1, float& b1) {
  const float d = h2f((uint16_t)(head.x & 0xFFFF)), dmin = h2f((uint16_t)(head.x >> 16));
  int sc0, sc1, mn0, mn1;
  if (j < 2) {
    const int s = 16 * j;
    sc0 = (head.y >> s) & 63; sc1 = (head.y >> (s + 8)) & 63;
    mn0 = (head.z >> s) & 63; mn1 = (head.z >> (s + 8)) & 63;
  } else {
    const int s = 16 * (j - 2);
    sc0 = ((head.w >> s) & 0xF) | (((head.y >> (s + 6)) & 3) << 4);
    sc1 = ((head.w >> (s + 8)) & 0xF) | (((head.y >> (s + 14)) & 3) << 4);
    mn0 = ((head.w >> (s + 4)) & 0xF) | (((head.z >> (s + 6)) & 3) << 4);
    mn1 = ((head.w >> (s + 12)) & 0xF) | (((head.z >> (s + 14)) & 3) << 4);
  }
  a0 = d * (float)sc0; b0 = dmin * (float)mn0; a1 = d * (float)sc1; b1 = dmin * (float)mn1;
}

template <int M, int EPI>
__global__ void __launch_bounds__(QG_WARPS * 32)
q4k_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ W, void* __restrict__ out,
                const __nv_bfloat16* __restrict__ resid, int N, int K, int ldx, int ldo) {
  __shared__ float red[QG_WARPS][M][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane >> 3, seg = lane & 7, j = seg >> 1;
  const int nblk = K >> 8, n0 = blockIdx.x * 2;
  const size_t row_bytes = (size_t)nblk * 144;
  const uint8_t* r0 = W + (size_t)n0 * row_bytes;
  const uint8_t* r1 = W + (size_t)(n0 + 1 < N ? n0 + 1 : n0) * row_bytes;
  Q4kLane c0, c1;
  int b = warp * 4 + sub;
  if (b < nblk) {
    c0.head = ld_stream16(r0 + (size_t)b * 144); c0.qs = ld_stream16(r0 + (size_t)b * 144 + 16 + seg * 16);
    c1.head = ld_stream16(r1 + (size_t)b * 144); c1.qs = ld_stream16(r1 + (size_t)b * 144 + 16 + seg * 16);
  }
  pdl_wait(); pdl_launch();
  float acc[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
  for (; b - sub < nblk; b += QG_WARPS * 4) {
    const bool live = b < nblk;
    const Q4kLane u0 = c0, u1 = c1;
    const int bn = b + QG_WARPS * 4;
    if (bn < nblk) {   // next pass of this warp: in flight while this one is consumed
      c0.head = ld_stream16(r0 + (size_t)bn * 144); c0.qs = ld_stream16(r0 + (size_t)bn * 144 + 16 + seg * 16);
      c1.head = ld_stream16(r1 + (size_t)bn * 144); c1.qs = ld_stream16(r1 + (size_t)bn * 144 + 16 + seg * 16);
    }
    if (!live) continue;
    float a00, b00, a01, b01, a10, b10, a11, b11;
    q4k_scales(u0.head, j, a00, b00, a01, b01);
    q4k_scales(u1.head, j, a10, b10, a11, b11);
    const uint32_t w0[4] = {u0.qs.x, u0.qs.y, u0.qs.z, u0.qs.w}, w1[4] = {u1.qs.x, u1.qs.y, u1.qs.z, u1.qs.w};
    const int k_lo = b * 256 + j * 64 + (seg & 1) * 16;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const __nv_bfloat16* xp = x + (size_t)m * ldx + k_lo;
      float xl[16], xh[16];
      unpack8(*reinterpret_cast<const uint4*>(xp), xl); unpack8(*reinterpret_cast<const uint4*>(xp + 8), xl + 8);
      unpack8(*reinterpret_cast<const uint4*>(xp + 32), xh); unpack8(*reinterpret_cast<const uint4*>(xp + 40), xh + 8);
      float sxl = 0.f, sxh = 0.f, l0 = 0.f, h0 = 0.f, l1 = 0.f, h1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t lo0 = w0[w] & 0x0F0F0F0Fu, hi0 = (w0[w] >> 4) & 0x0F0F0F0Fu;
        const uint32_t lo1 = w1[w] & 0x0F0F0F0Fu, hi1 = (w1[w] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float xa = xl[w * 4 + i], xb = xh[w * 4 + i];
          sxl += xa; sxh += xb;
          l0 += nib_to_f128(lo0, i) * xa; h0 += nib_to_f128(hi0, i) * xb;
          l1 += nib_to_f128(lo1, i) * xa; h1 += nib_to_f128(hi1, i) * xb;
        }
      }
      // sum((128 + q) x) - 128 sum(x) = sum(q x);  value = a * q - b
      acc[m][0] += a00 * (l0 - 128.f * sxl) - b00 * sxl + a01 * (h0 - 128.f * sxh) - b01 * sxh;
      acc[m][1] += a10 * (l1 - 128.f * sxl) - b10 * sxl + a11 * (h1 - 128.f * sxh) - b11 * sxh;
    }
  }
  qg_block_epilogue<M, EPI>(acc, red, out, resid, n0, N, ldo);
}

// Q8_0: a warp pass covers 32 blocks (1088 bytes) of each row, staged through shared memory because the 34-byte
// blocks are only 2-byte aligned; lane = block of the pass.
template <int M, int EPI>
__global__ void __launch_bounds__(QG_WARPS * 32)
q80_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ W, void* __restrict__ out,
                const __nv_bfloat16* __restrict__ resid, int N, int K, int ldx, int ldo) {
  __shared__ float red[QG_WARPS][M][2];
  __shared__ __align__(16) uint8_t stage[QG_WARPS][2][1088];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nblk = K >> 5, n0 = blockIdx.x * 2;
  const size_t row_bytes = (size_t)nblk * 34;               // K % 256 == 0: a multiple of 16 bytes
  const uint8_t* r0 = W + (size_t)n0 * row_bytes;
  const uint8_t* r1 = W + (size_t)(n0 + 1 < N ? n0 + 1 : n0) * row_bytes;
  const int npass = (nblk + 31) >> 5;
  uint4 f0[3], f1[3];
  auto fetch = [&](int pass) {
    const size_t base = (size_t)pass * 1088;
    const size_t lim = row_bytes - base;                    // bytes left in the row from this pass on (multiple of 16)
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const size_t off = (size_t)(lane + 32 * t) * 16;
      if (off < 1088 && off < lim) { f0[t] = ld_stream16(r0 + base + off); f1[t] = ld_stream16(r1 + base + off); }
    }
  };
  if (warp < npass) fetch(warp);
  pdl_wait(); pdl_launch();
  float acc[M][2];
#pragma unroll
  for (int m = 0; m < M; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }
  for (int pass = warp; pass < npass; pass += QG_WARPS) {
    __syncwarp();
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const int off = (lane + 32 * t) * 16;
      if (off < 1088) {
        *reinterpret_cast<uint4*>(&stage[warp][0][off]) = f0[t];
        *reinterpret_cast<uint4*>(&stage[warp][1][off]) = f1[t];
      }
    }
    __syncwarp();
    if (pass + QG_WARPS < npass) fetch(pass + QG_WARPS);
    const int blk = pass * 32 + lane;
    if (blk < nblk) {
      const uint16_t* s0 = reinterpret_cast<const uint16_t*>(&stage[warp][0][lane * 34]);
      const uint16_t* s1 = reinterpret_cast<const uint16_t*>(&stage[warp][1][lane * 34]);
      const float d0 = h2f(s0[0]), d1 = h2f(s1[0]);
      uint32_t q0[8], q1[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        q0[w] = ((uint32_t)s0[1 + 2 * w] | ((uint32_t)s0[2 + 2 * w] << 16)) ^ 0x80808080u;
        q1[w] = ((uint32_t)s1[1 + 2 * w] | ((uint32_t)s1[2 + 2 * w] << 16)) ^ 0x80808080u;
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const __nv_bfloat16* xp = x + (size_t)m * ldx + (size_t)blk * 32;
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float xf[8];
          unpack8(*reinterpret_cast<const uint4*>(xp + 8 * v), xf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            t0 += byte_to_f(q0[2 * v + (i >> 2)], i & 3) * xf[i];
            t1 += byte_to_f(q1[2 * v + (i >> 2)], i & 3) * xf[i];
          }
        }
        acc[m][0] += d0 * t0; acc[m][1] += d1 * t1;
      }
    }
  }
  qg_block_epilogue<M, EPI>(acc, red, out, resid, n0, N, ldo);
}

template <int FMT, int M, int EPI> struct QKernelFor {
  static constexpr auto fn = quant_gemv_kernel<FMT, M, EPI>;
  static constexpr bool per_pair = false;
};
template <int M, int EPI> struct QKernelFor<QF_Q4_K, M, EPI> {
  static constexpr auto fn = q4k_gemv_kernel<M, EPI>;
  static constexpr bool per_pair = true;
};
template <int M, int EPI> struct QKernelFor<QF_Q8_0, M, EPI> {
  static constexpr auto fn = q80_gemv_kernel<M, EPI>;
  static constexpr bool per_pair = true;
};

template <int FMT, int M>
static int launch_qgemv_m(int epi, const void* x, const void* W, void* out, const void* resid, int N, int K, int ldx,
                          int ldo, cudaStream_t s) {
  if (QKernelFor<FMT, M, QEPI_STORE>::per_pair) {
    dim3 g((N + 1) / 2), b(QG_WARPS * 32);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const uint8_t* wb = (const uint8_t*)W;
    const __nv_bfloat16* rb = (const __nv_bfloat16*)resid;
    switch (epi) {
      case QEPI_STORE: return launch_k(QKernelFor<FMT, M, QEPI_STORE>::fn, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
      case QEPI_F32: return launch_k(QKernelFor<FMT, M, QEPI_F32>::fn, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
      case QEPI_RESID: return launch_k(QKernelFor<FMT, M, QEPI_RESID>::fn, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
      case QEPI_SWIGLU: return launch_k(QKernelFor<FMT, M, QEPI_SWIGLU>::fn, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
      default: return (int)cudaErrorInvalidValue;
    }
  }
  int pairs = (N + 1) / 2, blocks = (pairs + QG_WARPS - 1) / QG_WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  dim3 g(blocks), b(QG_WARPS * 32);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const uint8_t* wb = (const uint8_t*)W;
  const __nv_bfloat16* rb = (const __nv_bfloat16*)resid;
  switch (epi) {
    case QEPI_STORE: return launch_k(quant_gemv_kernel<FMT, M, QEPI_STORE>, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
    case QEPI_F32: return launch_k(quant_gemv_kernel<FMT, M, QEPI_F32>, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
    case QEPI_RESID: return launch_k(quant_gemv_kernel<FMT, M, QEPI_RESID>, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
    case QEPI_SWIGLU: return launch_k(quant_gemv_kernel<FMT, M, QEPI_SWIGLU>, g, b, 0, s, xb, wb, out, rb, N, K, ldx, ldo);
    default: return (int)cudaErrorInvalidValue;
  }
}
template <int FMT>
static int launch_qgemv(int epi, const void* x, const void* W, void* out, const void* resid, int M, int N, int K,
                        int ldx, int ldo, cudaStream_t s) {
  switch (M) {
    case 1: return launch_qgemv_m<FMT, 1>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    case 2: return launch_qgemv_m<FMT, 2>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    case 3: return launch_qgemv_m<FMT, 3>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    case 4: return launch_qgemv_m<FMT, 4>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace poot

using namespace poot;

#define POOT_QDISPATCH(fmt, CALL)                                   \
  switch (fmt) {                                                    \
    case QF_Q4_K: return CALL(QF_Q4_K);                             \
    case QF_Q5_K: return CALL(QF_Q5_K);                             \
    case QF_Q6_K: return CALL(QF_Q6_K);                             \
    case QF_Q8_0: return CALL(QF_Q8_0);                             \
    case QF_Q4_0: return CALL(QF_Q4_0);                             \
    case QF_Q4_1: return CALL(QF_Q4_1);                             \
    case QF_Q5_0: return CALL(QF_Q5_0);                             \
    case QF_Q5_1: return CALL(QF_Q5_1);                             \
    case QF_IQ4_NL: return CALL(QF_IQ4_NL);                         \
    case QF_MXFP4: return CALL(QF_MXFP4);                           \
    case QF_Q2_K: return CALL(QF_Q2_K);                             \
    case QF_Q3_K: return CALL(QF_Q3_K);                             \
    case QF_IQ4_XS: return CALL(QF_IQ4_XS);                         \
    default: return (int)cudaErrorInvalidValue;                     \
  }

// fmt = ggml type id (see QFmt).  x [M, ldx] bf16, W packed [N rows of K values].
POOT_API int poot_quant_gemv(int fmt, int epi, const void* x, const void* W, void* out, const void* resid, int M, int N,
                             int K, int ldx, int ldo, cudaStream_t s) {
  if (K % 256 || ldx % 8 || M < 1 || M > 4) return (int)cudaErrorInvalidValue;
  if (epi == QEPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
#define CALL(F) launch_qgemv<F>(epi, x, W, out, resid, M, N, K, ldx, ldo, s)
  POOT_QDISPATCH(fmt, CALL)
#undef CALL
}

// Host build of the block decoders the kernels run: values [k, k + 8) of one packed row as scale * q - offset.
// Needs no GPU; returns 0, or cudaErrorInvalidValue for an unknown format or a k that is not a multiple of 8.
POOT_API int poot_quant_decode8_host(int fmt, const void* row, int k, float* out8) {
  if (k % 8) return (int)cudaErrorInvalidValue;
  float q[8], s, o;
#define CALL(F) (decode8<F>((const uint8_t*)row, k, q, s, o), 0)
  int r = [&]() -> int { POOT_QDISPATCH(fmt, CALL) }();
#undef CALL
  if (r) return r;
  for (int i = 0; i < 8; ++i) out8[i] = s * q[i] - o;
  return 0;
}

POOT_API int poot_quant_row_gather(int fmt, const int* ids, const void* table, void* out, int T, int D, int vocab,
                                   cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 256) return (int)cudaErrorInvalidValue;
#define CALL(F) launch_k(quant_row_gather_kernel<F>, dim3(T), dim3(128), 0, s, ids, (const uint8_t*)table, (__nv_bfloat16*)out, D, vocab)
  POOT_QDISPATCH(fmt, CALL)
#undef CALL
}

POOT_API int poot_quant_dequant_bf16(int fmt, const void* W, void* out, int N, int K, cudaStream_t s) {
  if (K % 256) return (int)cudaErrorInvalidValue;
  long long chunks = (long long)N * (K / 8);
  int blocks = (int)((chunks + 255) / 256 > 148 * 16 ? 148 * 16 : (chunks + 255) / 256);
  if (blocks < 1) return 0;
#define CALL(F) (quant_dequant_kernel<F><<<blocks, 256, 0, s>>>((const uint8_t*)W, (__nv_bfloat16*)out, N, K), (int)cudaGetLastError())
  POOT_QDISPATCH(fmt, CALL)
#undef CALL
}
