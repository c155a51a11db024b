// Block decoders of the GGUF quantised formats (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL,
// IQ4_XS, MXFP4), shared by the dequant-fused GEMV, the row gather, the whole-tensor decode and the dequant-fused
// skinny GEMM.  Block layouts: crates/poot-quant/src/blocks.rs:174-346.
#pragma once
#include "common.cuh"
#include <cstring>

namespace poot {

// The block decoders are host-and-device code: the same source that the kernels run is exported for the host
// (poot_quant_decode8_host), so its index arithmetic can be checked against the host codec without a GPU.
#define POOT_HD __host__ __device__ __forceinline__
POOT_HD float bits_to_f32(uint32_t u) {
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  float f; memcpy(&f, &u, 4); return f;
#endif
}
POOT_HD float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
POOT_HD uint16_t ld16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
// ggml type ids
enum QFmt { QF_Q4_0 = 2, QF_Q4_1 = 3, QF_Q5_0 = 6, QF_Q5_1 = 7, QF_Q8_0 = 8, QF_Q2_K = 10, QF_Q3_K = 11, QF_Q4_K = 12,
            QF_Q5_K = 13, QF_Q6_K = 14, QF_IQ4_NL = 20, QF_IQ4_XS = 23, QF_MXFP4 = 39 };

// Non-uniform 4-bit code books (format constants of the GGUF block types).
#define POOT_IQ4NL_VALUES {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f, 1.f, 13.f, 25.f, 38.f, 53.f, 69.f, 89.f, 113.f}
#define POOT_MXFP4_VALUES {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f, 0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f}
static __constant__ float kIq4nlF[16] = POOT_IQ4NL_VALUES;
static __constant__ float kMxfp4F[16] = POOT_MXFP4_VALUES;
static const float kIq4nlHost[16] = POOT_IQ4NL_VALUES;
static const float kMxfp4Host[16] = POOT_MXFP4_VALUES;
POOT_HD float iq4nl_value(uint32_t nib) {
#ifdef __CUDA_ARCH__
  return kIq4nlF[nib];
#else
  return kIq4nlHost[nib];
#endif
}
POOT_HD float mxfp4_value(uint32_t nib) {
#ifdef __CUDA_ARCH__
  return kMxfp4F[nib];
#else
  return kMxfp4Host[nib];
#endif
}

// 2^(e - 127) / 2: the scale of an MXFP4 block (its code book stores doubled magnitudes)
POOT_HD float e8m0_half(uint32_t e) { return bits_to_f32(e < 2u ? (0x00200000u << e) : ((e - 1u) << 23)); }
// 8 bytes from an address with no alignment guarantee
POOT_HD void ld8_a1(const uint8_t* p, uint32_t& lo, uint32_t& hi) {
  lo = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
  hi = (uint32_t)p[4] | ((uint32_t)p[5] << 8) | ((uint32_t)p[6] << 16) | ((uint32_t)p[7] << 24);
}

// 8 bytes from a 2-byte aligned address
POOT_HD void ld8_a2(const uint8_t* p, uint32_t& lo, uint32_t& hi) {
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  lo = (uint32_t)q[0] | ((uint32_t)q[1] << 16);
  hi = (uint32_t)q[2] | ((uint32_t)q[3] << 16);
}
POOT_HD void scale_min_k4(int j, const uint8_t* q, int& d, int& m) {
  if (j < 4) { d = q[j] & 63; m = q[j + 4] & 63; }
  else { d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

template <int FMT> struct QGeom;
template <> struct QGeom<QF_Q4_K> { static constexpr int BYTES = 144, ELEMS = 256; };
template <> struct QGeom<QF_Q5_K> { static constexpr int BYTES = 176, ELEMS = 256; };
template <> struct QGeom<QF_Q6_K> { static constexpr int BYTES = 210, ELEMS = 256; };
template <> struct QGeom<QF_Q8_0> { static constexpr int BYTES = 34, ELEMS = 32; };
template <> struct QGeom<QF_Q4_0> { static constexpr int BYTES = 18, ELEMS = 32; };
template <> struct QGeom<QF_Q4_1> { static constexpr int BYTES = 20, ELEMS = 32; };
template <> struct QGeom<QF_Q5_0> { static constexpr int BYTES = 22, ELEMS = 32; };
template <> struct QGeom<QF_Q5_1> { static constexpr int BYTES = 24, ELEMS = 32; };
template <> struct QGeom<QF_IQ4_NL> { static constexpr int BYTES = 18, ELEMS = 32; };
template <> struct QGeom<QF_MXFP4> { static constexpr int BYTES = 17, ELEMS = 32; };
template <> struct QGeom<QF_Q2_K> { static constexpr int BYTES = 84, ELEMS = 256; };
template <> struct QGeom<QF_Q3_K> { static constexpr int BYTES = 110, ELEMS = 256; };
template <> struct QGeom<QF_IQ4_XS> { static constexpr int BYTES = 136, ELEMS = 256; };

// Decode the 8 consecutive values [k, k+8) of a packed row (k a multiple of 8) as
//   value_i = scale * q[i] - offset      (offset = 0 for the symmetric formats)
template <int FMT>
POOT_HD void decode8(const uint8_t* row, int k, float* q, float& scale, float& offset) {
  if (FMT == QF_Q4_K || FMT == QF_Q5_K) {
    const uint8_t* b = row + (size_t)(k >> 8) * QGeom<FMT>::BYTES;
    const int e = k & 255, sub = e >> 5, j = sub >> 1, h = sub & 1, l = e & 31;
    const uint4 head = *reinterpret_cast<const uint4*>(b);          // d, dmin, 12 scale bytes
    const uint8_t* hb = reinterpret_cast<const uint8_t*>(&head);
    int sc, mn;
    scale_min_k4(sub, hb + 4, sc, mn);
    scale = h2f((uint16_t)(head.x & 0xFFFF)) * (float)sc;
    offset = h2f((uint16_t)(head.x >> 16)) * (float)mn;
    const int ql_off = (FMT == QF_Q4_K ? 16 : 48) + j * 32 + l;
    const uint2 w = *reinterpret_cast<const uint2*>(b + ql_off);
    const uint32_t lo = h ? (w.x >> 4) : w.x, hi = h ? (w.y >> 4) : w.y;
    uint32_t hx = 0, hy = 0;
    if (FMT == QF_Q5_K) {
      const uint2 qh = *reinterpret_cast<const uint2*>(b + 16 + l);
      hx = (qh.x >> sub) & 0x01010101u; hy = (qh.y >> sub) & 0x01010101u;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = (float)(((lo >> (8 * i)) & 0xF) | (((hx >> (8 * i)) & 1) << 4));
      q[4 + i] = (float)(((hi >> (8 * i)) & 0xF) | (((hy >> (8 * i)) & 1) << 4));
    }
  } else if (FMT == QF_Q6_K) {
    const uint8_t* b = row + (size_t)(k >> 8) * 210;
    const int e = k & 255, n = e >> 7, g = (e >> 5) & 3, l = e & 31;
    uint32_t lx, ly, hx, hy;
    ld8_a2(b + n * 64 + (g & 1) * 32 + l, lx, ly);
    ld8_a2(b + 128 + n * 32 + l, hx, hy);
    if (g >= 2) { lx >>= 4; ly >>= 4; }
    hx >>= 2 * g; hy >>= 2 * g;
    const int8_t sc = (int8_t)b[192 + n * 8 + (l >> 4) + 2 * g];
    scale = h2f(ld16(b + 208)) * (float)sc;
    offset = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = (float)((int)(((lx >> (8 * i)) & 0xF) | (((hx >> (8 * i)) & 3) << 4)) - 32);
      q[4 + i] = (float)((int)(((ly >> (8 * i)) & 0xF) | (((hy >> (8 * i)) & 3) << 4)) - 32);
    }
  } else if (FMT == QF_Q8_0) {
    const uint8_t* b = row + (size_t)(k >> 5) * 34;
    uint32_t lo, hi;
    ld8_a2(b + 2 + (k & 31), lo, hi);
    scale = h2f(ld16(b)); offset = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = (float)(int8_t)(lo >> (8 * i));
      q[4 + i] = (float)(int8_t)(hi >> (8 * i));
    }
  } else if (FMT == QF_Q4_1 || FMT == QF_Q5_0 || FMT == QF_Q5_1 || FMT == QF_IQ4_NL || FMT == QF_MXFP4) {
    // 32-value blocks whose values 0..15 are the low nibbles of qs[0..15] and 16..31 the high nibbles
    const uint8_t* b = row + (size_t)(k >> 5) * QGeom<FMT>::BYTES;
    const int e = k & 31, j0 = e & 15;
    const int qs_off = FMT == QF_Q4_1 ? 4 : FMT == QF_Q5_0 ? 6 : FMT == QF_Q5_1 ? 8 : FMT == QF_IQ4_NL ? 2 : 1;
    uint32_t lo, hi;
    if (FMT == QF_MXFP4) ld8_a1(b + qs_off + j0, lo, hi); else ld8_a2(b + qs_off + j0, lo, hi);
    if (e >= 16) { lo >>= 4; hi >>= 4; }
    uint32_t qh = 0;
    if (FMT == QF_Q5_0 || FMT == QF_Q5_1) {
      const uint8_t* hp = b + (FMT == QF_Q5_0 ? 2 : 4);
      qh = ((uint32_t)ld16(hp) | ((uint32_t)ld16(hp + 2) << 16)) >> (e >= 16 ? j0 + 16 : j0);   // bit i = fifth bit of value i
    }
    if (FMT == QF_MXFP4) { scale = e8m0_half(b[0]); offset = 0.f; }
    else { scale = h2f(ld16(b)); offset = (FMT == QF_Q4_1 || FMT == QF_Q5_1) ? -h2f(ld16(b + 2)) : 0.f; }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t nib = ((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xF;
      if (FMT == QF_Q4_1) q[i] = (float)nib;
      else if (FMT == QF_Q5_0) q[i] = (float)((int)(nib | (((qh >> i) & 1u) << 4)) - 16);
      else if (FMT == QF_Q5_1) q[i] = (float)(nib | (((qh >> i) & 1u) << 4));
      else if (FMT == QF_IQ4_NL) q[i] = iq4nl_value(nib);
      else q[i] = mxfp4_value(nib);
    }
  } else if (FMT == QF_IQ4_XS) {
    const uint8_t* b = row + (size_t)(k >> 8) * 136;
    const int e = k & 255, ib = e >> 5, r = e & 31, j0 = r & 15;
    const uint32_t sh = ld16(b + 2);
    const int ls = (int)(((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((sh >> (2 * ib)) & 3u) << 4));
    scale = h2f(ld16(b)) * (float)(ls - 32); offset = 0.f;
    uint32_t lo, hi;
    ld8_a2(b + 8 + 16 * ib + j0, lo, hi);
    if (r >= 16) { lo >>= 4; hi >>= 4; }
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = iq4nl_value(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xF);
  } else if (FMT == QF_Q2_K || FMT == QF_Q3_K) {
    // 256-value super-blocks of 2-bit levels: element e sits in half n = e / 128, group j = (e % 128) / 32 (bit pair
    // 2j of its byte), 16-value sub-block is = 8n + 2j + (e % 32) / 16, byte qs[32n + (e % 32)]
    const uint8_t* b = row + (size_t)(k >> 8) * QGeom<FMT>::BYTES;
    const int e = k & 255, n = e >> 7, j = (e & 127) >> 5, r = e & 31, is = 8 * n + 2 * j + (r >> 4);
    uint32_t lo, hi;
    ld8_a2(b + (FMT == QF_Q2_K ? 16 : 32) + 32 * n + r, lo, hi);
    lo >>= 2 * j; hi >>= 2 * j;
    if (FMT == QF_Q2_K) {
      const uint32_t sc = b[is];
      scale = h2f(ld16(b + 80)) * (float)(sc & 0xF);
      offset = h2f(ld16(b + 82)) * (float)(sc >> 4);
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = (float)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 3u);
    } else {
      const uint8_t* sp = b + 96;
      const int g = is >> 2, i4 = is & 3;
      const uint32_t low4 = g < 2 ? (sp[4 * (g & 1) + i4] & 0xFu) : (sp[4 * (g & 1) + i4] >> 4);
      const int sc6 = (int)(low4 | (((sp[8 + i4] >> (2 * g)) & 3u) << 4));
      scale = h2f(ld16(b + 108)) * (float)(sc6 - 32); offset = 0.f;
      uint32_t mlo, mhi;
      ld8_a2(b + r, mlo, mhi);                       // hmask[r .. r + 8): bit (4n + j) set = no -4
      mlo >>= 4 * n + j; mhi >>= 4 * n + j;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t w = i < 4 ? lo : hi, m = i < 4 ? mlo : mhi;
        q[i] = (float)((int)((w >> (8 * (i & 3))) & 3u) - (((m >> (8 * (i & 3))) & 1u) ? 0 : 4));
      }
    }
  } else {  // Q4_0: values 0..15 are the low nibbles of qs[0..15], 16..31 the high nibbles
    const uint8_t* b = row + (size_t)(k >> 5) * 18;
    const int e = k & 31;
    uint32_t lo, hi;
    ld8_a2(b + 2 + (e & 15), lo, hi);
    if (e >= 16) { lo >>= 4; hi >>= 4; }
    scale = h2f(ld16(b)); offset = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = (float)((int)((lo >> (8 * i)) & 0xF) - 8);
      q[4 + i] = (float)((int)((hi >> (8 * i)) & 0xF) - 8);
    }
  }
}

// Runtime-format form: one switch per eight values (uniform across a warp), for kernels that are not instantiated per
// format.  Returns false for a format id that has no decoder.
__device__ __forceinline__ bool decode8_rt(int fmt, const uint8_t* row, int k, float* q, float& scale, float& offset) {
  switch (fmt) {
    case QF_Q4_K: decode8<QF_Q4_K>(row, k, q, scale, offset); return true;
    case QF_Q5_K: decode8<QF_Q5_K>(row, k, q, scale, offset); return true;
    case QF_Q6_K: decode8<QF_Q6_K>(row, k, q, scale, offset); return true;
    case QF_Q8_0: decode8<QF_Q8_0>(row, k, q, scale, offset); return true;
    case QF_Q4_0: decode8<QF_Q4_0>(row, k, q, scale, offset); return true;
    case QF_Q4_1: decode8<QF_Q4_1>(row, k, q, scale, offset); return true;
    case QF_Q5_0: decode8<QF_Q5_0>(row, k, q, scale, offset); return true;
    case QF_Q5_1: decode8<QF_Q5_1>(row, k, q, scale, offset); return true;
    case QF_IQ4_NL: decode8<QF_IQ4_NL>(row, k, q, scale, offset); return true;
    case QF_MXFP4: decode8<QF_MXFP4>(row, k, q, scale, offset); return true;
    case QF_Q2_K: decode8<QF_Q2_K>(row, k, q, scale, offset); return true;
    case QF_Q3_K: decode8<QF_Q3_K>(row, k, q, scale, offset); return true;
    case QF_IQ4_XS: decode8<QF_IQ4_XS>(row, k, q, scale, offset); return true;
    default: return false;
  }
}

// Bytes of one packed row of K values, or 0 for an unknown format.
__host__ __device__ inline size_t quant_row_bytes(int fmt, int K) {
  switch (fmt) {
    case QF_Q4_K: return (size_t)(K / 256) * 144;
    case QF_Q5_K: return (size_t)(K / 256) * 176;
    case QF_Q6_K: return (size_t)(K / 256) * 210;
    case QF_Q2_K: return (size_t)(K / 256) * 84;
    case QF_Q3_K: return (size_t)(K / 256) * 110;
    case QF_IQ4_XS: return (size_t)(K / 256) * 136;
    case QF_Q8_0: return (size_t)(K / 32) * 34;
    case QF_Q4_0: return (size_t)(K / 32) * 18;
    case QF_Q4_1: return (size_t)(K / 32) * 20;
    case QF_Q5_0: return (size_t)(K / 32) * 22;
    case QF_Q5_1: return (size_t)(K / 32) * 24;
    case QF_IQ4_NL: return (size_t)(K / 32) * 18;
    case QF_MXFP4: return (size_t)(K / 32) * 17;
    default: return 0;
  }
}

}  // namespace poot
