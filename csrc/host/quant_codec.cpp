// Weight storage codecs for the GGUF block formats (host side): block geometry, exact decoders and
// reference encoders.  Format ids are the ggml type ids of the GGUF tensor directory.
//
// One value formula, products left to right in f32 as ggml-quants.c writes them:
//     w = (Scale * SubScale) * value(Codes, Zero)  (+|-)  (Min * SubMin)
// (crates/poot-quant/src/format.rs:10-22; block layouts src/blocks.rs:174-346, bit layouts
// format.rs:54-66).  Decoders are bit-exact with those definitions.  Encoders exist for Q8_0, Q4_0,
// Q4_1, Q5_0, Q5_1, MXFP4 (as the reference, src/encode.rs:71-76) and additionally Q4_K / Q6_K /
// Q5_K / Q2_K / Q3_K (range-based sub-block quantisation in the ggml layout), which the reference lacks.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

namespace {

enum GgmlType : int {
  F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q2_K = 10, Q3_K = 11, Q4_K = 12, Q5_K = 13,
  Q6_K = 14, IQ4_NL = 20, IQ4_XS = 23, BF16 = 30, MXFP4 = 39,
};

inline float fp16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
  if (e == 0) {
    if (m == 0) bits = s;
    else { int sh = 0; while (!(m & 0x400)) { m <<= 1; ++sh; } m &= 0x3FF; bits = s | ((uint32_t)(113 - sh) << 23) | (m << 13); }
  } else if (e == 31) bits = s | 0x7F800000u | (m << 13);
  else bits = s | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &bits, 4); return f;
}
inline uint16_t f32_to_fp16(float f) {
  uint32_t x; memcpy(&x, &f, 4);
  uint32_t s = (x >> 16) & 0x8000; int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15; uint32_t m = x & 0x7FFFFF;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(s | 0x7C00 | (m ? 0x200 : 0));
  if (e >= 31) return (uint16_t)(s | 0x7C00);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    m |= 0x800000; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(s | r);
  }
  uint32_t r = (uint32_t)(e << 10) | (m >> 13), rem = m & 0x1FFF;
  if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) ++r;
  return (uint16_t)(s | r);
}
inline float e8m0_half(uint8_t e) {  // 2^(e-127) / 2, as ggml's GGML_E8M0_TO_FP32_HALF
  uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
  float f; memcpy(&f, &bits, 4); return f;
}

const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
const int8_t kMxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

struct Geom { int elems, bytes; };
Geom geom(int t) {
  switch (t) {
    case F32: return {1, 4}; case F16: case BF16: return {1, 2};
    case Q4_0: return {32, 18}; case Q4_1: return {32, 20}; case Q5_0: return {32, 22}; case Q5_1: return {32, 24};
    case Q8_0: return {32, 34}; case Q2_K: return {256, 84}; case Q3_K: return {256, 110}; case Q4_K: return {256, 144};
    case Q5_K: return {256, 176}; case Q6_K: return {256, 210}; case IQ4_NL: return {32, 18}; case IQ4_XS: return {256, 136};
    case MXFP4: return {32, 17};
    default: return {0, 0};
  }
}

inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

void dequant_block(int t, const uint8_t* b, float* y) {
  switch (t) {
    case Q4_0: { float d = fp16_to_f32(rd16(b)); const uint8_t* q = b + 2;
      for (int j = 0; j < 16; ++j) { y[j] = ((int)(q[j] & 0xF) - 8) * d; y[j + 16] = ((int)(q[j] >> 4) - 8) * d; } break; }
    case Q4_1: { float d = fp16_to_f32(rd16(b)), m = fp16_to_f32(rd16(b + 2)); const uint8_t* q = b + 4;
      for (int j = 0; j < 16; ++j) { y[j] = (q[j] & 0xF) * d + m; y[j + 16] = (q[j] >> 4) * d + m; } break; }
    case Q5_0: { float d = fp16_to_f32(rd16(b)); uint32_t qh; memcpy(&qh, b + 2, 4); const uint8_t* q = b + 6;
      for (int j = 0; j < 16; ++j) {
        uint8_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
        y[j] = ((int)((q[j] & 0xF) | h0) - 16) * d; y[j + 16] = ((int)((q[j] >> 4) | h1) - 16) * d; } break; }
    case Q5_1: { float d = fp16_to_f32(rd16(b)), m = fp16_to_f32(rd16(b + 2)); uint32_t qh; memcpy(&qh, b + 4, 4);
      const uint8_t* q = b + 8;
      for (int j = 0; j < 16; ++j) {
        uint8_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
        y[j] = ((q[j] & 0xF) | h0) * d + m; y[j + 16] = ((q[j] >> 4) | h1) * d + m; } break; }
    case Q8_0: { float d = fp16_to_f32(rd16(b)); const int8_t* q = (const int8_t*)(b + 2);
      for (int j = 0; j < 32; ++j) y[j] = q[j] * d; break; }
    case IQ4_NL: { float d = fp16_to_f32(rd16(b)); const uint8_t* q = b + 2;
      for (int j = 0; j < 16; ++j) { y[j] = d * kIq4nl[q[j] & 0xF]; y[j + 16] = d * kIq4nl[q[j] >> 4]; } break; }
    case MXFP4: { float d = e8m0_half(b[0]); const uint8_t* q = b + 1;
      for (int j = 0; j < 16; ++j) { y[j] = kMxfp4[q[j] & 0xF] * d; y[j + 16] = kMxfp4[q[j] >> 4] * d; } break; }
    case Q2_K: { const uint8_t* sc = b; const uint8_t* q = b + 16; float d = fp16_to_f32(rd16(b + 80)), mn = fp16_to_f32(rd16(b + 82));
      int is = 0;
      for (int n = 0; n < 256; n += 128) { int shift = 0;
        for (int j = 0; j < 4; ++j) {
          uint8_t s = sc[is++]; float dl = d * (s & 0xF), ml = mn * (s >> 4);
          for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l] >> shift) & 3)) - ml;
          s = sc[is++]; dl = d * (s & 0xF); ml = mn * (s >> 4);
          for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l + 16] >> shift) & 3)) - ml;
          shift += 2; }
        q += 32; } break; }
    case Q3_K: { const uint8_t* hm = b; const uint8_t* q = b + 32; float d_all = fp16_to_f32(rd16(b + 108));
      const uint32_t kmask1 = 0x03030303, kmask2 = 0x0f0f0f0f; uint32_t aux[4]; memcpy(aux, b + 96, 12);
      uint32_t tmp = aux[2];
      aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
      aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
      aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
      aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
      const int8_t* scales = (const int8_t*)aux; int is = 0; uint8_t m = 1;
      for (int n = 0; n < 256; n += 128) { int shift = 0;
        for (int j = 0; j < 4; ++j) {
          float dl = d_all * (scales[is++] - 32);
          for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
          dl = d_all * (scales[is++] - 32);
          for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
          shift += 2; m <<= 1; }
        q += 32; } break; }
    case Q4_K: { float d = fp16_to_f32(rd16(b)), mn = fp16_to_f32(rd16(b + 2)); const uint8_t* sc = b + 4; const uint8_t* q = b + 16;
      int is = 0;
      for (int j = 0; j < 256; j += 64) { uint8_t s, m;
        scale_min_k4(is, sc, &s, &m); float d1 = d * s, m1 = mn * m;
        scale_min_k4(is + 1, sc, &s, &m); float d2 = d * s, m2 = mn * m;
        for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
        for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
        q += 32; is += 2; } break; }
    case Q5_K: { float d = fp16_to_f32(rd16(b)), mn = fp16_to_f32(rd16(b + 2)); const uint8_t* sc = b + 4; const uint8_t* qh = b + 16;
      const uint8_t* ql = b + 48; int is = 0; uint8_t u1 = 1, u2 = 2;
      for (int j = 0; j < 256; j += 64) { uint8_t s, m;
        scale_min_k4(is, sc, &s, &m); float d1 = d * s, m1 = mn * m;
        scale_min_k4(is + 1, sc, &s, &m); float d2 = d * s, m2 = mn * m;
        for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
        for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
        ql += 32; is += 2; u1 <<= 2; u2 <<= 2; } break; }
    case Q6_K: { const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192);
      float d = fp16_to_f32(rd16(b + 208));
      for (int n = 0; n < 256; n += 128) {
        for (int l = 0; l < 32; ++l) { int is = l / 16;
          int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
          int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
          int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          y[l] = d * sc[is] * q1; y[l + 32] = d * sc[is + 2] * q2; y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4; }
        y += 128; ql += 64; qh += 32; sc += 8; } break; }
    case IQ4_XS: { float d = fp16_to_f32(rd16(b)); uint16_t sh = rd16(b + 2); const uint8_t* sl = b + 4; const uint8_t* q = b + 8;
      for (int ib = 0; ib < 8; ++ib) {
        int ls = ((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4); float dl = d * (ls - 32);
        for (int j = 0; j < 16; ++j) { y[j] = dl * kIq4nl[q[j] & 0xF]; y[j + 16] = dl * kIq4nl[q[j] >> 4]; }
        y += 32; q += 16; } break; }
    default: break;
  }
}

inline int nearest_int(float v) { return (int)lrintf(v); }

// ---- encoders -----------------------------------------------------------------------------------------
void quant_q8_0(const float* x, uint8_t* b) {
  float amax = 0; for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[j]));
  float d = amax / 127.f, id = d ? 1.f / d : 0.f; uint16_t dh = f32_to_fp16(d); memcpy(b, &dh, 2);
  int8_t* q = (int8_t*)(b + 2); for (int j = 0; j < 32; ++j) q[j] = (int8_t)nearest_int(x[j] * id);
}
void quant_q4_0(const float* x, uint8_t* b) {
  float amax = 0, mx = 0; for (int j = 0; j < 32; ++j) if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); mx = x[j]; }
  float d = mx / -8.f, id = d ? 1.f / d : 0.f; uint16_t dh = f32_to_fp16(d); memcpy(b, &dh, 2);
  for (int j = 0; j < 16; ++j) {
    uint8_t a = (uint8_t)std::min(15, (int)(x[j] * id + 8.5f)), c = (uint8_t)std::min(15, (int)(x[j + 16] * id + 8.5f));
    b[2 + j] = a | (c << 4); }
}
void quant_q4_1(const float* x, uint8_t* b) {
  float mn = x[0], mx = x[0]; for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[j]); mx = std::max(mx, x[j]); }
  float d = (mx - mn) / 15.f, id = d ? 1.f / d : 0.f; uint16_t dh = f32_to_fp16(d), mh = f32_to_fp16(mn);
  memcpy(b, &dh, 2); memcpy(b + 2, &mh, 2);
  for (int j = 0; j < 16; ++j) {
    uint8_t a = (uint8_t)std::min(15, (int)((x[j] - mn) * id + 0.5f)), c = (uint8_t)std::min(15, (int)((x[j + 16] - mn) * id + 0.5f));
    b[4 + j] = a | (c << 4); }
}
void quant_q5_0(const float* x, uint8_t* b) {
  float amax = 0, mx = 0; for (int j = 0; j < 32; ++j) if (fabsf(x[j]) > amax) { amax = fabsf(x[j]); mx = x[j]; }
  float d = mx / -16.f, id = d ? 1.f / d : 0.f; uint16_t dh = f32_to_fp16(d); memcpy(b, &dh, 2);
  uint32_t qh = 0;
  for (int j = 0; j < 16; ++j) {
    uint8_t a = (uint8_t)std::min(31, (int)(x[j] * id + 16.5f)), c = (uint8_t)std::min(31, (int)(x[j + 16] * id + 16.5f));
    b[6 + j] = (a & 0xF) | ((c & 0xF) << 4);
    qh |= ((a & 0x10u) >> 4) << j; qh |= ((c & 0x10u) >> 4) << (j + 16); }
  memcpy(b + 2, &qh, 4);
}
void quant_q5_1(const float* x, uint8_t* b) {
  float mn = x[0], mx = x[0]; for (int j = 1; j < 32; ++j) { mn = std::min(mn, x[j]); mx = std::max(mx, x[j]); }
  float d = (mx - mn) / 31.f, id = d ? 1.f / d : 0.f; uint16_t dh = f32_to_fp16(d), mh = f32_to_fp16(mn);
  memcpy(b, &dh, 2); memcpy(b + 2, &mh, 2); uint32_t qh = 0;
  for (int j = 0; j < 16; ++j) {
    uint8_t a = (uint8_t)std::min(31, (int)((x[j] - mn) * id + 0.5f)), c = (uint8_t)std::min(31, (int)((x[j + 16] - mn) * id + 0.5f));
    b[8 + j] = (a & 0xF) | ((c & 0xF) << 4);
    qh |= ((a & 0x10u) >> 4) << j; qh |= ((c & 0x10u) >> 4) << (j + 16); }
  memcpy(b + 4, &qh, 4);
}
void quant_mxfp4(const float* x, uint8_t* b) {
  float amax = 0; for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(x[j]));
  int e = amax > 0 ? (int)floorf(log2f(amax)) - 2 + 127 : 0;   // largest magnitude 6 = 1.5 * 2^2
  e = std::max(0, std::min(254, e)); b[0] = (uint8_t)e; float d = e8m0_half((uint8_t)e);
  auto best = [&](float v) { int bi = 0; float be = 1e30f;
    for (int i = 0; i < 16; ++i) { float err = fabsf(kMxfp4[i] * d - v); if (err < be) { be = err; bi = i; } } return bi; };
  for (int j = 0; j < 16; ++j) b[1 + j] = (uint8_t)(best(x[j]) | (best(x[j + 16]) << 4));
}

// 6-bit (scale, min) packing of the K-quants: 8 sub-blocks into 12 bytes.
void pack_scales_k4(const uint8_t* ls, const uint8_t* lm, uint8_t* sc) {
  memset(sc, 0, 12);
  for (int j = 0; j < 8; ++j) {
    if (j < 4) { sc[j] = ls[j]; sc[j + 4] = lm[j]; }
    else { sc[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4); sc[j - 4] |= (ls[j] >> 4) << 6; sc[j] |= (lm[j] >> 4) << 6; } }
}
void sub_ranges(const float* x, int nsub, int sub, int levels, float* scales, float* mins) {
  for (int s = 0; s < nsub; ++s) {
    float mn = x[s * sub], mx = mn;
    for (int l = 1; l < sub; ++l) { mn = std::min(mn, x[s * sub + l]); mx = std::max(mx, x[s * sub + l]); }
    if (mn > 0) mn = 0;
    scales[s] = (mx - mn) / (float)levels; mins[s] = -mn; }
}
void quant_q4_k(const float* x, uint8_t* b) {
  float scales[8], mins[8]; sub_ranges(x, 8, 32, 15, scales, mins);
  float ms = *std::max_element(scales, scales + 8), mm = *std::max_element(mins, mins + 8);
  float d = ms / 63.f, dm = mm / 63.f; uint16_t dh = f32_to_fp16(d), mh = f32_to_fp16(dm);
  float df = fp16_to_f32(dh), dmf = fp16_to_f32(mh);
  uint8_t ls[8], lm[8];
  for (int j = 0; j < 8; ++j) {
    ls[j] = (uint8_t)std::min(63, df ? nearest_int(scales[j] / df) : 0);
    lm[j] = (uint8_t)std::min(63, dmf ? nearest_int(mins[j] / dmf) : 0); }
  memcpy(b, &dh, 2); memcpy(b + 2, &mh, 2); pack_scales_k4(ls, lm, b + 4);
  uint8_t L[256];
  for (int j = 0; j < 8; ++j) { float dl = df * ls[j], ml = dmf * lm[j];
    for (int l = 0; l < 32; ++l) { int q = dl ? nearest_int((x[j * 32 + l] + ml) / dl) : 0; L[j * 32 + l] = (uint8_t)std::max(0, std::min(15, q)); } }
  uint8_t* q = b + 16;
  for (int j = 0; j < 256; j += 64) { for (int l = 0; l < 32; ++l) q[l] = L[j + l] | (L[j + l + 32] << 4); q += 32; }
}
void quant_q5_k(const float* x, uint8_t* b) {
  float scales[8], mins[8]; sub_ranges(x, 8, 32, 31, scales, mins);
  float ms = *std::max_element(scales, scales + 8), mm = *std::max_element(mins, mins + 8);
  float d = ms / 63.f, dm = mm / 63.f; uint16_t dh = f32_to_fp16(d), mh = f32_to_fp16(dm);
  float df = fp16_to_f32(dh), dmf = fp16_to_f32(mh);
  uint8_t ls[8], lm[8];
  for (int j = 0; j < 8; ++j) {
    ls[j] = (uint8_t)std::min(63, df ? nearest_int(scales[j] / df) : 0);
    lm[j] = (uint8_t)std::min(63, dmf ? nearest_int(mins[j] / dmf) : 0); }
  memcpy(b, &dh, 2); memcpy(b + 2, &mh, 2); pack_scales_k4(ls, lm, b + 4);
  uint8_t L[256];
  for (int j = 0; j < 8; ++j) { float dl = df * ls[j], ml = dmf * lm[j];
    for (int l = 0; l < 32; ++l) { int q = dl ? nearest_int((x[j * 32 + l] + ml) / dl) : 0; L[j * 32 + l] = (uint8_t)std::max(0, std::min(31, q)); } }
  uint8_t* qh = b + 16; uint8_t* ql = b + 48; memset(qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < 256; n += 64) {
    for (int l = 0; l < 32; ++l) { int l1 = L[n + l], l2 = L[n + l + 32];
      if (l1 > 15) { l1 -= 16; qh[l] |= m1; } if (l2 > 15) { l2 -= 16; qh[l] |= m2; }
      ql[l] = (uint8_t)(l1 | (l2 << 4)); }
    m1 <<= 2; m2 <<= 2; ql += 32; }
}
void quant_q6_k(const float* x, uint8_t* b) {
  float scales[16]; float maxabs = 0, maxs = 0;
  for (int s = 0; s < 16; ++s) { float am = 0, mv = 0;
    for (int l = 0; l < 16; ++l) if (fabsf(x[s * 16 + l]) > am) { am = fabsf(x[s * 16 + l]); mv = x[s * 16 + l]; }
    scales[s] = mv / -32.f; if (fabsf(scales[s]) > maxabs) { maxabs = fabsf(scales[s]); maxs = scales[s]; } }
  uint8_t* ql = b; uint8_t* qh = b + 128; int8_t* sc = (int8_t*)(b + 192);
  if (maxabs == 0) { memset(b, 0, 210); return; }
  float iscale = -128.f / maxs; float d = 1.f / iscale; uint16_t dh = f32_to_fp16(d); memcpy(b + 208, &dh, 2);
  float df = fp16_to_f32(dh);
  uint8_t L[256];
  for (int s = 0; s < 16; ++s) { sc[s] = (int8_t)std::max(-128, std::min(127, nearest_int(iscale * scales[s])));
    float dl = df * sc[s];
    for (int l = 0; l < 16; ++l) { int q = dl ? nearest_int(x[s * 16 + l] / dl) : 0; L[s * 16 + l] = (uint8_t)(std::max(-32, std::min(31, q)) + 32); } }
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      uint8_t q1 = L[n + l] & 0xF, q2 = L[n + l + 32] & 0xF, q3 = L[n + l + 64] & 0xF, q4 = L[n + l + 96] & 0xF;
      ql[l] = q1 | (q3 << 4); ql[l + 32] = q2 | (q4 << 4);
      qh[l] = (L[n + l] >> 4) | ((L[n + l + 32] >> 4) << 2) | ((L[n + l + 64] >> 4) << 4) | ((L[n + l + 96] >> 4) << 6); }
    ql += 64; qh += 32; }
}
void quant_q2_k(const float* x, uint8_t* b) {
  float scales[16], mins[16]; sub_ranges(x, 16, 16, 3, scales, mins);
  float ms = *std::max_element(scales, scales + 16), mm = *std::max_element(mins, mins + 16);
  float d = ms / 15.f, dm = mm / 15.f; uint16_t dh = f32_to_fp16(d), mh = f32_to_fp16(dm);
  float df = fp16_to_f32(dh), dmf = fp16_to_f32(mh);
  memcpy(b + 80, &dh, 2); memcpy(b + 82, &mh, 2);
  uint8_t L[256];
  for (int j = 0; j < 16; ++j) {
    int ls = std::min(15, df ? nearest_int(scales[j] / df) : 0), lm = std::min(15, dmf ? nearest_int(mins[j] / dmf) : 0);
    b[j] = (uint8_t)(ls | (lm << 4)); float dl = df * ls, ml = dmf * lm;
    for (int l = 0; l < 16; ++l) { int q = dl ? nearest_int((x[j * 16 + l] + ml) / dl) : 0; L[j * 16 + l] = (uint8_t)std::max(0, std::min(3, q)); } }
  uint8_t* q = b + 16;
  for (int n = 0; n < 256; n += 128) { for (int l = 0; l < 32; ++l) q[l] = L[n + l] | (L[n + l + 32] << 2) | (L[n + l + 64] << 4) | (L[n + l + 96] << 6); q += 32; }
}
void quant_q3_k(const float* x, uint8_t* b) {
  float scales[16]; float maxabs = 0, maxs = 0;
  for (int s = 0; s < 16; ++s) { float am = 0, mv = 0;
    for (int l = 0; l < 16; ++l) if (fabsf(x[s * 16 + l]) > am) { am = fabsf(x[s * 16 + l]); mv = x[s * 16 + l]; }
    scales[s] = mv / -4.f; if (fabsf(scales[s]) > maxabs) { maxabs = fabsf(scales[s]); maxs = scales[s]; } }
  memset(b, 0, 110);
  if (maxabs == 0) return;
  float iscale = -32.f / maxs; float d = 1.f / iscale; uint16_t dh = f32_to_fp16(d); memcpy(b + 108, &dh, 2);
  float df = fp16_to_f32(dh);
  int8_t ls[16]; uint8_t L[256];
  for (int s = 0; s < 16; ++s) { int l = std::max(-32, std::min(31, nearest_int(iscale * scales[s]))); ls[s] = (int8_t)l;
    float dl = df * l;
    for (int i = 0; i < 16; ++i) { int q = dl ? nearest_int(x[s * 16 + i] / dl) : 0; L[s * 16 + i] = (uint8_t)(std::max(-4, std::min(3, q)) + 4); } }
  uint8_t* sc = b + 96;
  for (int j = 0; j < 16; ++j) { int l = ls[j] + 32;
    if (j < 8) sc[j] = l & 0xF; else sc[j - 8] |= (l & 0xF) << 4;
    sc[8 + j % 4] |= (uint8_t)((l >> 4) << (2 * (j / 4))); }
  uint8_t* hm = b; int m = 0; uint8_t hb = 1;
  for (int j = 0; j < 256; ++j) { if (L[j] > 3) { hm[m] |= hb; L[j] -= 4; } if (++m == 32) { m = 0; hb <<= 1; } }
  uint8_t* q = b + 32;
  for (int n = 0; n < 256; n += 128) { for (int l = 0; l < 32; ++l) q[l] = L[n + l] | (L[n + l + 32] << 2) | (L[n + l + 64] << 4) | (L[n + l + 96] << 6); q += 32; }
}

template <typename F>
void parallel_blocks(long long nblocks, F fn) {
  unsigned nt = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
  if (nblocks < 4096) { for (long long i = 0; i < nblocks; ++i) fn(i); return; }
  std::vector<std::thread> th;
  for (unsigned t = 0; t < nt; ++t)
    th.emplace_back([=]() { for (long long i = t; i < nblocks; i += nt) fn(i); });
  for (auto& x : th) x.join();
}

}  // namespace

HOST_API int poot_quant_geometry(int type, int* block_elems, int* block_bytes) {
  Geom g = geom(type);
  if (g.elems == 0) return -1;
  *block_elems = g.elems; *block_bytes = g.bytes;
  return 0;
}

// src: packed blocks; dst: n floats.  n must be a multiple of the block size.  Returns 0, or -1 for an unknown type.
HOST_API int poot_dequantize(int type, const void* src, float* dst, long long n) {
  Geom g = geom(type);
  if (g.elems == 0 || n % g.elems) return -1;
  const uint8_t* s = (const uint8_t*)src;
  if (type == F32) { memcpy(dst, s, (size_t)n * 4); return 0; }
  if (type == F16) { const uint16_t* h = (const uint16_t*)s; for (long long i = 0; i < n; ++i) dst[i] = fp16_to_f32(h[i]); return 0; }
  if (type == BF16) { const uint16_t* h = (const uint16_t*)s; for (long long i = 0; i < n; ++i) { uint32_t b = (uint32_t)h[i] << 16; memcpy(dst + i, &b, 4); } return 0; }
  parallel_blocks(n / g.elems, [=](long long i) { dequant_block(type, s + (size_t)i * g.bytes, dst + (size_t)i * g.elems); });
  return 0;
}

HOST_API int poot_quantize(int type, const float* src, void* dst, long long n) {
  Geom g = geom(type);
  if (g.elems == 0 || n % g.elems) return -1;
  uint8_t* d = (uint8_t*)dst;
  void (*fn)(const float*, uint8_t*) = nullptr;
  switch (type) {
    case Q8_0: fn = quant_q8_0; break; case Q4_0: fn = quant_q4_0; break; case Q4_1: fn = quant_q4_1; break;
    case Q5_0: fn = quant_q5_0; break; case Q5_1: fn = quant_q5_1; break; case MXFP4: fn = quant_mxfp4; break;
    case Q4_K: fn = quant_q4_k; break; case Q5_K: fn = quant_q5_k; break; case Q6_K: fn = quant_q6_k; break;
    case Q2_K: fn = quant_q2_k; break; case Q3_K: fn = quant_q3_k; break;
    case F16: { uint16_t* h = (uint16_t*)d; for (long long i = 0; i < n; ++i) h[i] = f32_to_fp16(src[i]); return 0; }
    default: return -2;   // no encoder for this format
  }
  parallel_blocks(n / g.elems, [=](long long i) { fn(src + (size_t)i * g.elems, d + (size_t)i * g.bytes); });
  return 0;
}

// Content check of packed data: every block scale must be finite (a NaN/Inf scale poisons a whole block).
// Returns the index of the first bad block or -1.
HOST_API long long poot_quant_check_scales(int type, const void* src, long long n) {
  Geom g = geom(type);
  if (g.elems <= 1) return -1;
  const uint8_t* s = (const uint8_t*)src;
  auto bad16 = [](uint16_t h) { return ((h >> 10) & 0x1F) == 0x1F; };
  for (long long i = 0; i < n / g.elems; ++i) {
    const uint8_t* b = s + (size_t)i * g.bytes; bool bad = false;
    switch (type) {
      case Q4_0: case Q5_0: case Q8_0: case IQ4_NL: case IQ4_XS: bad = bad16(rd16(b)); break;
      case Q4_1: case Q5_1: case Q4_K: case Q5_K: bad = bad16(rd16(b)) || bad16(rd16(b + 2)); break;
      case Q2_K: bad = bad16(rd16(b + 80)) || bad16(rd16(b + 82)); break;
      case Q3_K: bad = bad16(rd16(b + 108)); break;
      case Q6_K: bad = bad16(rd16(b + 208)); break;
      case MXFP4: bad = b[0] == 0xFF; break;
      default: break;
    }
    if (bad) return i;
  }
  return -1;
}
