// RoPE (+ optional per-head q/k RMSNorm) on the fused QKV projection output and
// scatter of K / V rows into the paged KV pool through a write map.
//
//   qkv  [T, (Hq + 2*Hkv) * D] bf16   (q heads | k heads | v heads)
//   q_out[T, Hq * D]            bf16   rotated queries
//   pool [num_blocks, Hkv, 16, D]      slot s -> block s/16, offset s%16;  slot -1 = no write
//
// Half-split (GPT-NeoX) rotary over the leading `rot` channels:
//   out = x*cos + concat(-x2, x1)*sin,  x1 = x[:rot/2], x2 = x[rot/2:rot];  [rot, D) passes through.
//
// Reference behaviour covered: Rope kernel family (crates/poot-kernelgen/src/data_movement/rope.rs,
// op semantics crates/poot-graph-ir/src/ops/rope.rs:5-58) and the paged ScatterUpdate KV write
// (crates/poot-models/src/components/attention.rs:453-533).
#include "common.cuh"

namespace poot {

constexpr int KV_BLOCK = 16;

template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <> __device__ __forceinline__ __nv_bfloat16 to_kv<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half to_kv<__half>(float v) { return __float2half_rn(v); }

template <typename KV>
__global__ void __launch_bounds__(256)
rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
               KV* __restrict__ kpool, KV* __restrict__ vpool, const int* __restrict__ positions,
               const int* __restrict__ slots, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
               const __nv_bfloat16* __restrict__ q_norm_w, const __nv_bfloat16* __restrict__ k_norm_w,
               float norm_eps, int T, int Hq, int Hkv, int D, int rot, int max_pos) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = Hq + 2 * Hkv;
  if (item >= T * heads) return;
  const int t = item / heads;
  const int h = item - t * heads;
  const __nv_bfloat16* src = qkv + (size_t)t * heads * D + (size_t)h * D;

  if (h >= Hq + Hkv) {  // V head: plain copy into the pool
    int slot = slots[t];
    if (slot < 0) return;
    if (!POOT_IN_RANGE(slot, POOT_LIMIT(kLimPoolSlots), kSiteKvSlot)) return;
    int kvh = h - Hq - Hkv;
    KV* dst = vpool + (((size_t)(slot / KV_BLOCK) * Hkv + kvh) * KV_BLOCK + (slot % KV_BLOCK)) * D;
    for (int d = lane; d < D; d += 32) dst[d] = to_kv<KV>(__bfloat162float(src[d]));
    return;
  }

  const bool is_q = h < Hq;
  int slot = 0;
  if (!is_q) {
    slot = slots[t];
    if (slot < 0) return;
    if (!POOT_IN_RANGE(slot, POOT_LIMIT(kLimPoolSlots), kSiteKvSlot)) return;
  }
  const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
  float inv = 1.f;
  if (nw != nullptr) {
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { float v = __bfloat162float(src[d]); ss += v * v; }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)D + norm_eps);
  }
  int pos = positions[t];
  POOT_IN_RANGE(pos, max_pos, kSitePosition);
  if (pos < 0) pos = 0;
  if (pos >= max_pos) pos = max_pos - 1;
  const int half = rot >> 1;
  const float* cr = cos_t + (size_t)pos * half;
  const float* sr = sin_t + (size_t)pos * half;

  __nv_bfloat16* qdst = is_q ? q_out + (size_t)t * Hq * D + (size_t)h * D : nullptr;
  KV* kdst = is_q ? nullptr
                  : kpool + (((size_t)(slot / KV_BLOCK) * Hkv + (h - Hq)) * KV_BLOCK + (slot % KV_BLOCK)) * D;

  for (int j = lane; j < half; j += 32) {
    float x1 = __bfloat162float(src[j]), x2 = __bfloat162float(src[j + half]);
    if (nw != nullptr) {
      // The normalised head is rounded to bf16 before the rotation, as a separate norm kernel would.
      x1 = __bfloat162float(__float2bfloat16(x1 * inv * __bfloat162float(nw[j])));
      x2 = __bfloat162float(__float2bfloat16(x2 * inv * __bfloat162float(nw[j + half])));
    }
    float c = cr[j], s = sr[j];
    float o1 = x1 * c - x2 * s;
    float o2 = x2 * c + x1 * s;
    if (is_q) { qdst[j] = __float2bfloat16(o1); qdst[j + half] = __float2bfloat16(o2); }
    else { kdst[j] = to_kv<KV>(o1); kdst[j + half] = to_kv<KV>(o2); }
  }
  for (int d = rot + lane; d < D; d += 32) {
    float v = __bfloat162float(src[d]);
    if (nw != nullptr) v = __bfloat162float(__float2bfloat16(v * inv * __bfloat162float(nw[d])));
    if (is_q) qdst[d] = __float2bfloat16(v); else kdst[d] = to_kv<KV>(v);
  }
}

}  // namespace poot

using namespace poot;

// kv_dtype: 0 = bf16, 1 = f16
POOT_API int poot_rope_kv_write(const void* qkv, void* q_out, void* kpool, void* vpool, const int* positions,
                                const int* slots, const float* cos_t, const float* sin_t, const void* q_norm_w,
                                const void* k_norm_w, float norm_eps, int T, int Hq, int Hkv, int D, int rot,
                                int max_pos, int kv_dtype, cudaStream_t s) {
  if (T == 0) return 0;
  if (rot % 2 || rot > D) return (int)cudaErrorInvalidValue;
  int items = T * (Hq + 2 * Hkv);
  int blocks = (items + 7) / 8;
  if (kv_dtype == 0)
    return launch_k(rope_kv_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s,
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, positions,
        slots, cos_t, sin_t, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, norm_eps, T, Hq, Hkv,
        D, rot, max_pos);
  else
    return (int)cudaErrorInvalidValue;  // f16 pools are read by no attention kernel yet
  return (int)cudaGetLastError();
}
