// Multi-head latent attention in its expanded form (components/mla.rs): assembles, per token and head, the query
// [no-position part | rotary part] and the key [no-position part from the up-projected latent | the one rotary key all
// heads share], applies the rotary to the two rotary parts, and writes the query rows, and the key / value rows into
// the paged pools.  Pool rows are `pool_d = dn + dr` wide; a value uses the first `dv` elements of its row.
#include "common.cuh"

namespace poot {

constexpr int KV_BLOCK = 16;

// grid: one warp per (token, head).  q [T, nh * (dn + dr)], kvb [T, nh * (dn + dv)], kva [T, ld_kva] with the shared rotary key
// at columns [rope_col, rope_col + dr).  cos / sin are [max_pos, dr / 2] (half-split rotary).
__global__ void __launch_bounds__(256)
mla_qkv_write_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kvb, const __nv_bfloat16* __restrict__ kva,
                     int ld_kva, int rope_col, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kpool,
                     __nv_bfloat16* __restrict__ vpool, const int* __restrict__ positions, const int* __restrict__ slots,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int nh, int dn, int dr, int dv,
                     int max_pos) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= T * nh) return;
  const int t = item / nh, h = item - t * nh;
  const int dq = dn + dr, half = dr >> 1;
  int pos = positions[t];
  if (pos < 0) pos = 0;
  if (pos >= max_pos) pos = max_pos - 1;
  const float* cr = cos_t + (size_t)pos * half;
  const float* sr = sin_t + (size_t)pos * half;
  const __nv_bfloat16* qs = q + ((size_t)t * nh + h) * dq;
  __nv_bfloat16* qd = q_out + ((size_t)t * nh + h) * dq;
  for (int d = lane; d < dn; d += 32) qd[d] = qs[d];
  for (int j = lane; j < half; j += 32) {
    const float x1 = __bfloat162float(qs[dn + j]), x2 = __bfloat162float(qs[dn + j + half]);
    qd[dn + j] = __float2bfloat16(x1 * cr[j] - x2 * sr[j]);
    qd[dn + j + half] = __float2bfloat16(x2 * cr[j] + x1 * sr[j]);
  }
  const int slot = slots[t];
  if (slot < 0) return;
  if (!POOT_IN_RANGE(slot, POOT_LIMIT(kLimPoolSlots), kSiteKvSlot)) return;
  const size_t base = (((size_t)(slot / KV_BLOCK) * nh + h) * KV_BLOCK + (slot % KV_BLOCK)) * dq;
  const __nv_bfloat16* kb = kvb + ((size_t)t * nh + h) * (dn + dv);
  __nv_bfloat16* kd = kpool + base;
  __nv_bfloat16* vd = vpool + base;
  for (int d = lane; d < dn; d += 32) kd[d] = kb[d];
  const __nv_bfloat16* kr = kva + (size_t)t * ld_kva + rope_col;
  for (int j = lane; j < half; j += 32) {
    const float x1 = __bfloat162float(kr[j]), x2 = __bfloat162float(kr[j + half]);
    kd[dn + j] = __float2bfloat16(x1 * cr[j] - x2 * sr[j]);
    kd[dn + j + half] = __float2bfloat16(x2 * cr[j] + x1 * sr[j]);
  }
  for (int d = lane; d < dv; d += 32) vd[d] = kb[dn + d];
}

}  // namespace poot

using namespace poot;

POOT_API int poot_mla_qkv_write(const void* q, const void* kvb, const void* kva, int ld_kva, int rope_col, void* q_out, void* kpool,
                                void* vpool, const int* positions, const int* slots, const float* cos_t, const float* sin_t, int T,
                                int nh, int dn, int dr, int dv, int max_pos, cudaStream_t s) {
  if (T == 0) return 0;
  if (dr % 2 || dn < 0 || dv < 1 || dv > dn + dr || nh < 1 || rope_col < 0 || ld_kva < rope_col + dr) return (int)cudaErrorInvalidValue;
  const int items = T * nh;
  return launch_k(mla_qkv_write_kernel, dim3((items + 7) / 8), dim3(256), 0, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kvb,
                  (const __nv_bfloat16*)kva, ld_kva, rope_col, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool,
                  positions, slots, cos_t, sin_t, T, nh, dn, dr, dv, max_pos);
}
