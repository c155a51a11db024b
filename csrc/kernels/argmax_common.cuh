// Candidate ordering of the greedy pick, shared by the sampling kernels and the cross-rank exchange:
// the larger value wins, equal values resolve to the lower index, an index below zero means "no candidate".
#pragma once
#include "common.cuh"

namespace poot {

struct Cand { float v; int i; };
__device__ __forceinline__ Cand better(Cand a, Cand b) {
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}
__device__ __forceinline__ Cand warp_best(Cand c) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Cand t; t.v = __shfl_xor_sync(0xffffffffu, c.v, o); t.i = __shfl_xor_sync(0xffffffffu, c.i, o);
    c = better(c, t);
  }
  return c;
}
__device__ __forceinline__ int warp_min_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace poot
