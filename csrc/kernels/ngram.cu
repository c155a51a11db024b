// Hashed n-gram ids of a per-layer embedding block (crates/poot-models/src/components/ple.rs `row_ids`).
//
// For every token of a sequence piece the id of hash head h is
//     ((m0 * s0) ^ (m1 * s1) [^ (m2 * s2)]) % prime[h] + offset[h]
// over wrapping 64-bit words, with s0 the token, s1 the token before it and, for the heads of order 3, s2 the token two
// back (or the end-of-sequence id when s1 is the end-of-sequence id: a context that ends a segment hides what precedes
// it).  Tokens before the piece come from the sequence's carried history of `ctx` ids, stored xor-ed with the
// end-of-sequence id so that a zeroed history reads as a sequence start; a piece at position 0 ignores the history.
// The kernel also writes the history the next piece of the sequence reads.
//
// A step names its pieces in a table of (first row, rows, sequence row, first position), like the recurrent mixers;
// entries with zero rows are skipped, so one grid shape serves every step of a captured graph.
#include "common.cuh"

namespace poot {

// grid (pieces), block 128 threads: threads stride over (token, head) pairs of the piece; thread 0 writes the history last.
__global__ void ngram_hash_kernel(const int* __restrict__ tokens, int* __restrict__ history, int history_rows,
                                  const int* __restrict__ segs, const unsigned long long* __restrict__ mult,
                                  const unsigned* __restrict__ primes, const int* __restrict__ offsets, int ctx, int heads,
                                  int per_order, int eos, int vocab, int* __restrict__ ids) {
  pdl_wait(); pdl_launch();
  const int s = blockIdx.x;
  const int first = segs[4 * s], n = segs[4 * s + 1], seq = segs[4 * s + 2], pos0 = segs[4 * s + 3];
  if (n <= 0 || seq < 0 || seq >= history_rows) return;
  int* hist = history + (size_t)seq * ctx;
  // the ctx tokens before the piece, oldest first (decoded); a fresh sequence starts behind end-of-sequence ids
  __shared__ int before[2];
  if (threadIdx.x < ctx) before[threadIdx.x] = pos0 == 0 ? eos : (hist[threadIdx.x] ^ eos);
  __syncthreads();
  auto at = [&](int i) -> int {            // token at piece offset i (negative: the carried context); out-of-vocabulary reads 0
    if (i < 0) return before[ctx + i];
    const int t = tokens[first + i];
    return (t >= 0 && t < vocab) ? t : 0;
  };
  for (int w = threadIdx.x; w < n * heads; w += blockDim.x) {
    const int i = w / heads, h = w % heads;
    const unsigned long long s0 = (unsigned long long)at(i), s1 = (unsigned long long)at(i - 1);
    unsigned long long mix = (s0 * mult[0]) ^ (s1 * mult[1]);
    if (h >= per_order) {                   // order 3
      const unsigned long long s2 = at(i - 1) == eos ? (unsigned long long)eos : (unsigned long long)at(i - 2);
      mix ^= s2 * mult[2];
    }
    ids[(size_t)(first + i) * heads + h] = (int)(mix % primes[h]) + offsets[h];
  }
  __syncthreads();                          // every read of the old context is done
  if (threadIdx.x < ctx) hist[threadIdx.x] = at(n - ctx + threadIdx.x) ^ eos;
}

}  // namespace poot

POOT_API int poot_ngram_hash(const int* tokens, int* history, int history_rows, const int* segs, int n_segs,
                             const unsigned long long* mult, const unsigned* primes, const int* offsets, int ctx, int heads,
                             int per_order, int eos, int vocab, int* ids, cudaStream_t s) {
  using namespace poot;
  if (n_segs == 0) return 0;
  if (ctx < 1 || ctx > 2 || per_order < 1 || heads != ctx * per_order || vocab < 1) return (int)cudaErrorInvalidValue;
  return launch_k(ngram_hash_kernel, dim3(n_segs), dim3(128), 0, s, tokens, history, history_rows, segs, mult, primes, offsets, ctx,
                  heads, per_order, eos, vocab, ids);
}
