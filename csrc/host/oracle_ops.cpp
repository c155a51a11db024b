// Native inner loops of the host evaluator, for whole-model checks at sizes the NumPy loops do not reach.
//
//  * poot_host_packed_matmul: y[M, N] = x[M, K] . W[N, K]^T with W in a GGUF block format, decoded row by row inside the
//    product (a row's blocks are decoded once into a per-thread buffer and multiplied with every activation row), so a
//    quantised model is evaluated at its packed size instead of being expanded to f32 matrices.  Both operands may be
//    rounded to bf16 first (the "narrow" operand precision of the graph's contractions); sums are f32 in K order within
//    eight interleaved partial sums, the same for every thread count.
//  * poot_host_delta_rule / poot_host_ssd: the two recurrences of the scan equation, one token at a time, heads in parallel.
//  * poot_host_arg_top_k: ids of the entries whose rank is below k, placed at their rank.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

extern "C" int poot_quant_geometry(int type, int* block_elems, int* block_bytes);
extern "C" int poot_dequantize(int type, const void* src, float* dst, long long n);

namespace {

inline float bf16_round(float f) {
  uint32_t x; memcpy(&x, &f, 4);
  if ((x & 0x7F800000u) == 0x7F800000u) return f;            // inf / nan pass through
  x += 0x7FFFu + ((x >> 16) & 1u);                             // round to nearest, ties to even
  x &= 0xFFFF0000u;
  float r; memcpy(&r, &x, 4); return r;
}

inline float dot8(const float* a, const float* b, long long n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long i = 0;
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
  float tail = 0.f;
  for (; i < n; ++i) tail += a[i] * b[i];
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7])) + tail;
}

template <class F>
void parallel_for(long long n, int threads, F f) {
  int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nt = (int)std::max<long long>(1, std::min<long long>(nt, n));
  if (nt == 1) { for (long long i = 0; i < n; ++i) f(i, 0); return; }
  std::vector<std::thread> th;
  for (int t = 0; t < nt; ++t)
    th.emplace_back([=]() { for (long long i = t; i < n; i += nt) f(i, t); });
  for (auto& x : th) x.join();
}

}  // namespace

// Returns 0; -1 unknown format or K not a whole number of blocks.
HOST_API int poot_host_packed_matmul(int type, const void* w, long long N, long long K, const float* x, long long M, float* y,
                                     int narrow_x, int threads) {
  int be = 0, bb = 0;
  if (poot_quant_geometry(type, &be, &bb) != 0 || be <= 0 || K % be) return -1;
  const size_t row_bytes = (size_t)(K / be) * bb;
  std::vector<float> xs((size_t)M * K);
  for (long long i = 0; i < M * K; ++i) xs[i] = narrow_x ? bf16_round(x[i]) : x[i];
  int nt = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
  nt = std::max(1, nt);
  std::vector<std::vector<float>> rowbuf(nt, std::vector<float>((size_t)K));
  const uint8_t* wb = (const uint8_t*)w;
  const float* xp = xs.data();
  parallel_for(N, nt, [&](long long n, int t) {
    float* r = rowbuf[t].data();
    // one row at a time: the codec's own decoder (single-threaded for a row's worth of blocks)
    poot_dequantize(type, wb + (size_t)n * row_bytes, r, K);
    if (narrow_x) for (long long i = 0; i < K; ++i) r[i] = bf16_round(r[i]);    // narrow precision rounds both operands
    for (long long m = 0; m < M; ++m) y[(size_t)m * N + n] = dot8(xp + (size_t)m * K, r, K);
  });
  return 0;
}

// q, k, v [H, L, D]; g [H, L, G] with G = 1 (one decay per head and token) or D (one per key channel); beta [H, L];
// state [H, D, D] in / out (key channel, then value channel); y [H, L, D].
HOST_API void poot_host_delta_rule(const float* q, const float* k, const float* v, const float* g, int G, const float* beta,
                                   float* state, float* y, int H, int L, int D, int threads) {
  parallel_for(H, threads, [&](long long h, int) {
    float* S = state + (size_t)h * D * D;
    std::vector<float> kv(D), dlt(D);
    for (int t = 0; t < L; ++t) {
      const float* qt = q + ((size_t)h * L + t) * D; const float* kt = k + ((size_t)h * L + t) * D;
      const float* vt = v + ((size_t)h * L + t) * D; const float* gt = g + ((size_t)h * L + t) * G;
      for (int i = 0; i < D; ++i) {
        const float dec = std::exp(gt[G == 1 ? 0 : i]);
        for (int j = 0; j < D; ++j) S[(size_t)i * D + j] *= dec;
      }
      for (int j = 0; j < D; ++j) { float a = 0.f; for (int i = 0; i < D; ++i) a += kt[i] * S[(size_t)i * D + j]; kv[j] = a; }
      const float b = beta[(size_t)h * L + t];
      for (int j = 0; j < D; ++j) dlt[j] = (vt[j] - kv[j]) * b;
      for (int i = 0; i < D; ++i) for (int j = 0; j < D; ++j) S[(size_t)i * D + j] += kt[i] * dlt[j];
      float* yt = y + ((size_t)h * L + t) * D;
      for (int j = 0; j < D; ++j) { float a = 0.f; for (int i = 0; i < D; ++i) a += qt[i] * S[(size_t)i * D + j]; yt[j] = a; }
    }
  });
}

// x [H, L, P]; b, c [H, L, N]; delta [H, L]; a, d [H]; state [H, N, P] in / out; y [H, L, P].
HOST_API void poot_host_ssd(const float* x, const float* b, const float* c, const float* delta, const float* a, const float* d,
                            float* state, float* y, int H, int L, int P, int N, int threads) {
  parallel_for(H, threads, [&](long long h, int) {
    float* S = state + (size_t)h * N * P;
    for (int t = 0; t < L; ++t) {
      const float dt = delta[(size_t)h * L + t], dec = std::exp(dt * a[h]);
      const float* xt = x + ((size_t)h * L + t) * P; const float* bt = b + ((size_t)h * L + t) * N;
      const float* ct = c + ((size_t)h * L + t) * N;
      float* yt = y + ((size_t)h * L + t) * P;
      for (int p = 0; p < P; ++p) yt[p] = d[h] * xt[p];
      for (int n = 0; n < N; ++n) {
        const float w = dt * bt[n];
        for (int p = 0; p < P; ++p) {
          const float s = dec * S[(size_t)n * P + p] + w * xt[p];
          S[(size_t)n * P + p] = s;
          yt[p] += ct[n] * s;
        }
      }
    }
  });
}

// rank [R, E] int32 -> ids [R, k]: entry e with 0 <= rank < k lands at ids[r, rank]; unfilled places stay 0.
HOST_API void poot_host_arg_top_k(const int32_t* rank, int R, int E, int k, int32_t* ids) {
  std::fill(ids, ids + (size_t)R * k, 0);
  for (int r = 0; r < R; ++r)
    for (int e = 0; e < E; ++e) {
      const int32_t rk = rank[(size_t)r * E + e];
      if (rk >= 0 && rk < k) ids[(size_t)r * k + rk] = e;
    }
}
