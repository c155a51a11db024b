// Gated delta net mixer (linear attention with a carried matrix state) and gated attention helpers:
//
//  * causal_conv_silu: depthwise causal convolution + SiLU over the (q | k | v) channels, per sequence piece, continuing
//    from and updating the sequence's window of the previous K-1 inputs;
//  * gdn_scan: the gated delta rule  S <- S * exp(g);  d = (v - k.S) * beta;  S <- S + k (x) d;  y = q.S  per value head,
//    the D x D state of the (sequence, head) held in shared memory for the whole piece
//    (crates/poot-graph-ir/src/ops/ssm.rs, crates/poot-kernelgen/src/scan.rs:1-8: "workgroup per (head, column block),
//    state column in LDS");
//  * kda_scan: the same rule with a decay per key channel (Kimi delta attention);
//  * gated_rmsnorm: RMSNorm per head times SiLU(z);  sigmoid_mul: a *= sigmoid(g).
//
// A step names its sequence pieces in a table of (first row, rows, sequence row, first position); entries with zero rows
// are skipped, so one grid shape serves every step of a captured graph.  A piece at position 0 starts from zero state.
#include "common.cuh"

namespace poot {

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <int KC>
__global__ void causal_conv_silu_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int col0, int C,
                                        const float* __restrict__ w, const float* __restrict__ bias, float* __restrict__ state,
                                        int state_rows, const int* __restrict__ segs, __nv_bfloat16* __restrict__ out) {
  pdl_wait(); pdl_launch();
  const int s = blockIdx.y;
  const int first = segs[4 * s], n = segs[4 * s + 1], seq = segs[4 * s + 2], pos0 = segs[4 * s + 3];
  if (n <= 0 || seq < 0 || seq >= state_rows) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float win[KC - 1];                        // the previous KC-1 inputs of this channel, oldest first
  float* st = state + (size_t)seq * (KC - 1) * C + c;
#pragma unroll
  for (int k = 0; k < KC - 1; ++k) win[k] = pos0 == 0 ? 0.f : st[(size_t)k * C];
  float wk[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) wk[k] = w[(size_t)c * KC + k];
  const float b0 = bias ? bias[c] : 0.f;
  for (int i = 0; i < n; ++i) {
    const float v = bf2f(x[(size_t)(first + i) * ldx + col0 + c]);
    float acc = b0 + wk[KC - 1] * v;
#pragma unroll
    for (int k = 0; k < KC - 1; ++k) acc += wk[k] * win[k];
#pragma unroll
    for (int k = 0; k + 1 < KC - 1; ++k) win[k] = win[k + 1];
    win[KC - 2] = v;
    out[(size_t)(first + i) * C + c] = __float2bfloat16(silu(acc));
  }
#pragma unroll
  for (int k = 0; k < KC - 1; ++k) st[(size_t)k * C] = win[k];
}

template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();                          // the previous call's readers are done with red
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) t += red[i];
  return t;
}

// grid (value heads, pieces), block D threads: thread j owns column j of the head's state S[key i][value j].
template <int D>
__global__ void __launch_bounds__(D) gdn_scan_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ ba,
                                                     int ldb, int b_col, int a_col, const float* __restrict__ dt_bias,
                                                     const float* __restrict__ a_log, float* __restrict__ state, int state_rows,
                                                     const int* __restrict__ segs, __nv_bfloat16* __restrict__ out, int nk, int nv) {
  extern __shared__ float sm[];
  float* S = sm;                            // [D][D]
  float* qs = S + D * D;
  float* ks = qs + D;
  float* red = ks + D;                      // [8]
  pdl_wait(); pdl_launch();
  const int s = blockIdx.y, h = blockIdx.x, j = threadIdx.x;
  const int first = segs[4 * s], n = segs[4 * s + 1], seq = segs[4 * s + 2], pos0 = segs[4 * s + 3];
  if (n <= 0 || seq < 0 || seq >= state_rows) return;
  float* St = state + ((size_t)seq * nv + h) * D * D;
  for (int i = 0; i < D; ++i) S[i * D + j] = pos0 == 0 ? 0.f : St[(size_t)i * D + j];
  const int hk = h / (nv / nk);
  const size_t C = (size_t)(2 * nk + nv) * D;
  const float A = -__expf(a_log[h]), bias = dt_bias[h];
  const float qscale = rsqrtf((float)D);
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)first + t;
    const __nv_bfloat16* r = qkv + row * C;
    const float qv = bf2f(r[hk * D + j]), kv = bf2f(r[nk * D + hk * D + j]), vv = bf2f(r[2 * nk * D + h * D + j]);
    const float q2 = block_sum<D>(qv * qv, red);
    const float k2 = block_sum<D>(kv * kv, red);
    qs[j] = qv * rsqrtf(q2 + 1e-6f) * qscale;
    ks[j] = kv * rsqrtf(k2 + 1e-6f);
    __syncthreads();
    const float a = bf2f(ba[row * ldb + a_col + h]) + bias, b = bf2f(ba[row * ldb + b_col + h]);
    const float sp = a > 20.f ? a : log1pf(__expf(a));
    const float decay = __expf(A * sp), beta = 1.f / (1.f + __expf(-b));
    float kvm = 0.f;
    for (int i = 0; i < D; ++i) {
      const float sij = S[i * D + j] * decay;
      S[i * D + j] = sij;
      kvm += ks[i] * sij;
    }
    const float delta = (vv - kvm) * beta;
    float y = 0.f;
    for (int i = 0; i < D; ++i) {
      const float sij = S[i * D + j] + ks[i] * delta;
      S[i * D + j] = sij;
      y += qs[i] * sij;
    }
    out[row * ((size_t)nv * D) + h * D + j] = __float2bfloat16(y);
    __syncthreads();                        // qs / ks are rewritten for the next row
  }
  for (int i = 0; i < D; ++i) St[(size_t)i * D + j] = S[i * D + j];
}

// Kimi delta attention: the same delta rule with a decay PER KEY CHANNEL.  Row i of the head's state decays by
//   exp(lower_bound * sigmoid(exp(a_log[h]) * (f[h, i] + dt_bias[h, i])))
// before the read; q, k, v come from the convolution as [T, 3 * heads * D] (q | k | v), `f` holds the raw output of the
// low-rank gate projection [T, heads * D], beta the raw b projection at column b_col of `bm`.
// grid (heads, pieces), block D threads: thread j owns column j of S[key i][value j] and computes the decay of row j.
template <int D>
__global__ void __launch_bounds__(D) kda_scan_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ f,
                                                     const __nv_bfloat16* __restrict__ bm, int ldb, int b_col,
                                                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                     float lower_bound, float* __restrict__ state, int state_rows,
                                                     const int* __restrict__ segs, __nv_bfloat16* __restrict__ out, int heads) {
  extern __shared__ float sm[];
  float* S = sm;                            // [D][D]
  float* qs = S + D * D;
  float* ks = qs + D;
  float* ds = ks + D;                       // decay of each key channel for this row
  float* red = ds + D;                      // [8]
  pdl_wait(); pdl_launch();
  const int s = blockIdx.y, h = blockIdx.x, j = threadIdx.x;
  const int first = segs[4 * s], n = segs[4 * s + 1], seq = segs[4 * s + 2], pos0 = segs[4 * s + 3];
  if (n <= 0 || seq < 0 || seq >= state_rows) return;
  float* St = state + ((size_t)seq * heads + h) * D * D;
  for (int i = 0; i < D; ++i) S[i * D + j] = pos0 == 0 ? 0.f : St[(size_t)i * D + j];
  const size_t C = (size_t)heads * D;
  const float rate = __expf(a_log[h]), bias = dt_bias[h * D + j];
  const float qscale = rsqrtf((float)D);
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)first + t;
    const __nv_bfloat16* r = qkv + row * 3 * C;
    const float qv = bf2f(r[h * D + j]), kv = bf2f(r[C + h * D + j]), vv = bf2f(r[2 * C + h * D + j]);
    const float q2 = block_sum<D>(qv * qv, red);
    const float k2 = block_sum<D>(kv * kv, red);
    qs[j] = qv * rsqrtf(q2 + 1e-6f) * qscale;
    ks[j] = kv * rsqrtf(k2 + 1e-6f);
    const float gate = 1.f / (1.f + __expf(-rate * (bf2f(f[row * C + h * D + j]) + bias)));
    ds[j] = __expf(lower_bound * gate);
    __syncthreads();
    const float b = bf2f(bm[row * ldb + b_col + h]);
    const float beta = 1.f / (1.f + __expf(-b));
    float kvm = 0.f;
    for (int i = 0; i < D; ++i) {
      const float sij = S[i * D + j] * ds[i];
      S[i * D + j] = sij;
      kvm += ks[i] * sij;
    }
    const float delta = (vv - kvm) * beta;
    float y = 0.f;
    for (int i = 0; i < D; ++i) {
      const float sij = S[i * D + j] + ks[i] * delta;
      S[i * D + j] = sij;
      y += qs[i] * sij;
    }
    out[row * C + h * D + j] = __float2bfloat16(y);
    __syncthreads();                        // qs / ks / ds are rewritten for the next row
  }
  for (int i = 0; i < D; ++i) St[(size_t)i * D + j] = S[i * D + j];
}

// Mamba2 selective state-space recurrence per head: h <- exp(dt A) h + dt B (x) x;  y = C.h + D x, with dt = softplus(raw + bias).
// grid (heads, pieces), block P threads: thread p owns column p of the head's state h[N][P] (shared memory).
// xbc [T, C] holds x (heads * P) | B (groups * N) | C (groups * N) after the convolution; dt_raw is read from `dtm` at dt_col.
template <int P>
__global__ void __launch_bounds__(P) ssd_scan_kernel(const __nv_bfloat16* __restrict__ xbc, const __nv_bfloat16* __restrict__ dtm,
                                                     int ldd, int dt_col, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                     const float* __restrict__ dskip, float* __restrict__ state, int state_rows,
                                                     const int* __restrict__ segs, __nv_bfloat16* __restrict__ out, int nh, int groups, int N) {
  extern __shared__ float sm[];
  float* H = sm;                            // [N][P]
  float* Bs = H + (size_t)N * P;            // [N]
  float* Cs = Bs + N;                       // [N]
  pdl_wait(); pdl_launch();
  const int s = blockIdx.y, h = blockIdx.x, p = threadIdx.x;
  const int first = segs[4 * s], n = segs[4 * s + 1], seq = segs[4 * s + 2], pos0 = segs[4 * s + 3];
  if (n <= 0 || seq < 0 || seq >= state_rows) return;
  float* St = state + ((size_t)seq * nh + h) * N * P;
  for (int i = 0; i < N; ++i) H[i * P + p] = pos0 == 0 ? 0.f : St[(size_t)i * P + p];
  const int I = nh * P, g = h / (nh / groups);
  const size_t C = (size_t)I + 2 * (size_t)groups * N;
  const float A = -__expf(a_log[h]), bias = dt_bias[h], Dh = dskip[h];
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)first + t;
    const __nv_bfloat16* r = xbc + row * C;
    __syncthreads();                        // the previous row's readers are done with Bs / Cs
    for (int i = p; i < N; i += P) { Bs[i] = bf2f(r[I + g * N + i]); Cs[i] = bf2f(r[I + groups * N + g * N + i]); }
    __syncthreads();
    const float xv = bf2f(r[h * P + p]);
    const float raw = bf2f(dtm[row * ldd + dt_col + h]) + bias;
    const float dt = raw > 20.f ? raw : log1pf(__expf(raw));
    const float dA = __expf(dt * A), dx = dt * xv;
    float y = 0.f;
    for (int i = 0; i < N; ++i) {
      const float hv = dA * H[i * P + p] + Bs[i] * dx;
      H[i * P + p] = hv;
      y += Cs[i] * hv;
    }
    out[row * (size_t)I + h * P + p] = __float2bfloat16(y + Dh * xv);
  }
  for (int i = 0; i < N; ++i) St[(size_t)i * P + p] = H[i * P + p];
}

// grid (rows, ceil(heads / 8)), block 256: one warp per (row, head)
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z, int ldz, int z_col,
                                     const __nv_bfloat16* __restrict__ w, int w_per_head, float eps, int gate_first,
                                     __nv_bfloat16* __restrict__ out, int T, int heads, int D) {
  pdl_wait(); pdl_launch();
  const int t = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads) return;
  const __nv_bfloat16* yr = y + ((size_t)t * heads + h) * D;
  const __nv_bfloat16* zr = z + (size_t)t * ldz + z_col + (size_t)h * D;
  __nv_bfloat16* o = out + ((size_t)t * heads + h) * D;
  // gate_first: norm(y * silu(z)) * w (Mamba2, one norm per channel group); else norm(y) * w * silu(z) (gated delta net)
  const __nv_bfloat16* wr = w + (w_per_head ? (size_t)h * D : 0);
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float v = bf2f(yr[i]);
    if (gate_first) v *= silu(bf2f(zr[i]));
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)D + eps);
  for (int i = lane; i < D; i += 32) {
    const float v = bf2f(yr[i]), g = silu(bf2f(zr[i]));
    o[i] = __float2bfloat16(gate_first ? v * g * inv * bf2f(wr[i]) : v * inv * bf2f(wr[i]) * g);
  }
}

__global__ void sigmoid_mul_kernel(__nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ g, size_t n) {
  pdl_wait(); pdl_launch();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    a[i] = __float2bfloat16(bf2f(a[i]) / (1.f + __expf(-bf2f(g[i]))));
}

}  // namespace poot

using namespace poot;

POOT_API int poot_causal_conv_silu(const void* x, int ldx, int col0, int C, int Kc, const float* w, const float* bias, float* state,
                                   int state_rows, const int* segs, int n_segs, void* out, cudaStream_t s) {
  if (n_segs == 0 || C == 0) return 0;
  if (Kc < 2 || Kc > 4 || col0 < 0 || ldx < col0 + C) return (int)cudaErrorInvalidValue;
  dim3 grid((C + 127) / 128, n_segs), block(128);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  __nv_bfloat16* ob = (__nv_bfloat16*)out;
  switch (Kc) {
    case 2: return launch_k(causal_conv_silu_kernel<2>, grid, block, 0, s, xb, ldx, col0, C, w, bias, state, state_rows, segs, ob);
    case 3: return launch_k(causal_conv_silu_kernel<3>, grid, block, 0, s, xb, ldx, col0, C, w, bias, state, state_rows, segs, ob);
    default: return launch_k(causal_conv_silu_kernel<4>, grid, block, 0, s, xb, ldx, col0, C, w, bias, state, state_rows, segs, ob);
  }
}

template <int D>
static int launch_gdn_scan(const void* qkv, const void* ba, int ldb, int b_col, int a_col, const float* dt_bias, const float* a_log,
                           float* state, int state_rows, const int* segs, int n_segs, void* out, int nk, int nv, cudaStream_t s) {
  constexpr size_t smem = ((size_t)D * D + 2 * D + 8) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_scan_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_k(gdn_scan_kernel<D>, dim3(nv, n_segs), dim3(D), smem, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)ba, ldb,
                  b_col, a_col, dt_bias, a_log, state, state_rows, segs, (__nv_bfloat16*)out, nk, nv);
}

POOT_API int poot_gdn_scan(const void* qkv, const void* ba, int ldb, int b_col, int a_col, const float* dt_bias, const float* a_log,
                           float* state, int state_rows, const int* segs, int n_segs, void* out, int nk, int nv, int D,
                           cudaStream_t s) {
  if (n_segs == 0) return 0;
  if (nk < 1 || nv < nk || nv % nk || b_col < 0 || a_col < 0) return (int)cudaErrorInvalidValue;
  if (D == 128) return launch_gdn_scan<128>(qkv, ba, ldb, b_col, a_col, dt_bias, a_log, state, state_rows, segs, n_segs, out, nk, nv, s);
  if (D == 64) return launch_gdn_scan<64>(qkv, ba, ldb, b_col, a_col, dt_bias, a_log, state, state_rows, segs, n_segs, out, nk, nv, s);
  return (int)cudaErrorInvalidValue;
}

template <int D>
static int launch_kda_scan(const void* qkv, const void* f, const void* bm, int ldb, int b_col, const float* dt_bias, const float* a_log,
                           float lower_bound, float* state, int state_rows, const int* segs, int n_segs, void* out, int heads,
                           cudaStream_t s) {
  constexpr size_t smem = ((size_t)D * D + 3 * D + 8) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kda_scan_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_k(kda_scan_kernel<D>, dim3(heads, n_segs), dim3(D), smem, s, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)f,
                  (const __nv_bfloat16*)bm, ldb, b_col, dt_bias, a_log, lower_bound, state, state_rows, segs, (__nv_bfloat16*)out, heads);
}

POOT_API int poot_kda_scan(const void* qkv, const void* f, const void* bm, int ldb, int b_col, const float* dt_bias, const float* a_log,
                           float lower_bound, float* state, int state_rows, const int* segs, int n_segs, void* out, int heads, int D,
                           cudaStream_t s) {
  if (n_segs == 0) return 0;
  if (heads < 1 || b_col < 0 || !(lower_bound < 0.f)) return (int)cudaErrorInvalidValue;
  if (D == 128) return launch_kda_scan<128>(qkv, f, bm, ldb, b_col, dt_bias, a_log, lower_bound, state, state_rows, segs, n_segs, out, heads, s);
  if (D == 64) return launch_kda_scan<64>(qkv, f, bm, ldb, b_col, dt_bias, a_log, lower_bound, state, state_rows, segs, n_segs, out, heads, s);
  return (int)cudaErrorInvalidValue;
}

template <int P>
static int launch_ssd_scan(const void* xbc, const void* dtm, int ldd, int dt_col, const float* dt_bias, const float* a_log,
                           const float* dskip, float* state, int state_rows, const int* segs, int n_segs, void* out, int nh,
                           int groups, int N, cudaStream_t s) {
  const size_t smem = ((size_t)N * P + 2 * (size_t)N) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return launch_k(ssd_scan_kernel<P>, dim3(nh, n_segs), dim3(P), smem, s, (const __nv_bfloat16*)xbc, (const __nv_bfloat16*)dtm, ldd,
                  dt_col, dt_bias, a_log, dskip, state, state_rows, segs, (__nv_bfloat16*)out, nh, groups, N);
}

POOT_API int poot_ssd_scan(const void* xbc, const void* dtm, int ldd, int dt_col, const float* dt_bias, const float* a_log,
                           const float* dskip, float* state, int state_rows, const int* segs, int n_segs, void* out, int nh,
                           int groups, int N, int P, cudaStream_t s) {
  if (n_segs == 0) return 0;
  if (nh < 1 || groups < 1 || nh % groups || N < 1 || dt_col < 0) return (int)cudaErrorInvalidValue;
  if (P == 64) return launch_ssd_scan<64>(xbc, dtm, ldd, dt_col, dt_bias, a_log, dskip, state, state_rows, segs, n_segs, out, nh, groups, N, s);
  if (P == 128) return launch_ssd_scan<128>(xbc, dtm, ldd, dt_col, dt_bias, a_log, dskip, state, state_rows, segs, n_segs, out, nh, groups, N, s);
  if (P == 32) return launch_ssd_scan<32>(xbc, dtm, ldd, dt_col, dt_bias, a_log, dskip, state, state_rows, segs, n_segs, out, nh, groups, N, s);
  return (int)cudaErrorInvalidValue;
}

POOT_API int poot_gated_rmsnorm(const void* y, const void* z, int ldz, int z_col, const void* w, int w_per_head, float eps,
                                int gate_first, void* out, int T, int heads, int D, cudaStream_t s) {
  if (T == 0) return 0;
  if (heads < 1 || D < 1 || z_col < 0) return (int)cudaErrorInvalidValue;
  return launch_k(gated_rmsnorm_kernel, dim3(T, (heads + 7) / 8), dim3(256), 0, s, (const __nv_bfloat16*)y,
                  (const __nv_bfloat16*)z, ldz, z_col, (const __nv_bfloat16*)w, w_per_head, eps, gate_first, (__nv_bfloat16*)out, T,
                  heads, D);
}

POOT_API int poot_sigmoid_mul(void* a, const void* g, long long n, cudaStream_t s) {
  if (n == 0) return 0;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_k(sigmoid_mul_kernel, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)a, (const __nv_bfloat16*)g, (size_t)n);
}
