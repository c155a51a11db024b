// Decode GEMV / skinny GEMM over a checkpoint-order bf16 weight W[N,K]:
//   out[m, n] = sum_k x[m, k] * W[n, k]        for 1 <= m <= 4
// Memory-bound: every weight byte is read once with 16-byte streaming loads,
// eight loads in flight per lane, fp32 accumulation, warp-shuffle reduction.
//
// Epilogues (in registers, no extra pass over memory):
//   EPI_STORE   out bf16
//   EPI_F32     out fp32 (logits)
//   EPI_RESID   out = resid + acc (bf16; out may alias resid)
//   EPI_SWIGLU  weight rows interleaved (2j = gate_j, 2j+1 = up_j): out[m, j] = silu(g)*u
//
// Reference behaviour covered: Contraction::DenseGemv and its register
// epilogues (crates/poot-kernelgen/src/contraction/gemv.rs:1-3,
// crates/poot-graph-plan/src/passes/fuse.rs ContractionEpilogue).
#include "common.cuh"

namespace poot {

enum { EPI_STORE = 0, EPI_F32 = 1, EPI_RESID = 2, EPI_SWIGLU = 3 };

constexpr int GEMV_WARPS = 4;
constexpr int GEMV_ROWS = 2;  // weight rows per warp step

template <int M, int EPI>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                 void* __restrict__ out, const __nv_bfloat16* __restrict__ resid, int N, int K,
                 int ldx, int ldo) {
  pdl_wait(); pdl_launch();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * GEMV_WARPS + warp;
  const int nwarps = gridDim.x * GEMV_WARPS;
  const int K8 = K >> 3;  // 16-byte chunks per row

  for (int pair = gwarp; pair * GEMV_ROWS < N; pair += nwarps) {
    const int n0 = pair * GEMV_ROWS;
    const uint4* w0 = reinterpret_cast<const uint4*>(W + (size_t)n0 * K);
    const uint4* w1 = reinterpret_cast<const uint4*>(W + (size_t)(n0 + 1 < N ? n0 + 1 : n0) * K);
    float acc[M][GEMV_ROWS];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m][0] = 0.f; acc[m][1] = 0.f; }

    int c = lane;
    // main loop: 4 chunks x 2 rows = 8 loads in flight per lane
    for (; c + 96 < K8; c += 128) {
      uint4 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) { a[u] = ld_stream16(w0 + c + 32 * u); b[u] = ld_stream16(w1 + c + 32 * u); }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float fa[8], fb[8];
        unpack8(a[u], fa); unpack8(b[u], fb);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          float fx[8];
          unpack8(ld_cached16(reinterpret_cast<const uint4*>(x + (size_t)m * ldx) + c + 32 * u), fx);
#pragma unroll
          for (int j = 0; j < 8; ++j) { acc[m][0] += fa[j] * fx[j]; acc[m][1] += fb[j] * fx[j]; }
        }
      }
    }
    for (; c < K8; c += 32) {
      float fa[8], fb[8];
      unpack8(ld_stream16(w0 + c), fa); unpack8(ld_stream16(w1 + c), fb);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float fx[8];
        unpack8(ld_cached16(reinterpret_cast<const uint4*>(x + (size_t)m * ldx) + c), fx);
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc[m][0] += fa[j] * fx[j]; acc[m][1] += fb[j] * fx[j]; }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) { acc[m][0] = warp_sum(acc[m][0]); acc[m][1] = warp_sum(acc[m][1]); }

    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (EPI == EPI_SWIGLU) {
          // rows (n0, n0+1) are (gate_j, up_j) with j = n0/2
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + (n0 >> 1)] =
              __float2bfloat16(silu(acc[m][0]) * acc[m][1]);
        } else {
#pragma unroll
          for (int r = 0; r < GEMV_ROWS; ++r) {
            int n = n0 + r;
            if (n >= N) break;
            float v = acc[m][r];
            if (EPI == EPI_F32) {
              reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
            } else {
              if (EPI == EPI_RESID) v += __bfloat162float(resid[(size_t)m * ldo + n]);
              reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
  }
}

template <int M>
static int launch_gemv(int epi, const void* x, const void* W, void* out, const void* resid, int N, int K,
                       int ldx, int ldo, cudaStream_t s) {
  int pairs = (N + GEMV_ROWS - 1) / GEMV_ROWS;
  int blocks = (pairs + GEMV_WARPS - 1) / GEMV_WARPS;
  int cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  dim3 g(blocks), b(GEMV_WARPS * 32);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)W;
  const __nv_bfloat16* rb = (const __nv_bfloat16*)resid;
  switch (epi) {
    case EPI_STORE: return launch_k(gemv_bf16_kernel<M, EPI_STORE>, g, b, 0, s, (const __nv_bfloat16*)xb, (const __nv_bfloat16*)wb, out, (const __nv_bfloat16*)rb, N, K, ldx, ldo);
    case EPI_F32: return launch_k(gemv_bf16_kernel<M, EPI_F32>, g, b, 0, s, (const __nv_bfloat16*)xb, (const __nv_bfloat16*)wb, out, (const __nv_bfloat16*)rb, N, K, ldx, ldo);
    case EPI_RESID: return launch_k(gemv_bf16_kernel<M, EPI_RESID>, g, b, 0, s, (const __nv_bfloat16*)xb, (const __nv_bfloat16*)wb, out, (const __nv_bfloat16*)rb, N, K, ldx, ldo);
    case EPI_SWIGLU: return launch_k(gemv_bf16_kernel<M, EPI_SWIGLU>, g, b, 0, s, (const __nv_bfloat16*)xb, (const __nv_bfloat16*)wb, out, (const __nv_bfloat16*)rb, N, K, ldx, ldo);
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

}  // namespace poot

using namespace poot;

// x [M, ldx] bf16, W [N, K] bf16, out [M, ldo] (bf16 or fp32 by epilogue).  K % 8 == 0, M <= 4.
POOT_API int poot_gemv_bf16(int epi, const void* x, const void* W, void* out, const void* resid, int M, int N,
                            int K, int ldx, int ldo, cudaStream_t s) {
  if (K % 8 || ldx % 8 || M < 1 || M > 4) return (int)cudaErrorInvalidValue;
  if (epi == EPI_SWIGLU && (N % 2)) return (int)cudaErrorInvalidValue;
  if (epi == EPI_RESID && resid == nullptr) return (int)cudaErrorInvalidValue;
  switch (M) {
    case 1: return launch_gemv<1>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    case 2: return launch_gemv<2>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    case 3: return launch_gemv<3>(epi, x, W, out, resid, N, K, ldx, ldo, s);
    default: return launch_gemv<4>(epi, x, W, out, resid, N, K, ldx, ldo, s);
  }
}
