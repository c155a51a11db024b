// Dequant-fused skinny GEMM over GGUF block-quantised weights:  out[M, N] = X[M, K] . dequant(W)[N, K]^T  for decode
// batches of 5 to 128 rows.  The packed weight is read once from HBM in its checkpoint layout and never exists as
// bf16 outside shared memory: the four warps that will later run the epilogue first decode each 128 x 64 weight tile
// (one weight row per thread, eight values per decoder call) straight into the ring stage in the 128-byte-swizzled
// K-major layout the tensor core reads, while one lane of warp 0 streams the activation tile with TMA and one lane of
// warp 1 issues tcgen05.mma with the accumulators in tensor memory (swap-AB: weight rows are the 128-row operand, the
// step's tokens the N dimension, as in gemm_skinny.cu).  A stage is full when the activation bytes have landed AND the
// decoders have arrived; it is released by the MMA's commit.
//
// One CTA per 128 weight rows, no split over K (a cluster split like the bf16 kernel's is the next step).
// Reference behaviour covered: Contraction::Packed for batched decode (crates/poot-kernelgen/src/packed/mod.rs:1-7).
#include "tc_common.cuh"
#include "quant_decode.cuh"

namespace poot {

enum { QSEPI_STORE = 0, QSEPI_F32 = 1, QSEPI_RESID = 2, QSEPI_SWIGLU = 3 };
constexpr int QS_BM = 128;
constexpr int QS_BK = 64;
constexpr int QS_THREADS = 192;
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);

template <int BT, int STAGES>
struct QsSmem {
  static constexpr int W_BYTES = QS_BM * QS_BK * 2;
  static constexpr int X_BYTES = BT * QS_BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;
};

template <int BT, int STAGES, int EPI>
__global__ void __launch_bounds__(QS_THREADS)
gemm_skinny_quant_kernel(const __grid_constant__ CUtensorMap tmX, const uint8_t* __restrict__ Wq, int fmt, long long row_bytes,
                         void* __restrict__ out, const __nv_bfloat16* __restrict__ resid, int M, int N, int K, int ldo,
                         int* __restrict__ status) {
  using S = QsSmem<BT, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t full_bar = base + S::BAR_OFFSET;
  const uint32_t empty_bar = full_bar + STAGES * 8;
  const uint32_t accum_bar = empty_bar + STAGES * 8;
  const uint32_t tmem_slot = accum_bar + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + (2 * STAGES + 1) * 8);
  __shared__ volatile int s_cta_fail;
  __shared__ volatile int s_go;              // one decoder thread's verdict on the ring slot, read by all of them

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * QS_BM;
  const int num_kt = (K + QS_BK - 1) / QS_BK;
  constexpr uint32_t TMEM_COLS = BT < 32 ? 32 : BT;

  if (threadIdx.x == 0) {
    s_cta_fail = 0;
    for (int s = 0; s < STAGES; ++s) {
      tc::mbar_init(full_bar + 8 * s, 2);      // the activation copy's arrive.expect_tx + the decoders' arrive
      tc::mbar_init(empty_bar + 8 * s, 1);
    }
    tc::mbar_init(accum_bar, 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  pdl_launch();

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmX);
      pdl_wait();                                   // the activations are the previous kernel's output
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!tc::mbar_wait(empty_bar + 8 * s, ph ^ 1u)) { ok = false; break; }
        tc::mbar_expect_tx(full_bar + 8 * s, S::X_BYTES);
        tc::tma_load_2d(base + s * S::STAGE_BYTES + S::W_BYTES, &tmX, i * QS_BK, 0, full_bar + 8 * s);
        ++issued;
      }
      if (!ok) {
        s_cta_fail = 1;
        ctl_fail(status, (int)kTimeoutProducer, issued);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(QS_BM, BT);
      bool ok = true;
      for (int i = 0; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        // the first stage fills only after the producer has passed its wait for the previous kernel
        const bool arrived = (i == 0) ? tc::mbar_wait_dependent(full_bar + 8 * s, ph, status, &s_cta_fail)
                                      : tc::mbar_wait(full_bar + 8 * s, ph);
        if (!arrived) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t sa = base + s * S::STAGE_BYTES;
        const uint64_t wdesc = tc::smem_desc_sw128(sa);
        const uint64_t xdesc = tc::smem_desc_sw128(sa + S::W_BYTES);
#pragma unroll
        for (int k = 0; k < QS_BK / 16; ++k)
          tc::mma_bf16_ss(tmem_base, wdesc + (uint64_t)(2 * k), xdesc + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc::tc_commit(empty_bar + 8 * s);
      }
      if (!ok) ctl_fail(status, (int)kTimeoutMma);
      tc::tc_commit(accum_bar);
    }
  } else {
    // ---- decoders (warps 2..5, 128 threads: thread t owns weight row n0 + t of every tile) ----
    const int t = threadIdx.x - 64;
    const int n = n0 + t;
    const uint8_t* wrow = Wq + (size_t)(n < N ? n : 0) * (size_t)row_bytes;
    bool live = true;
    for (int i = 0; i < num_kt; ++i) {
      const int s = i % STAGES;
      const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
      // One thread waits for the slot and all take its verdict: 128 separate bounded waits could disagree at the limit,
      // and a thread that left the loop alone would strand the others at the group barrier below.
      if (t == 0) s_go = tc::mbar_wait(empty_bar + 8 * s, ph ^ 1u) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (s_go == 0) { live = false; break; }
      // the weights do not depend on the previous kernel: decoding runs ahead of the dependency wait
      uint8_t* tile = gen_base + s * S::STAGE_BYTES;
#pragma unroll
      for (int c = 0; c < QS_BK / 8; ++c) {
        const int k = i * QS_BK + c * 8;
        float f[8];
        if (live && n < N && k < K) {
          float q[8], scale, offset;
          if (!decode8_rt(fmt, wrow, k, q, scale, offset)) {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = 0.f;
            scale = 0.f; offset = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = scale * q[j] - offset;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = 0.f;
        }
        // K-major tile with 128-byte rows, 16-byte chunks XOR-swizzled by the row's low three bits (SWIZZLE_128B)
        *reinterpret_cast<uint4*>(tile + t * 128 + ((c ^ (t & 7)) << 4)) = pack8(f);
      }
      tc::fence_proxy_async();                       // generic-proxy stores -> visible to the tensor core's async proxy
      asm volatile("bar.sync 1, 128;" ::: "memory"); // the four decoder warps
      if (t == 0) tc::mbar_arrive(full_bar + 8 * s);
    }
    if (!live && t == 0) { s_cta_fail = 1; ctl_fail(status, (int)kTimeoutProducer, -1); }

    // ---- epilogue: TMEM lane (weight row) quadrant = warp % 4; columns = tokens ----
    const int quad = warp & 3;
    const int r = n0 + quad * 32 + lane;             // this thread's output column (weight row)
    const bool ok = __all_sync(0xffffffffu, tc::mbar_wait_dependent(accum_bar, 0, status, nullptr));
    if (!ok && lane == 0) ctl_fail(status, (int)kTimeoutEpilogue);
    tc::tc_fence_after();
    pdl_wait();                                      // `out` and `resid` may belong to the previous kernel until it is done
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        uint32_t v[32];
        tc::tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int tok = c0 + j;
          if (tok >= BT) break;
          float a = __uint_as_float(v[j]);
          if (EPI == QSEPI_SWIGLU) {
            // interleaved rows: even lanes hold the gate, odd lanes the up value of the same output column
            const float up = __shfl_down_sync(0xffffffffu, a, 1);
            if (tok < M && !(lane & 1) && r < N)
              reinterpret_cast<__nv_bfloat16*>(out)[(size_t)tok * ldo + (r >> 1)] = __float2bfloat16(silu(a) * up);
          } else if (tok < M && r < N) {
            const size_t o = (size_t)tok * ldo + r;
            if (EPI == QSEPI_F32) reinterpret_cast<float*>(out)[o] = a;
            else {
              if (EPI == QSEPI_RESID) a += __bfloat162float(resid[o]);
              reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16(a);
            }
          }
        }
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BT, int STAGES, int EPI>
static int launch_qs_cfg(const CUtensorMap& tx, const void* Wq, int fmt, long long row_bytes, void* out, const void* resid,
                         int M, int N, int K, int ldo, int* status, cudaStream_t s) {
  using S = QsSmem<BT, STAGES>;
  auto kern = gemm_skinny_quant_kernel<BT, STAGES, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_k(kern, dim3((N + QS_BM - 1) / QS_BM), dim3(QS_THREADS), (size_t)S::TOTAL, s, tx, (const uint8_t*)Wq, fmt,
                  row_bytes, out, (const __nv_bfloat16*)resid, M, N, K, ldo, status);
}

template <int BT, int STAGES>
static int launch_qs_epi(int epi, const CUtensorMap& tx, const void* Wq, int fmt, long long row_bytes, void* out,
                         const void* resid, int M, int N, int K, int ldo, int* status, cudaStream_t s) {
  switch (epi) {
    case QSEPI_STORE: return launch_qs_cfg<BT, STAGES, QSEPI_STORE>(tx, Wq, fmt, row_bytes, out, resid, M, N, K, ldo, status, s);
    case QSEPI_F32: return launch_qs_cfg<BT, STAGES, QSEPI_F32>(tx, Wq, fmt, row_bytes, out, resid, M, N, K, ldo, status, s);
    case QSEPI_RESID: return launch_qs_cfg<BT, STAGES, QSEPI_RESID>(tx, Wq, fmt, row_bytes, out, resid, M, N, K, ldo, status, s);
    case QSEPI_SWIGLU: return launch_qs_cfg<BT, STAGES, QSEPI_SWIGLU>(tx, Wq, fmt, row_bytes, out, resid, M, N, K, ldo, status, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace poot

using namespace poot;

// fmt = ggml type id.  x [M, ldx] bf16 with M <= 128, W packed [N rows of K values], out [M, ldo].
//   epi 0 bf16 store, 1 fp32 store, 2 bf16 residual add, 3 SwiGLU over interleaved (gate, up) rows (N / 2 outputs).
POOT_API int poot_quant_gemm_skinny(int fmt, int epi, const void* x, const void* Wq, void* out, const void* resid, int M, int N,
                                    int K, int ldx, int ldo, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  const size_t rb = quant_row_bytes(fmt, K);
  if (rb == 0 || M > 128 || K % 32 || ldx % 8 || status == nullptr) return (int)cudaErrorInvalidValue;
  if ((fmt == QF_Q4_K || fmt == QF_Q5_K || fmt == QF_Q6_K || fmt == QF_Q2_K || fmt == QF_Q3_K || fmt == QF_IQ4_XS) && K % 256)
    return (int)cudaErrorInvalidValue;
  if (epi == QSEPI_SWIGLU && (N % 2)) return (int)cudaErrorInvalidValue;
  if (epi == QSEPI_RESID && resid == nullptr) return (int)cudaErrorInvalidValue;
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap tx;
  int e = make_tmap_bf16_2d(&tx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)bt);
  if (e) return e;
  switch (bt) {
    case 16: return launch_qs_epi<16, 6>(epi, tx, Wq, fmt, (long long)rb, out, resid, M, N, K, ldo, status, s);
    case 32: return launch_qs_epi<32, 5>(epi, tx, Wq, fmt, (long long)rb, out, resid, M, N, K, ldo, status, s);
    case 64: return launch_qs_epi<64, 4>(epi, tx, Wq, fmt, (long long)rb, out, resid, M, N, K, ldo, status, s);
    default: return launch_qs_epi<128, 3>(epi, tx, Wq, fmt, (long long)rb, out, resid, M, N, K, ldo, status, s);
  }
}
