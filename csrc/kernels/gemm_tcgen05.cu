// bf16 GEMM on the 5th-generation tensor cores:   out[M,N] = X[M,K] . W[N,K]^T
//
// W is the checkpoint-order weight ([out, in], K contiguous), X the activations, so both
// operands are K-major and stream through TMA as 128-byte-swizzled 64-column tiles.
// One CTA owns a 128 x BN output tile (and one K split of it):
//   warp 0      TMA producer (one lane): fills a STAGES-deep shared-memory ring
//   warp 1      TMEM allocator + MMA issuer (one lane): tcgen05.mma 128xBNx16, fp32 in TMEM,
//               tcgen05.commit releases each ring slot and finally signals the epilogue
//   warps 2..5  epilogue: tcgen05.ld of their 32 TMEM lanes, fused epilogue, vector stores
// Rows of X beyond M and rows of W beyond N are zero-filled by TMA and masked on store.
//
// Epilogues: bf16 store, fp32 store (logits), residual add, SwiGLU over interleaved
// gate/up weight rows, and fp32 split-K partial slices (reduced by the consumer kernel).
//
// Reference behaviour covered: Contraction::DenseTiled over an [N,K] weight with register
// epilogues (crates/poot-kernelgen/src/contraction/tiled.rs:1-6,
// crates/poot-graph-plan/src/passes/fuse.rs ContractionEpilogue).  The reference lowers this
// family to wmma m16n16k16 for sm_80; this file is the sm_100a design.
#include "tc_common.cuh"
#include "tp_common.cuh"
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <cstring>

namespace poot {

// ---------------------------------------------------------------------------
// Host: tensor-map creation (driver entry point resolved lazily; cached per operand)
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct TmapKey {
  const void* base; uint64_t rows, cols, ld; uint32_t box_rows;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ k.rows; h = h * 1000003u ^ k.cols; h = h * 1000003u ^ k.ld; h = h * 1000003u ^ k.box_rows;
    return h;
  }
};

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapHash> cache;
  static std::mutex mu;
  TmapKey key{base, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return (int)cudaErrorNotSupported;
  if (((uintptr_t)base & 15) || (ld * 2) % 16) return (int)cudaErrorInvalidValue;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
  {
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return 0;
}

// ---------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------
enum { GEPI_STORE = 0, GEPI_F32 = 1, GEPI_RESID = 2, GEPI_SWIGLU = 3, GEPI_PARTIAL = 4 };

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;  // +1024 for base alignment
};

// Grouped form (mixture of experts over rows grouped by expert): row tile blockIdx.x belongs to expert
// tile_expert[blockIdx.x] of a stacked weight [experts * N, K]; a negative entry is an unused tile (nothing is stored).
// row_scale (optional) multiplies each stored row (the routing gate of the down projection).
struct TileGroups {
  const int* tile_expert;
  int w_rows_per_expert;
  const float* row_scale;
};

// Tensor-parallel form (prefill-sized steps of the token-sharded program, more than 128 padded rows): the policy type
// carries the peer pointers.  With ag_site >= 0 the X operand is this rank's gather buffer [2][world * S][K] (every rank
// pushed its normalised rows into it): the producer waits for the ranks' flags of the site, then loads tiles of the
// buffer half the site's parity names (plain TMA loads of local memory, no multicast).  With rs_site >= 0 the bf16
// result is not stored locally: each output row goes to the inbox of the rank that owns the token row
// (row / S), into this rank's slot, and the last CTA publishes the site's flag - GEMM + reduce-scatter in one kernel;
// the consumer is the same reduce + norm kernel as for decode-sized steps.
struct NoTp {};
__device__ __forceinline__ void gemm_fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

template <int BN, int STAGES, int EPI, bool GROUPED = false, typename TP = NoTp>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         void* __restrict__ out, const __nv_bfloat16* __restrict__ resid, int M, int N, int K,
                         int ldo, int k_tiles_per_split, long long partial_stride, int* __restrict__ status,
                         const TileGroups grp, const __grid_constant__ TP tp) {
  constexpr bool kTp = !std::is_same<TP, NoTp>::value;
  using S = GemmSmem<BN, STAGES>;
  __shared__ volatile int s_cta_fail;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t full_bar = base + S::BAR_OFFSET;
  const uint32_t empty_bar = full_bar + STAGES * 8;
  const uint32_t accum_bar = empty_bar + STAGES * 8;
  const uint32_t tmem_slot = accum_bar + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + (2 * STAGES + 1) * 8);

  pdl_wait(); pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * GEMM_BM;
  const int n0 = blockIdx.y * BN;
  const int split = blockIdx.z;
  const int total_k_tiles = (K + GEMM_BK - 1) / GEMM_BK;
  const int kt_begin = split * k_tiles_per_split;
  int kt_end = kt_begin + k_tiles_per_split;
  if (kt_end > total_k_tiles) kt_end = total_k_tiles;
  int num_kt = kt_end > kt_begin ? kt_end - kt_begin : 0;
  int w_n0 = n0;            // row of the weight operand this tile starts at
  bool dead = false;        // grouped form: a row tile no expert owns
  if (GROUPED) {
    const int ex = grp.tile_expert[blockIdx.x];
    dead = ex < 0;
    w_n0 = (dead ? 0 : ex) * grp.w_rows_per_expert + n0;
    if (dead) num_kt = 0;
  }

  if (threadIdx.x == 0) {
    s_cta_fail = 0;
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(full_bar + 8 * s, 1); tc::mbar_init(empty_bar + 8 * s, 1); }
    tc::mbar_init(accum_bar, 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, BN < 32 ? 32 : BN);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmB);
      int issued = 0;
      bool ok = true;
      int a_row0 = m0;
      if constexpr (kTp) {
        if (tp.world > 1 && tp.ag_site >= 0) {
          const uint32_t target = tp_target(tp, tp.ag_site, tp.ag_sites);
          a_row0 = (int)(target & 1u) * (tp.world * tp.S) + m0;
          // If a flag does not arrive the cause is recorded and the kernel goes on over whatever the buffer holds: the
          // ring keeps moving, the kernel ends at once and the host sees the failure with the step's result.
          tp_wait_all(tp.flags_local, tp.world, TP_CH_AG, target, tp.ag_site, status);
          gemm_fence_proxy_async_global();   // the rows were written with ordinary (peer) stores; TMA reads them
        }
      }
      for (int i = 0; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!tc::mbar_wait(empty_bar + 8 * s, ph ^ 1u)) { ok = false; break; }
        tc::mbar_expect_tx(full_bar + 8 * s, S::STAGE_BYTES);
        const uint32_t sa = base + s * S::STAGE_BYTES;
        const int kx = (kt_begin + i) * GEMM_BK;
        tc::tma_load_2d(sa, &tmA, kx, a_row0, full_bar + 8 * s);
        tc::tma_load_2d(sa + S::A_BYTES, &tmB, kx, w_n0, full_bar + 8 * s);
        ++issued;
      }
      if (!ok) {
        s_cta_fail = 1;
        ctl_fail(status, (int)kTimeoutProducer);
        // let the copies already in flight land before the CTA can exit
        for (int j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j)
          tc::mbar_wait(full_bar + 8 * (j % STAGES), (uint32_t)(j / STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(GEMM_BM, BN);
      bool ok = true;
      for (int i = 0; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        // gathered form: the first tile arrives only after the producer's wait for the peers' flags, whose limit is the
        // step deadline; this wait's limit is the later one
        const bool arrived = (kTp && i == 0) ? tc::mbar_wait_dependent(full_bar + 8 * s, ph, status, &s_cta_fail)
                                             : tc::mbar_wait(full_bar + 8 * s, ph);
        if (!arrived) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t sa = base + s * S::STAGE_BYTES;
        const uint64_t adesc = tc::smem_desc_sw128(sa);
        const uint64_t bdesc = tc::smem_desc_sw128(sa + S::A_BYTES);
#pragma unroll
        for (int k = 0; k < GEMM_BK / 16; ++k) {
          // +32 bytes per K step of 16 bf16 = +2 in the 16-byte-unit address field
          tc::mma_bf16_ss(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                          (i > 0 || k > 0) ? 1u : 0u);
        }
        tc::tc_commit(empty_bar + 8 * s);
      }
      if (!ok) ctl_fail(status, (int)kTimeoutMma);
      tc::tc_commit(accum_bar);  // arrives once every MMA issued above has completed
    }
  } else {
    // ---- epilogue warps: TMEM lane quadrant = warp % 4 ----
    const int quad = warp & 3;
    const int row = m0 + quad * 32 + lane;
    // one verdict per warp (the tensor-memory loads below are warp-wide instructions)
    const bool ok = __all_sync(0xffffffffu, kTp ? tc::mbar_wait_dependent(accum_bar, 0, status, nullptr)
                                               : tc::mbar_wait(accum_bar, 0));
    if (!ok && lane == 0) ctl_fail(status, (int)kTimeoutEpilogue);
    tc::tc_fence_after();
    bool scatter = false;
    __nv_bfloat16* peer_row = nullptr;       // this output row in its owner's inbox (scattered form)
    if constexpr (kTp) {
      scatter = tp.world > 1 && tp.rs_site >= 0 && EPI == GEPI_STORE;
      if (scatter && row < M) {
        const int parity = (int)(tp_target(tp, tp.rs_site, tp.rs_sites) & 1u);
        const int owner = row / tp.S, local = row - owner * tp.S;
        peer_row = tp.inbox_peer[owner] + ((size_t)((parity * tp.world + tp.rank) * tp.S + local)) * tp.ld_inbox;
      }
    }
    if (ok && !dead) {
      const float rs = (GROUPED && grp.row_scale != nullptr && row < M) ? grp.row_scale[row] : 1.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        if (num_kt > 0) {
          tc::tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
          tc::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int n = n0 + c0;
        if (row < M && n < N) {
          if (EPI == GEPI_SWIGLU) {
            // columns (2j, 2j+1) = (gate_j, up_j); output column (n/2 + j)
            __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldo + (n >> 1);
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              if (n + 16 * v < N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float g = __uint_as_float(r[16 * v + 2 * j]), u = __uint_as_float(r[16 * v + 2 * j + 1]);
                  f[j] = silu(g) * u;
                }
                *reinterpret_cast<uint4*>(orow + 8 * v) = pack8(f);
              }
            }
          } else if (EPI == GEPI_F32 || EPI == GEPI_PARTIAL) {
            float* orow = reinterpret_cast<float*>(out) + (EPI == GEPI_PARTIAL ? (size_t)split * partial_stride : 0) +
                          (size_t)row * ldo + n;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (n + 4 * v < N) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                *reinterpret_cast<float4*>(orow + 4 * v) = o;
              }
            }
          } else {
            __nv_bfloat16* orow = scatter ? peer_row + n : reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * ldo + n;
            const __nv_bfloat16* rrow = resid + (size_t)row * ldo + n;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (n + 8 * v < N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * v + j]);
                if (GROUPED) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] *= rs;
                }
                if (EPI == GEPI_RESID) {
                  float rf[8];
                  unpack8(*reinterpret_cast<const uint4*>(rrow + 8 * v), rf);
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] += rf[j];
                }
                *reinterpret_cast<uint4*>(orow + 8 * v) = pack8(f);
              }
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
    tc::tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
  }
  if constexpr (kTp) {
    // every CTA arrives (all threads: the call contains a barrier); the last one publishes the site's flag everywhere
    if (tp.world > 1 && tp.rs_site >= 0 && EPI == GEPI_STORE)
      tp_signal_all(tp, TP_CH_RS, tp_target(tp, tp.rs_site, tp.rs_sites), (int)(gridDim.x * gridDim.y * gridDim.z), status);
  }
}

template <int BN, int STAGES, int EPI>
static int launch_gemm_cfg(const CUtensorMap& ta, const CUtensorMap& tb, void* out, const void* resid, int M, int N,
                           int K, int ldo, int splits, long long partial_stride, int* status, cudaStream_t s) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int total_kt = (K + GEMM_BK - 1) / GEMM_BK;
  int per = (total_kt + splits - 1) / splits;
  dim3 grid((M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN, splits);
  return launch_k(kern, grid, dim3(GEMM_THREADS), (size_t)S::TOTAL, s, ta, tb, out, (const __nv_bfloat16*)resid, M, N, K,
                  ldo, per, partial_stride, status, TileGroups{nullptr, 0, nullptr}, NoTp{});
}

template <int BN, int STAGES>
static int launch_gemm_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, void* out, const void* resid, int M,
                           int N, int K, int ldo, int splits, long long partial_stride, int* status, cudaStream_t s) {
  switch (epi) {
    case GEPI_STORE: return launch_gemm_cfg<BN, STAGES, GEPI_STORE>(ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case GEPI_F32: return launch_gemm_cfg<BN, STAGES, GEPI_F32>(ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case GEPI_RESID: return launch_gemm_cfg<BN, STAGES, GEPI_RESID>(ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case GEPI_SWIGLU: return launch_gemm_cfg<BN, STAGES, GEPI_SWIGLU>(ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case GEPI_PARTIAL: return launch_gemm_cfg<BN, STAGES, GEPI_PARTIAL>(ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

template <int BN, int STAGES, int EPI>
static int launch_gemm_grouped_cfg(const CUtensorMap& ta, const CUtensorMap& tb, void* out, int M, int N, int K, int ldo,
                                   const TileGroups& grp, int* status, cudaStream_t s) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, EPI, true>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int total_kt = (K + GEMM_BK - 1) / GEMM_BK;
  dim3 grid((M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN, 1);
  return launch_k(kern, grid, dim3(GEMM_THREADS), (size_t)S::TOTAL, s, ta, tb, out, (const __nv_bfloat16*)nullptr, M, N, K,
                  ldo, total_kt, 0LL, status, grp, NoTp{});
}

template <int EPI>
static int launch_gemm_tp_cfg(const CUtensorMap& ta, const CUtensorMap& tb, void* out, int M, int N, int K, int ldo,
                              const TpArgs& tp, int* status, cudaStream_t s) {
  constexpr int BN = 128, STAGES = 3;
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, STAGES, EPI, false, TpArgs>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int total_kt = (K + GEMM_BK - 1) / GEMM_BK;
  dim3 grid((M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN, 1);
  return launch_k(kern, grid, dim3(GEMM_THREADS), (size_t)S::TOTAL, s, ta, tb, out, (const __nv_bfloat16*)nullptr, M, N, K,
                  ldo, total_kt, 0LL, status, TileGroups{nullptr, 0, nullptr}, tp);
}

}  // namespace poot

using namespace poot;

// Grouped tiled GEMM over rows grouped by expert (see moe_align): X [M, ldx] with M = tiles * 128 grouped rows, stacked
// weight W [experts * N, K], out [M, ldo]; row tile t multiplies with expert tile_expert[t] (negative: unused, nothing is
// stored).  epi 0 (bf16 store, optional row_scale [M]) or 3 (SwiGLU over interleaved gate / up rows).  N % 128 == 0.
POOT_API int poot_gemm_grouped_tiled(int epi, const void* x, const void* W, void* out, int M, int N, int K, int ldx,
                                     int ldo, int experts, const int* tile_expert, const float* row_scale, int* status,
                                     cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M % GEMM_BM || N % 128 || K % 8 || ldx % 8 || ldo % 8 || experts < 1) return (int)cudaErrorInvalidValue;
  if (epi != GEPI_STORE && epi != GEPI_SWIGLU) return (int)cudaErrorInvalidValue;
  if (tile_expert == nullptr || status == nullptr) return (int)cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  int e = make_tmap_bf16_2d(&ta, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, GEMM_BM);
  if (e) return e;
  e = make_tmap_bf16_2d(&tb, W, (uint64_t)experts * (uint64_t)N, (uint64_t)K, (uint64_t)K, 128u);
  if (e) return e;
  TileGroups grp{tile_expert, N, row_scale};
  if (epi == GEPI_SWIGLU) return launch_gemm_grouped_cfg<128, 3, GEPI_SWIGLU>(ta, tb, out, M, N, K, ldo, grp, status, s);
  return launch_gemm_grouped_cfg<128, 3, GEPI_STORE>(ta, tb, out, M, N, K, ldo, grp, status, s);
}

// X [M, ldx] bf16 (ldx >= K), W [N, K] bf16, out [M, ldo].
//   epi 0 bf16 store, 1 fp32 store, 2 bf16 residual add (resid has the layout of out),
//       3 SwiGLU (out is [M, ldo] with N/2 valid columns), 4 fp32 split-K partials
//       (out is [splits, M, ldo] fp32 with slice stride partial_stride elements).
//   bn: 64, 128 or 256.  splits > 1 only with epi 4.  status: device int, set non-zero on a wait timeout.
POOT_API int poot_gemm_bf16_tcgen05(int epi, const void* x, const void* W, void* out, const void* resid, int M, int N,
                                    int K, int ldx, int ldo, int bn, int splits, long long partial_stride,
                                    int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 || ldx % 8 || N % 8 || ldo % 4) return (int)cudaErrorInvalidValue;
  if ((epi == GEPI_STORE || epi == GEPI_RESID || epi == GEPI_SWIGLU) && ldo % 8) return (int)cudaErrorInvalidValue;
  if (epi == GEPI_SWIGLU && N % 16) return (int)cudaErrorInvalidValue;
  if (splits < 1 || (splits > 1 && epi != GEPI_PARTIAL)) return (int)cudaErrorInvalidValue;
  if (epi == GEPI_RESID && resid == nullptr) return (int)cudaErrorInvalidValue;
  if (status == nullptr) return (int)cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  int e = make_tmap_bf16_2d(&ta, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, GEMM_BM);
  if (e) return e;
  e = make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)bn);
  if (e) return e;
  switch (bn) {
    case 64: return launch_gemm_epi<64, 4>(epi, ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case 128: return launch_gemm_epi<128, 3>(epi, ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    case 256: return launch_gemm_epi<256, 4>(epi, ta, tb, out, resid, M, N, K, ldo, splits, partial_stride, status, s);
    default: return (int)cudaErrorInvalidValue;
  }
}

// Tiled GEMM of the token-sharded tensor-parallel program for steps above 128 padded rows (see the policy comment at
// the kernel).  M = world * S padded rows, a multiple of 128.
//   ag_site >= 0: `x` is this rank's gather buffer [2 * M, K] bf16 (double-buffered on the site's parity, row pitch ldx).
//   rs_site >= 0: epi must be 0; the result rows go to the owner ranks' inboxes [2][world][S][ld_inbox] and `out` is unused.
//   epi 0 bf16 store, 1 fp32 store (logits), 3 SwiGLU.
POOT_API int poot_gemm_tiled_tp(int epi, const void* x, const void* W, void* out, int N, int K, int ldx, int ldo,
                                int tp_world, int tp_rank, int S_rows, int ag_site, int ag_sites, int rs_site, int rs_sites,
                                const int* epoch, void* flags_local, void* const* flags_peer, void* const* inbox_peer,
                                int ld_inbox, int* ticket, int* status, cudaStream_t s) {
  const int M = tp_world * S_rows;
  if (tp_world < 2 || tp_world > TP_MAX_WORLD || tp_rank < 0 || tp_rank >= tp_world || S_rows < 1 || M % GEMM_BM)
    return (int)cudaErrorInvalidValue;
  if (N <= 0 || N % 8 || K % 8 || ldx % 8 || status == nullptr || epoch == nullptr || ticket == nullptr)
    return (int)cudaErrorInvalidValue;
  if (epi != GEPI_STORE && epi != GEPI_F32 && epi != GEPI_SWIGLU) return (int)cudaErrorInvalidValue;
  if (rs_site >= 0 && (epi != GEPI_STORE || inbox_peer == nullptr || ld_inbox % 8 || ld_inbox < N)) return (int)cudaErrorInvalidValue;
  if (rs_site < 0 && (out == nullptr || ldo % (epi == GEPI_F32 ? 4 : 8))) return (int)cudaErrorInvalidValue;
  if (epi == GEPI_SWIGLU && N % 16) return (int)cudaErrorInvalidValue;
  TpArgs tp = {};
  tp.world = tp_world; tp.rank = tp_rank; tp.S = S_rows; tp.ag_site = ag_site; tp.ag_sites = ag_sites; tp.rs_site = rs_site;
  tp.rs_sites = rs_sites; tp.ld_inbox = ld_inbox; tp.epoch = epoch; tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
  for (int r = 0; r < tp_world; ++r) {
    tp.flags_peer[r] = (uint32_t*)flags_peer[r];
    tp.inbox_peer[r] = inbox_peer ? (__nv_bfloat16*)inbox_peer[r] : nullptr;
  }
  CUtensorMap ta, tb;
  int e = make_tmap_bf16_2d(&ta, x, (uint64_t)(ag_site >= 0 ? 2 * M : M), (uint64_t)K, (uint64_t)ldx, GEMM_BM);
  if (e) return e;
  e = make_tmap_bf16_2d(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128u);
  if (e) return e;
  switch (epi) {
    case GEPI_STORE: return launch_gemm_tp_cfg<GEPI_STORE>(ta, tb, out, M, N, K, ldo, tp, status, s);
    case GEPI_F32: return launch_gemm_tp_cfg<GEPI_F32>(ta, tb, out, M, N, K, ldo, tp, status, s);
    default: return launch_gemm_tp_cfg<GEPI_SWIGLU>(ta, tb, out, M, N, K, ldo, tp, status, s);
  }
}
