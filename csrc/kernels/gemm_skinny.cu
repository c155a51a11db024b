// Skinny GEMM for decode batches (1 <= M <= 128 tokens):   out[M,N] = X[M,K] . W[N,K]^T
//
// Decode GEMMs are weight-streaming problems, so the weight is the 128-row MMA operand
// ("swap AB"): one CTA owns 128 weight rows, the few tokens are the MMA N dimension (16..128),
// and a deep TMA ring keeps >= 64 KB of weight bytes in flight per SM.  Small-N projections
// (o_proj, down_proj, qkv) cannot fill 148 SMs with row tiles alone, so a thread-block cluster
// of CK CTAs splits K for one row tile and reduces the fp32 tiles through distributed shared
// memory: no partial buffers in HBM, and the epilogue (bf16 / fp32 store, residual add, SwiGLU
// over interleaved gate/up rows) runs on the reduced values.
//
//   warp 0      TMA producer: weight tiles are requested before griddepcontrol.wait (they do not
//               depend on the previous kernel), activation tiles after it
//   warp 1      TMEM allocator + tcgen05.mma issuer (D[128 x BT] fp32 in TMEM)
//   warps 2..5  TMEM -> shared fp32 tile; after the cluster barrier every CTA reduces its slab
//               of rows over the CK peers with ld.shared::cluster and stores the result
//
// Reference behaviour covered: Contraction::DenseGemv / batched decode GEMM with register epilogues
// (crates/poot-kernelgen/src/contraction/gemv.rs:1-3, contraction/mod.rs:70-84).
#include "tc_common.cuh"
#include "tp_common.cuh"

namespace poot {

enum { SEPI_STORE = 0, SEPI_F32 = 1, SEPI_RESID = 2, SEPI_SWIGLU = 3 };

constexpr int SK_BM = 128;   // weight rows per CTA
constexpr int SK_BK = 64;
constexpr int SK_THREADS = 192;

// Grouped (mixture-of-experts) form: blockIdx.y selects a group; a group multiplies its own X rows / columns with
// one expert's slice of a stacked weight [experts * N, K] and writes its own output slice.
struct GroupArgs {
  const int* group_expert;      // group -> expert id (null: expert = group; a negative id yields zeros)
  int w_rows_per_expert;        // N of one expert inside the stacked weight
  int x_row_div;                // > 0: the group's X rows start at group / x_row_div
  int x_row_mul;                // the group's X rows start at group * x_row_mul (added to the above)
  int x_col_per_expert;         // the group's X columns (K range) start at expert * x_col_per_expert
  long long out_group_stride;   // elements between the outputs of consecutive groups
  const float* row_scale;       // [groups, M] factor applied to each result row (null = 1)
};

__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank)); return r;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v; asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory"); return v;
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

template <int BT, int STAGES, int WM>
struct SkinnySmem {
  static constexpr int W_BYTES = WM * SK_BM * SK_BK * 2;
  static constexpr int X_BYTES = BT * SK_BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int RED_BYTES = BT * WM * SK_BM * 4;
  static constexpr int RING = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = RING > RED_BYTES ? RING : RED_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;
};

template <int BT, int STAGES, int WM, int EPI>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   void* __restrict__ out, const __nv_bfloat16* resid, int M, int N, int K, int ldo, int CK,
                   int* __restrict__ status, const __grid_constant__ TpArgs tp, const __grid_constant__ GroupArgs grp) {
  using S = SkinnySmem<BT, STAGES, WM>;
  constexpr int ROWS = WM * SK_BM;  // weight rows per CTA
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t full_bar = base + S::BAR_OFFSET;
  const uint32_t empty_bar = full_bar + STAGES * 8;
  const uint32_t accum_bar = empty_bar + STAGES * 8;
  const uint32_t tmem_slot = accum_bar + 8;
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(gen_base + S::BAR_OFFSET + (2 * STAGES + 1) * 8);
  float* red = reinterpret_cast<float*>(gen_base);  // [BT][ROWS] fp32, reuses the ring after the last MMA

  __shared__ volatile int s_cta_fail;   // raised by the producer warp when it gives up on its ring
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = CK > 1 ? cluster_ctarank() : 0u;
  const int row_tile = blockIdx.x / CK;
  const int n0 = row_tile * ROWS;
  const int total_kt = (K + SK_BK - 1) / SK_BK;
  const int per = (total_kt + CK - 1) / CK;
  const int kt_begin = (int)crank * per;
  int kt_end = kt_begin + per;
  if (kt_end > total_kt) kt_end = total_kt;
  // grouped form: which expert's weight slice, which X rows / columns, which output slice
  const int grp_id = blockIdx.y;
  int expert = grp_id;
  if (grp.group_expert != nullptr) { pdl_wait(); expert = grp.group_expert[grp_id]; }  // produced by the router kernel
  const bool dead = expert < 0;
  const int w_row0 = (dead ? 0 : expert) * grp.w_rows_per_expert + n0;
  const int x_row0 = (grp.x_row_div > 0 ? grp_id / grp.x_row_div : 0) + grp_id * grp.x_row_mul;
  const int x_col0 = (dead ? 0 : expert) * grp.x_col_per_expert;
  const int num_kt = (dead || kt_end <= kt_begin) ? 0 : kt_end - kt_begin;
  constexpr uint32_t TMEM_COLS = (WM * BT) < 32 ? 32 : (WM * BT);

  if (threadIdx.x == 0) {
    s_cta_fail = 0;
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(full_bar + 8 * s, 1); tc::mbar_init(empty_bar + 8 * s, 1); }
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
      tc::tma_prefetch_desc(&tmW);
      tc::tma_prefetch_desc(&tmX);
      // Weight tiles of the first ring pass do not depend on the previous kernel's output.
      const int pre = num_kt < STAGES ? num_kt : STAGES;
      for (int i = 0; i < pre; ++i) {
        tc::mbar_expect_tx(full_bar + 8 * i, S::STAGE_BYTES);
        tc::tma_load_2d(base + i * S::STAGE_BYTES, &tmW, (kt_begin + i) * SK_BK, w_row0, full_bar + 8 * i);
      }
      pdl_wait();
      const bool gather = tp.world > 1 && tp.ag_site >= 0;
      int xrow = 0;  // row of the activation shard buffers that holds this site's data
      bool ok = true;
      if (gather) {
        const uint32_t target = tp_target(tp, tp.ag_site, tp.ag_sites);
        xrow = (int)(target & 1u) * BT;
        // Every rank pushed its normalised rows into this rank's gather buffer; wait until all have landed.  If a
        // flag does not arrive the cause is recorded and the kernel goes on over whatever the buffer holds: the
        // ring keeps moving, the kernel ends at once and the host sees the failure with the step's result.
        tp_wait_all(tp.flags_local, tp.world, TP_CH_AG, target, tp.ag_site, status);
        fence_proxy_async_global();  // the rows were written with ordinary (peer) stores; TMA reads them
      }
      auto load_x = [&](uint32_t dst, int kx, uint32_t bar) {
        tc::tma_load_2d(dst, &tmX, kx + x_col0, xrow + x_row0, bar);
      };
      for (int i = 0; i < pre; ++i)
        load_x(base + i * S::STAGE_BYTES + S::W_BYTES, (kt_begin + i) * SK_BK, full_bar + 8 * i);
      int issued = pre;
      for (int i = pre; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!tc::mbar_wait(empty_bar + 8 * s, ph ^ 1u)) { ok = false; break; }
        tc::mbar_expect_tx(full_bar + 8 * s, S::STAGE_BYTES);
        const uint32_t sa = base + s * S::STAGE_BYTES;
        const int kx = (kt_begin + i) * SK_BK;
        tc::tma_load_2d(sa, &tmW, kx, w_row0, full_bar + 8 * s);
        load_x(sa + S::W_BYTES, kx, full_bar + 8 * s);
        ++issued;
      }
      if (!ok) {
        s_cta_fail = 1;
        ctl_fail(status, (int)kTimeoutProducer, issued);
        // let the copies already in flight land before the CTA can exit
        for (int j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j)
          tc::mbar_wait(full_bar + 8 * (j % STAGES), (uint32_t)(j / STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(SK_BM, BT);
      bool ok = true;
      for (int i = 0; i < num_kt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        // The first tile arrives only after the producer has passed griddepcontrol.wait and, in the gathered form,
        // its wait for the peers' flags: that wait's limit is the later one.  Once one tile has landed, the rest
        // depends on this CTA's own copies only.
        const bool arrived = (i == 0) ? tc::mbar_wait_dependent(full_bar + 8 * s, ph, status, &s_cta_fail)
                                      : tc::mbar_wait(full_bar + 8 * s, ph);
        if (!arrived) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t sa = base + s * S::STAGE_BYTES;
        const uint64_t xdesc = tc::smem_desc_sw128(sa + S::W_BYTES);
#pragma unroll
        for (int wm = 0; wm < WM; ++wm) {
          const uint64_t wdesc = tc::smem_desc_sw128(sa + wm * (SK_BM * SK_BK * 2));
#pragma unroll
          for (int k = 0; k < SK_BK / 16; ++k)
            tc::mma_bf16_ss(tmem_base + (uint32_t)(wm * BT), wdesc + (uint64_t)(2 * k), xdesc + (uint64_t)(2 * k),
                            idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc::tc_commit(empty_bar + 8 * s);
      }
      if (!ok) ctl_fail(status, (int)kTimeoutMma);
      tc::tc_commit(accum_bar);
    }
  } else {
    // TMEM lane (weight row) quadrant = warp % 4; columns = tokens
    const int quad = warp & 3;
    // (one verdict per warp: the tensor-memory loads below are warp-wide instructions)
    const bool ok = __all_sync(0xffffffffu, tc::mbar_wait_dependent(accum_bar, 0, status, nullptr));
    if (!ok && lane == 0) ctl_fail(status, (int)kTimeoutEpilogue);
    tc::tc_fence_after();
#pragma unroll 1
    // A wait that ran out leaves the ring in an unknown state (copies may still be landing in it): the partial
    // tile is then not written at all, the step is already marked invalid.
    for (int wm = 0; ok && wm < WM; ++wm) {
      const int r = wm * SK_BM + quad * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BT; c0 += 32) {
        uint32_t v[32];
        if (num_kt > 0) {
          // (BT == 16, WM == 1: the allocation is 32 columns wide; the upper 16 are never written by the MMA)
          tc::tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(wm * BT + c0), v);
          tc::tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < BT) red[(c0 + j) * ROWS + r] = __uint_as_float(v[j]);
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (CK > 1) cluster_sync_all();

  // ---- reduce this CTA's slab of rows over the cluster and store ----
  pdl_wait();
  const int slab = ROWS / CK;
  const int slab0 = (int)crank * slab;
  const uint32_t red_s = base;  // shared-window address of red[0]
  const bool scatter = tp.world > 1 && tp.rs_site >= 0;
  const uint32_t rs_target = scatter ? tp_target(tp, tp.rs_site, tp.rs_sites) : 0u;
  const int rs_parity = (int)(rs_target & 1u);
  const int Mv = (scatter && !tp.oneshot) ? BT : (M < BT ? M : BT);
  const size_t out_off = (size_t)grp_id * (size_t)grp.out_group_stride;
  const float* rscale = grp.row_scale ? grp.row_scale + (size_t)grp_id * M : nullptr;
  if (EPI == SEPI_SWIGLU && (slab & 15) == 0 && n0 + slab0 + slab <= N && (ldo & 7) == 0 &&
      (grp.out_group_stride & 7) == 0 && ((uintptr_t)out & 15) == 0) {
    // sixteen interleaved (gate, up) columns per thread -> eight outputs, one 16-byte store
    const int vecs = slab >> 4;
    for (int idx = threadIdx.x; idx < vecs * Mv; idx += SK_THREADS) {
      const int pv = idx % vecs, tok = idx / vecs;
      const int rr = slab0 + 16 * pv;
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
      for (int c = 0; c < CK; ++c) {
        uint32_t a = red_s + (uint32_t)((tok * ROWS + rr) * 4);
        if (CK > 1) a = map_to_cta(a, (uint32_t)c);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float4 t = ld_dsmem_f32x4(a + 16 * q4);
          v[4 * q4] += t.x; v[4 * q4 + 1] += t.y; v[4 * q4 + 2] += t.z; v[4 * q4 + 3] += t.w;
        }
      }
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = silu(v[2 * j]) * v[2 * j + 1];
      const int n = n0 + rr;
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + out_off + (size_t)tok * ldo + (n >> 1)) = pack8(o);
    }
  } else if (EPI == SEPI_SWIGLU) {
    const int hp = slab >> 1;
    for (int idx = threadIdx.x; idx < hp * Mv; idx += SK_THREADS) {
      const int p = idx % hp, tok = idx / hp;
      const int rr = slab0 + 2 * p;
      float g = 0.f, u = 0.f;
      for (int c = 0; c < CK; ++c) {
        uint32_t a = red_s + (uint32_t)((tok * ROWS + rr) * 4);
        if (CK > 1) a = map_to_cta(a, (uint32_t)c);
        g += ld_dsmem_f32(a);
        u += ld_dsmem_f32(a + 4);
      }
      const int n = n0 + rr;
      if (n < N)
        reinterpret_cast<__nv_bfloat16*>(out)[out_off + (size_t)tok * ldo + (n >> 1)] = __float2bfloat16(silu(g) * u);
    }
  } else if ((slab & 7) == 0 && n0 + slab0 + slab <= N && (ldo & 7) == 0 && (grp.out_group_stride & 7) == 0 &&
             (((uintptr_t)out | (uintptr_t)resid) & 15) == 0 && (!scatter || (tp.ld_inbox & 7) == 0)) {
    // eight consecutive output columns per thread: 16-byte loads from the cluster's partial tiles and ONE 16-byte
    // store per destination (a 2-byte store per element and per rank made the collective epilogue the longest
    // part of the kernel)
    const int vecs = slab >> 3;
    for (int idx = threadIdx.x; idx < vecs * Mv; idx += SK_THREADS) {
      const int pv = idx % vecs, tok = idx / vecs;
      const int rr = slab0 + 8 * pv;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      for (int c = 0; c < CK; ++c) {
        uint32_t a = red_s + (uint32_t)((tok * ROWS + rr) * 4);
        if (CK > 1) a = map_to_cta(a, (uint32_t)c);
        const float4 lo = ld_dsmem_f32x4(a), hi = ld_dsmem_f32x4(a + 16);
        v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
        v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
      }
      const int n = n0 + rr;
      if (rscale != nullptr) {
        const float sc = rscale[tok];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= sc;
      }
      if (scatter && tp.oneshot) {
        const uint4 pk = pack8(v);
        const size_t off = ((size_t)((rs_parity * tp.world + tp.rank) * tp.S + tok)) * tp.ld_inbox + n;
        for (int d = 0; d < tp.world; ++d) *reinterpret_cast<uint4*>(tp.inbox_peer[d] + off) = pk;
      } else if (scatter) {
        const int d = tok / tp.S, tl = tok - d * tp.S;
        *reinterpret_cast<uint4*>(tp.inbox_peer[d] + ((size_t)((rs_parity * tp.world + tp.rank) * tp.S + tl)) * tp.ld_inbox + n) =
            pack8(v);
      } else if (EPI == SEPI_F32) {
        float* o = reinterpret_cast<float*>(out) + out_off + (size_t)tok * ldo + n;
        *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + out_off + (size_t)tok * ldo + n;
        if (EPI == SEPI_RESID) {
          float rf[8];
          unpack8(*reinterpret_cast<const uint4*>(resid + out_off + (size_t)tok * ldo + n), rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += rf[j];
        }
        *reinterpret_cast<uint4*>(o) = pack8(v);
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < slab * Mv; idx += SK_THREADS) {
      const int p = idx % slab, tok = idx / slab;
      const int rr = slab0 + p;
      float v = 0.f;
      for (int c = 0; c < CK; ++c) {
        uint32_t a = red_s + (uint32_t)((tok * ROWS + rr) * 4);
        if (CK > 1) a = map_to_cta(a, (uint32_t)c);
        v += ld_dsmem_f32(a);
      }
      const int n = n0 + rr;
      if (rscale != nullptr) v *= rscale[tok];
      if (n < N) {
        if (scatter && tp.oneshot) {
          // one-shot all-reduce: this rank's partial goes to slot `rank` of every rank's inbox
          const __nv_bfloat16 bv = __float2bfloat16(v);
          const size_t off = ((size_t)((rs_parity * tp.world + tp.rank) * tp.S + tok)) * tp.ld_inbox + n;
          for (int d = 0; d < tp.world; ++d) tp.inbox_peer[d][off] = bv;
        } else if (scatter) {
          // reduce-scatter: token row `tok` belongs to rank tok / S; write into that rank's inbox slice for this rank
          const int d = tok / tp.S, tl = tok - d * tp.S;
          tp.inbox_peer[d][((size_t)((rs_parity * tp.world + tp.rank) * tp.S + tl)) * tp.ld_inbox + n] =
              __float2bfloat16(v);
        } else if (EPI == SEPI_F32) {
          reinterpret_cast<float*>(out)[out_off + (size_t)tok * ldo + n] = v;
        } else {
          if (EPI == SEPI_RESID) v += __bfloat162float(resid[out_off + (size_t)tok * ldo + n]);
          reinterpret_cast<__nv_bfloat16*>(out)[out_off + (size_t)tok * ldo + n] = __float2bfloat16(v);
        }
      }
    }
  }
  if (scatter) tp_signal_all(tp, TP_CH_RS, rs_target, (int)gridDim.x, status);
  if (CK > 1) cluster_sync_all();  // no CTA may exit while a peer still reads its tile
}

template <int BT, int STAGES, int WM, int EPI>
static int launch_skinny_cfg(const CUtensorMap& tw, const CUtensorMap& tx, void* out, const void* resid, int M, int N,
                             int K, int ldo, int CK, int pdl, int* status, cudaStream_t s, const TpArgs& tp,
                             const GroupArgs& grp, int groups) {
  using S = SkinnySmem<BT, STAGES, WM>;
  auto kern = gemm_skinny_kernel<BT, STAGES, WM, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int row_tiles = (N + WM * SK_BM - 1) / (WM * SK_BM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(row_tiles * CK, groups, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (CK > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = CK; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl || g_poot_pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return (int)cudaLaunchKernelEx(&cfg, kern, tw, tx, out, (const __nv_bfloat16*)resid, M, N, K, ldo, CK, status, tp, grp);
}

template <int BT, int STAGES, int WM>
static int launch_skinny_epi(int epi, const CUtensorMap& tw, const CUtensorMap& tx, void* out, const void* resid,
                             int M, int N, int K, int ldo, int CK, int pdl, int* status, cudaStream_t s,
                             const TpArgs& tp, const GroupArgs& grp, int groups) {
  switch (epi) {
    case SEPI_STORE: return launch_skinny_cfg<BT, STAGES, WM, SEPI_STORE>(tw, tx, out, resid, M, N, K, ldo, CK, pdl, status, s, tp, grp, groups);
    case SEPI_F32: return launch_skinny_cfg<BT, STAGES, WM, SEPI_F32>(tw, tx, out, resid, M, N, K, ldo, CK, pdl, status, s, tp, grp, groups);
    case SEPI_RESID: return launch_skinny_cfg<BT, STAGES, WM, SEPI_RESID>(tw, tx, out, resid, M, N, K, ldo, CK, pdl, status, s, tp, grp, groups);
    case SEPI_SWIGLU: return launch_skinny_cfg<BT, STAGES, WM, SEPI_SWIGLU>(tw, tx, out, resid, M, N, K, ldo, CK, pdl, status, s, tp, grp, groups);
    default: return (int)cudaErrorInvalidValue;
  }
}

static int skinny_dispatch(int epi, const CUtensorMap& tw, const CUtensorMap& tx, void* out, const void* resid, int M,
                           int N, int K, int ldo, int ck, int bt, int pdl, int* status, cudaStream_t s, const TpArgs& tp,
                           const GroupArgs& grp = GroupArgs{}, int groups = 1) {
  switch (bt) {
    case 16: return launch_skinny_epi<16, 6, 1>(epi, tw, tx, out, resid, M, N, K, ldo, ck, pdl, status, s, tp, grp, groups);
    case 32: return launch_skinny_epi<32, 5, 1>(epi, tw, tx, out, resid, M, N, K, ldo, ck, pdl, status, s, tp, grp, groups);
    case 64: return launch_skinny_epi<64, 4, 1>(epi, tw, tx, out, resid, M, N, K, ldo, ck, pdl, status, s, tp, grp, groups);
    case 128: return launch_skinny_epi<128, 3, 1>(epi, tw, tx, out, resid, M, N, K, ldo, ck, pdl, status, s, tp, grp, groups);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace poot

using namespace poot;

// X [M, ldx] bf16 with M <= 128, W [N, K] bf16, out [M, ldo].  ck = cluster size (K split): 1, 2, 4 or 8.
// pdl != 0 launches with programmatic stream serialization (the kernel waits on its predecessor itself).
POOT_API int poot_gemm_skinny(int epi, const void* x, const void* W, void* out, const void* resid, int M, int N, int K,
                              int ldx, int ldo, int ck, int wm, int pdl, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K % 8 || ldx % 8 || wm != 1) return (int)cudaErrorInvalidValue;
  if (ck != 1 && ck != 2 && ck != 4 && ck != 8) return (int)cudaErrorInvalidValue;
  if (epi == SEPI_SWIGLU && (N % 2)) return (int)cudaErrorInvalidValue;
  if (epi == SEPI_RESID && resid == nullptr) return (int)cudaErrorInvalidValue;
  if (status == nullptr) return (int)cudaErrorInvalidValue;
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap tw, tx;
  int e = make_tmap_bf16_2d(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)SK_BM);
  if (e) return e;
  e = make_tmap_bf16_2d(&tx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)bt);
  if (e) return e;
  TpArgs tp = {};
  tp.world = 1; tp.ag_site = -1; tp.rs_site = -1;
  return skinny_dispatch(epi, tw, tx, out, resid, M, N, K, ldo, ck, bt, pdl, status, s, tp);
}

// Tensor-parallel form.  The step has world*S padded token rows (16, 32, 64 or 128).
//   ag_site >= 0: X is this rank's gather buffer `x` ([2 * world*S, K] bf16, double-buffered on the site parity) into
//                 which every rank pushed its normalised rows; the producer warp waits for all ranks' flags of the
//                 site before its first activation load.  Otherwise X is `x` ([world*S, ldx], local data).
//   rs_site >= 0: output rows are scattered (bf16) to their owner ranks' inboxes and the site is signalled;
//                 otherwise the epilogue `epi` writes to `out` locally.
POOT_API int poot_gemm_skinny_tp(int epi, const void* x, const void* W, void* out, int N, int K, int ldx, int ldo,
                                 int ck, int world, int rank, int S, int ag_site, int ag_sites, int rs_site,
                                 int rs_sites, const int* epoch, void* flags_local, void* const* flags_peer,
                                 void* const* inbox_peer, int ld_inbox, int oneshot_rows, int* ticket, int* status,
                                 cudaStream_t s) {
  // oneshot_rows > 0: one-shot all-reduce form over that many (unpadded) token rows; X is local, S = rows per slot.
  if (world < 2 || world > TP_MAX_WORLD || K % 8) return (int)cudaErrorInvalidValue;
  if (!oneshot_rows && S % 8) return (int)cudaErrorInvalidValue;
  if (oneshot_rows && (ag_site >= 0 || oneshot_rows > S || oneshot_rows > 128)) return (int)cudaErrorInvalidValue;
  const int M = oneshot_rows ? oneshot_rows : world * S;
  const int bt = oneshot_rows ? (M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128))) : world * S;
  if (bt != 16 && bt != 32 && bt != 64 && bt != 128) return (int)cudaErrorInvalidValue;
  if (ck != 1 && ck != 2 && ck != 4 && ck != 8) return (int)cudaErrorInvalidValue;
  if (status == nullptr || epoch == nullptr) return (int)cudaErrorInvalidValue;
  if (rs_site >= 0 && epi != SEPI_STORE) return (int)cudaErrorInvalidValue;
  CUtensorMap tw, tx;
  int e = make_tmap_bf16_2d(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)SK_BM);
  if (e) return e;
  if (ag_site >= 0) {
    e = make_tmap_bf16_2d(&tx, x, (uint64_t)(2 * bt), (uint64_t)K, (uint64_t)K, (uint32_t)bt);
    if (e) return e;
  } else {
    e = make_tmap_bf16_2d(&tx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, (uint32_t)bt);
    if (e) return e;
  }
  TpArgs tp = {};
  tp.oneshot = oneshot_rows ? 1 : 0;
  tp.world = world; tp.rank = rank; tp.S = S;
  tp.ag_site = ag_site; tp.ag_sites = ag_sites; tp.rs_site = rs_site; tp.rs_sites = rs_sites;
  tp.ld_inbox = ld_inbox; tp.epoch = epoch; tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
  for (int r = 0; r < world; ++r) {
    tp.flags_peer[r] = (uint32_t*)flags_peer[r];
    tp.inbox_peer[r] = inbox_peer ? (__nv_bfloat16*)inbox_peer[r] : nullptr;
  }
  return skinny_dispatch(epi, tw, tx, out, nullptr, M, N, K, ldo, ck, bt, 0, status, s, tp);
}

// Grouped (mixture-of-experts) form over a stacked weight W [experts * N, K]: `groups` independent problems, group g
// uses expert group_expert[g] (or g), X rows starting at g / x_row_div + g * x_row_mul, X columns starting at
// expert * x_col_per_expert (X is [*, ldx]), and writes out + g * out_group_stride.  row_scale [groups, M] (optional)
// multiplies each result row (the routing gate).  With tp_world > 1 and rs_site >= 0 the result goes to every rank's
// inbox as a one-shot all-reduce contribution (expert parallelism: the combine is the reduction over experts).
POOT_API int poot_gemm_skinny_grouped(int epi, const void* x, int x_rows, int x_cols, int ldx, const void* W,
                                      int experts, void* out, int M, int N, int K, int ldo, int ck, int groups,
                                      const int* group_expert, int x_row_div, int x_row_mul, int x_col_per_expert,
                                      long long out_group_stride, const float* row_scale, int* status,
                                      int tp_world, int tp_rank, int slot_rows, int rs_site, int rs_sites,
                                      const int* epoch, void* flags_local, void* const* flags_peer,
                                      void* const* inbox_peer, int ld_inbox, int* ticket, cudaStream_t s) {
  if (M <= 0 || N <= 0 || groups <= 0) return 0;
  if (M > 128 || K % 8 || ldx % 8) return (int)cudaErrorInvalidValue;
  if (ck != 1 && ck != 2 && ck != 4 && ck != 8) return (int)cudaErrorInvalidValue;
  if (status == nullptr) return (int)cudaErrorInvalidValue;
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap tw, tx;
  int e = make_tmap_bf16_2d(&tw, W, (uint64_t)experts * (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)SK_BM);
  if (e) return e;
  e = make_tmap_bf16_2d(&tx, x, (uint64_t)x_rows, (uint64_t)x_cols, (uint64_t)ldx, (uint32_t)bt);
  if (e) return e;
  TpArgs tp = {};
  tp.world = 1; tp.ag_site = -1; tp.rs_site = -1;
  if (tp_world > 1 && rs_site >= 0) {
    if (groups != 1 || epi != SEPI_STORE) return (int)cudaErrorInvalidValue;
    tp.world = tp_world; tp.rank = tp_rank; tp.S = slot_rows; tp.oneshot = 1; tp.rs_site = rs_site; tp.rs_sites = rs_sites;
    tp.ld_inbox = ld_inbox; tp.epoch = epoch; tp.flags_local = (uint32_t*)flags_local; tp.ticket = ticket;
    for (int r = 0; r < tp_world; ++r) {
      tp.flags_peer[r] = (uint32_t*)flags_peer[r];
      tp.inbox_peer[r] = (__nv_bfloat16*)inbox_peer[r];
    }
  }
  GroupArgs grp = {};
  grp.group_expert = group_expert; grp.w_rows_per_expert = N; grp.x_row_div = x_row_div; grp.x_row_mul = x_row_mul;
  grp.x_col_per_expert = x_col_per_expert; grp.out_group_stride = out_group_stride; grp.row_scale = row_scale;
  return skinny_dispatch(epi, tw, tx, out, nullptr, M, N, K, ldo, ck, bt, 0, status, s, tp, grp, groups);
}
