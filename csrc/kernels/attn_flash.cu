// Flash attention for prefill pieces over the paged K/V cache on the 5th-generation tensor cores (head_dim 128).
//
// One CTA owns a tile of up to 128 consecutive query tokens of ONE sequence and one query head, and walks the
// sequence's keys 128 at a time:
//     S = Q K^T          tcgen05.mma, Q and K both K-major (D contiguous), accumulator in tensor memory
//     P = softmax piece  128 threads, one query row each, read S from tensor memory, write P (bf16) to shared
//                        memory in the K-major 128-byte-swizzled layout the next MMA reads
//     O_t = P V          tcgen05.mma with V as an MN-major operand: V stays [key][D] as the cache stores it
//     acc = acc * alpha + O_t   in registers (online softmax)
// K and V arrive page by page (16 keys) with plain tiled TMA loads through the sequence's block table into a
// two-stage ring, so the next tile's pages are in flight while this tile is computed.  Warp roles: warp 0 issues
// TMA, warp 1 owns tensor memory and issues MMAs, warps 2..5 do the softmax.  Every wait is bounded; a wait that runs
// out records a status word, and the CTA still reaches the common tail that frees tensor memory.
//
// Reference behaviour covered: the Attention composite's flash pipeline with a causal (optionally windowed) mask,
// GQA head mapping and paged keys (crates/poot-kernelgen/src/attention.rs:1-52,
// crates/poot-graph-plan/src/planner/attention.rs:305-347).
#include "tc_common.cuh"

namespace poot {

constexpr int FA_D = 128;          // head_dim
constexpr int FA_BM = 128;         // query rows per tile
constexpr int FA_BN = 128;         // keys per step
constexpr int FA_PAGE = 16;        // keys per cache block
constexpr int FA_THREADS = 192;
constexpr int FA_HALF = 128 * 128; // bytes of one [128 rows x 64 bf16] swizzled slab
constexpr int FA_TILE = 2 * FA_HALF;

struct FaSmem {
  static constexpr int Q = 0;
  static constexpr int K = Q + FA_TILE;              // 2 stages
  static constexpr int V = K + 2 * FA_TILE;          // 2 stages
  static constexpr int P = V + 2 * FA_TILE;
  static constexpr int BARS = P + FA_TILE;
  static constexpr int NBARS = 12;
  static constexpr int TOTAL = BARS + NBARS * 8 + 16 + 1024;
};

// MN-major operand, 128-byte swizzle: 64 elements (128 B) contiguous along MN, 8 K-rows of 128 B per atom,
// atoms along K `sbo` bytes apart, the next 64 MN-elements `lbo` bytes away.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
attn_flash_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const int* __restrict__ block_tables,
                          int max_blocks, const int4* __restrict__ tiles, __nv_bfloat16* __restrict__ out,
                          int out_stride, int Hq, int Hkv, float scale, int window, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  pdl_wait(); pdl_launch();
  const int4 tile = tiles[blockIdx.x];       // (first token row, tokens, block-table row, position of the first token)
  const int n_tok = tile.y;
  if (n_tok <= 0) return;                    // unused tile slot (uniform for the CTA; nothing allocated yet)
  const int tok0 = tile.x, seq = tile.z, pos0 = tile.w;
  const int head = blockIdx.y;
  const int kvh = head / (Hq / Hkv);

  const uint32_t raw = tc::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t bars = base + FaSmem::BARS;
  const uint32_t bar_q = bars, full_k = bars + 8, empty_k = bars + 24, full_v = bars + 40, empty_v = bars + 56;
  const uint32_t bar_s = bars + 72, bar_p = bars + 80, bar_o = bars + 88;
  const uint32_t tmem_slot = bars + FaSmem::NBARS * 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + FaSmem::BARS + FaSmem::NBARS * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_end = pos0 + n_tok;                                   // keys [0, kv_end) can be visible
  const int t_begin = window > 0 ? max(0, pos0 - window + 1) / FA_BN : 0;
  const int t_end = (kv_end + FA_BN - 1) / FA_BN;
  const int n_tiles = t_end - t_begin;

  if (threadIdx.x == 0) {
    tc::mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(full_k + 8 * s, 1); tc::mbar_init(empty_k + 8 * s, 1);
      tc::mbar_init(full_v + 8 * s, 1); tc::mbar_init(empty_v + 8 * s, 1);
    }
    tc::mbar_init(bar_s, 1); tc::mbar_init(bar_p, 4); tc::mbar_init(bar_o, 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, 256);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmK); tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(bar_q, FA_TILE);
      tc::tma_load_2d(base + FaSmem::Q, &tmQ, head * FA_D, tok0, bar_q);
      tc::tma_load_2d(base + FaSmem::Q + FA_HALF, &tmQ, head * FA_D + 64, tok0, bar_q);
      const int* bt = block_tables + (size_t)seq * max_blocks;
      bool ok = true;
      int issued_k = 0, issued_v = 0;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        const int page0 = (t_begin + i) * (FA_BN / FA_PAGE);
        // the tile's eight block ids are independent loads issued together, ahead of the wait for a free stage
        int ys[FA_BN / FA_PAGE];
#pragma unroll
        for (int p = 0; p < FA_BN / FA_PAGE; ++p) {
          int pg = page0 + p; if (pg >= max_blocks) pg = max_blocks - 1;
          ys[p] = __ldg(bt + pg);
        }
#pragma unroll
        for (int p = 0; p < FA_BN / FA_PAGE; ++p) ys[p] = (ys[p] * Hkv + kvh) * FA_PAGE;
        if (!tc::mbar_wait(empty_k + 8 * s, ph ^ 1u)) { ok = false; break; }
        tc::mbar_expect_tx(full_k + 8 * s, FA_TILE);
#pragma unroll
        for (int p = 0; p < FA_BN / FA_PAGE; ++p) {
          const int y = ys[p];
          const uint32_t dst = base + FaSmem::K + s * FA_TILE + p * (FA_PAGE * 128);
          tc::tma_load_2d(dst, &tmK, 0, y, full_k + 8 * s);
          tc::tma_load_2d(dst + FA_HALF, &tmK, 64, y, full_k + 8 * s);
        }
        ++issued_k;
        if (!tc::mbar_wait(empty_v + 8 * s, ph ^ 1u)) { ok = false; break; }
        tc::mbar_expect_tx(full_v + 8 * s, FA_TILE);
#pragma unroll
        for (int p = 0; p < FA_BN / FA_PAGE; ++p) {
          const int y = ys[p];
          const uint32_t dst = base + FaSmem::V + s * FA_TILE + p * (FA_PAGE * 128);
          tc::tma_load_2d(dst, &tmV, 0, y, full_v + 8 * s);
          tc::tma_load_2d(dst + FA_HALF, &tmV, 64, y, full_v + 8 * s);
        }
        ++issued_v;
      }
      if (!ok) {
        ctl_fail(status, (int)kTimeoutProducer);
        // let the copies already in flight land before the CTA can exit
        for (int j = (issued_k > 2 ? issued_k - 2 : 0); j < issued_k; ++j)
          tc::mbar_wait(full_k + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
        for (int j = (issued_v > 2 ? issued_v - 2 : 0); j < issued_v; ++j)
          tc::mbar_wait(full_v + 8 * (j & 1), (uint32_t)(j >> 1) & 1u);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::idesc_bf16_f32(FA_BM, FA_BN);
      constexpr uint32_t idesc_o = tc::idesc_bf16_f32(FA_BM, FA_D) | (1u << 16);   // B (= V) is MN-major
      bool ok = tc::mbar_wait(bar_q, 0);
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!tc::mbar_wait(full_k + 8 * s, ph)) { ok = false; break; }
        tc::tc_fence_after();
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          const uint64_t a = tc::smem_desc_sw128(base + FaSmem::Q + (k >> 2) * FA_HALF) + (uint64_t)(2 * (k & 3));
          const uint64_t b = tc::smem_desc_sw128(base + FaSmem::K + s * FA_TILE + (k >> 2) * FA_HALF) + (uint64_t)(2 * (k & 3));
          tc::mma_bf16_ss(tmem_s, a, b, idesc_s, k > 0 ? 1u : 0u);
        }
        tc::tc_commit(bar_s);
        tc::tc_commit(empty_k + 8 * s);
        if (!tc::mbar_wait(bar_p, (uint32_t)i & 1u)) { ok = false; break; }
        if (!tc::mbar_wait(full_v + 8 * s, ph)) { ok = false; break; }
        tc::tc_fence_after();
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint64_t a = tc::smem_desc_sw128(base + FaSmem::P + (k >> 2) * FA_HALF) + (uint64_t)(2 * (k & 3));
          const uint64_t b = smem_desc_mn_sw128(base + FaSmem::V + s * FA_TILE + k * (16 * 128), FA_HALF, 1024);
          tc::mma_bf16_ss(tmem_o, a, b, idesc_o, k > 0 ? 1u : 0u);
        }
        tc::tc_commit(bar_o);
        tc::tc_commit(empty_v + 8 * s);
      }
      if (!ok) ctl_fail(status, (int)kTimeoutMma);
    }
  } else {
    // ---------------- softmax: thread <-> query row (tensor-memory lane) ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const int pos = pos0 + row;
    const float c1 = scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[FA_D];
#pragma unroll
    for (int j = 0; j < FA_D; ++j) acc[j] = 0.f;
    uint8_t* p_row = gen + FaSmem::P + row * 128;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      const int key0 = (t_begin + i) * FA_BN;
      if (!tc::mbar_wait(bar_s, (uint32_t)i & 1u)) { ok = false; break; }
      tc::tc_fence_after();
      const bool need_mask = (key0 + FA_BN - 1 > pos0) || window > 0;
      // pass 1: row maximum
      float m_new = m_run;
#pragma unroll 1
      for (int c = 0; c < FA_BN; c += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_s + lane_base + (uint32_t)c, r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = __uint_as_float(r[j]);
          if (need_mask) {
            const int key = key0 + c + j;
            if (key > pos || (window > 0 && key <= pos - window)) v = -INFINITY;
          }
          m_new = fmaxf(m_new, v);
        }
      }
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f((m_run - m_use) * c1);     // m_run = -inf on the first tile: alpha = 0
      float l_tile = 0.f;
      // pass 2: probabilities, written as the next MMA's A operand (K-major, 128-byte swizzle)
#pragma unroll 1
      for (int c = 0; c < FA_BN; c += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_s + lane_base + (uint32_t)c, r);
        tc::tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = __uint_as_float(r[j]);
          if (need_mask) {
            const int key = key0 + c + j;
            if (key > pos || (window > 0 && key <= pos - window)) v = -INFINITY;
          }
          p[j] = exp2f((v - m_use) * c1);
          l_tile += p[j];
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const int chunk16 = (c >> 3) + v4;                 // 16-byte chunk index along the 128 keys
          const int half = chunk16 >> 3, cc = chunk16 & 7;
          *reinterpret_cast<uint4*>(p_row + half * FA_HALF + ((cc ^ (row & 7)) << 4)) = pack8(p + 8 * v4);
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_use == 0.f && m_new == -INFINITY ? -INFINITY : m_use;
      tc::tc_fence_before();
      tc::fence_proxy_async();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(bar_p);
      // O_t = P V lands in tensor memory; fold it into the running output
      if (!tc::mbar_wait(bar_o, (uint32_t)i & 1u)) { ok = false; break; }
      tc::tc_fence_after();
#pragma unroll
      for (int c = 0; c < FA_D; c += 32) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_o + lane_base + (uint32_t)c, r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c + j] = acc[c + j] * alpha + __uint_as_float(r[j]);
      }
      tc::tc_fence_before();
    }
    if (!ok && lane == 0) ctl_fail(status, (int)kTimeoutEpilogue);
    if (ok && row < n_tok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)head * FA_D;
#pragma unroll
      for (int c = 0; c < FA_D; c += 8) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = acc[c + j] * inv;
        *reinterpret_cast<uint4*>(orow + c) = pack8(f);
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace poot

using namespace poot;

// q [rows, Hq*128] bf16 (row pitch q_stride), pools [num_blocks, Hkv, 16, 128] bf16, tiles [n_tiles] of
// (first row, tokens, block-table row, first position); tiles with tokens == 0 are skipped.
POOT_API int poot_attn_flash_prefill(const void* q, int q_stride, int q_rows, const void* kpool, const void* vpool,
                                     long long num_blocks, const int* block_tables, int max_blocks, const int* tiles,
                                     int n_tiles, void* out, int out_stride, int Hq, int Hkv, float scale, int window,
                                     int* status, cudaStream_t s) {
  if (n_tiles <= 0) return 0;
  if (Hq % Hkv || q_stride % 8 || out_stride % 8 || status == nullptr) return (int)cudaErrorInvalidValue;
  CUtensorMap tq, tk, tv;
  int e = make_tmap_bf16_2d(&tq, q, (uint64_t)q_rows, (uint64_t)Hq * FA_D, (uint64_t)q_stride, FA_BM);
  if (e) return e;
  const uint64_t pool_rows = (uint64_t)num_blocks * Hkv * FA_PAGE;
  e = make_tmap_bf16_2d(&tk, kpool, pool_rows, FA_D, FA_D, FA_PAGE);
  if (e) return e;
  e = make_tmap_bf16_2d(&tv, vpool, pool_rows, FA_D, FA_D, FA_PAGE);
  if (e) return e;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          FaSmem::TOTAL);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  return launch_k(attn_flash_prefill_kernel, dim3(n_tiles, Hq), dim3(FA_THREADS), (size_t)FaSmem::TOTAL, s, tq, tk, tv,
                  block_tables, max_blocks, reinterpret_cast<const int4*>(tiles), (__nv_bfloat16*)out, out_stride, Hq,
                  Hkv, scale, window, status);
}
