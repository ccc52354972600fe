// Fused landmark attention for sm_100a: TMA-fed tcgen05 MMAs with TMEM accumulators.
//
// Shape contract: bf16 / fp16, head dim 128, landmark block 64, Lq a multiple of 128, Lk a multiple of 64.
//
// Forward, one CTA per (128 query rows, batch*head); rows 0-63 belong to landmark block `own0`, rows 64-127 to
// `own0 + 1`.  Warps 0-3 run the softmax (thread = query row = TMEM lane), warp 4 issues TMA loads, warp 5 issues
// the MMAs and owns the TMEM allocation.
//   1. Pre-pass: S_lm = Q . K_lm^T against the landmark keys only (every 64th key, fetched with a strided 5-D TMA box)
//      gives each row the maximum landmark score of its earlier blocks.  Together with the row maximum of the
//      own (diagonal) block, which is processed first, this is the FINAL maximum of the outer softmax, so the O
//      accumulator in TMEM is never rescaled.
//   2. Main loop over key blocks n = own0+1 ... 0:  S = Q . K_n^T (N = 64);  the softmax threads read S from TMEM,
//      form the block's weights  p_j = softmax_inside_block(s)_j * exp(l_n - m)  (own block: exp(s_j - m), causal),
//      write them as bf16 into the shared-memory slot the K block just vacated (128-byte swizzled, K-major), and
//      O += P . V_n runs with V as an MN-major operand straight from its row-major TMA tile.
//   3. Epilogue: O / l -> global, plus the statistics L = l, M = m the backward pass needs.
// Reference semantics: llama/ltriton/flash_landmark_attention.py:6-122.
//
// Backward is recompute-based and atomic-free (bit-reproducible), in three launches:
//   a. delta = rowsum(O * dO)                                              (:125-149, without the 1/L pre-scaling)
//   b. dK/dV: one CTA per (key block of 64, batch*head) loops over the query tiles that see the block.  Per tile:
//      S = Q K^T and dP = dO V^T into TMEM; the softmax threads rebuild P and dS (bf16, [128 q x 64 k] swizzled tiles);
//      dV^T += dO^T P and dK^T += Q^T dS accumulate TRANSPOSED ([128 features x 64 keys], M = 128) so that every MMA
//      keeps the full 128-lane shape; dO, Q, P and dS are consumed as MN-major operands from their row-major tiles.
//   c. dQ: one CTA per (128 query rows, batch*head) loops over the key blocks like the forward pass:
//      S, dP -> dS (written over the V tile, which dP no longer needs) -> dQ += dS K with K as an MN-major operand.
//   Per tile pair: earlier block  dS_j = g s_j (dP_j - nD) scale,  dS_landmark = g (nD - delta) scale,  P_j = g s_j,
//   with s = softmax inside the block, g = exp(l_n - M) / L, nD = sum_j s_j dP_j;  own block: p = exp(S - M) / L,
//   dS = p (dP - delta) scale.                                                                      (:152-305)
#include "common.cuh"
#include "attn_params.h"
#include "sm100_ptx.cuh"

namespace lmk {

__device__ int g_lmk_status = 0;   // first bounded wait that expired (0 = none); see lmk_device_status()

namespace {

using namespace ptx;

constexpr int kD = 128;
constexpr int kBlk = 64;
constexpr int kQTile = 128;
constexpr int kFwdStages = 2;
constexpr int kFwdThreads = 192;
constexpr uint32_t kTileBytes = 16384;   // one [128 x 64] or two [64 x 64] 16-bit tiles
constexpr uint32_t kHalfTile = 8192;
constexpr float kLog2e = 1.4426950408889634f;

// error sites reported through g_lmk_status
enum { kErrFwdProducer = 101, kErrFwdMma = 102, kErrFwdSoftmax = 103, kErrFwdEpilogue = 104 };

struct FwdSmem {
  // tile storage is addressed manually from the 1024-byte aligned base; this struct holds the barriers only
  uint64_t q_full;
  uint64_t full[kFwdStages];
  uint64_t empty[kFwdStages];
  uint64_t p_ready[kFwdStages];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t o_full;
  uint32_t tmem_base;
};

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (kBf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

// write one row (64 16-bit values, given as 32 packed words) of a [128 x 64] K-major 128B-swizzled tile
__device__ __forceinline__ void store_row_sw128(uint32_t tile_base, int row, const uint32_t (&w)[32]) {
  const uint32_t row_addr = tile_base + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t addr = row_addr + ((c ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * c]), "r"(w[4 * c + 1]),
                 "r"(w[4 * c + 2]), "r"(w[4 * c + 3])
                 : "memory");
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 2)
sm100_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_klm,
                 void* __restrict__ o_ptr, float* __restrict__ L_ptr, float* __restrict__ M_ptr, int H, int Lq, int Lk,
                 int lm_box, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t q_tile = base;                                        // 32 KB: two [128 x 64] sub-tiles
  auto k_slot = [&](int s) { return base + 32768u + (uint32_t)s * 32768u; };   // 16 KB: K block, later P
  auto v_slot = [&](int s) { return base + 32768u + (uint32_t)s * 32768u + 16384u; };
  FwdSmem* sm = reinterpret_cast<FwdSmem*>(smem_raw + (base - raw) + 32768u + kFwdStages * 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQTile;
  const int t = n_tiles - 1 - (int)blockIdx.x;          // heaviest tiles first
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int own0 = prefix_blocks + 2 * t;               // block of rows 0-63; rows 64-127 own own0+1
  const int n_last = own0 + 1;
  const int n_lm_tiles = (n_last + 63) / 64;            // landmarks 0 .. n_last-1
  const int total = n_lm_tiles + n_last + 1;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->q_full), 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
      mbar_init(smem_u32(&sm->p_ready[s]), 128);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sm->s_full[s]), 1);
      mbar_init(smem_u32(&sm->s_free[s]), 128);
    }
    mbar_init(smem_u32(&sm->o_full), 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_u32(&sm->tmem_base), 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 128;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_klm);
      const uint32_t qb = smem_u32(&sm->q_full);
      mbar_arrive_expect_tx(qb, 2 * kTileBytes);
      tma_load_4d(q_tile, &tm_q, qb, 0, t * kQTile, h, b);
      tma_load_4d(q_tile + kTileBytes, &tm_q, qb, 64, t * kQTile, h, b);
      for (int i = 0; i < total; ++i) {
        const int s = i % kFwdStages;
        const uint32_t ph = (i / kFwdStages) & 1;
        mbar_wait(smem_u32(&sm->empty[s]), ph ^ 1, &g_lmk_status, kErrFwdProducer);
        const uint32_t fb = smem_u32(&sm->full[s]);
        if (i < n_lm_tiles) {
          // the landmark box holds lm_box <= 64 keys; rows beyond it keep stale data and are never used
          mbar_arrive_expect_tx(fb, (uint32_t)lm_box * 256u);
          tma_load_5d(k_slot(s), &tm_klm, fb, 0, kBlk - 1, i * 64, h, b);
          tma_load_5d(k_slot(s) + kHalfTile, &tm_klm, fb, 64, kBlk - 1, i * 64, h, b);
        } else {
          const int n = n_last - (i - n_lm_tiles);
          mbar_arrive_expect_tx(fb, 2 * kTileBytes);
          tma_load_4d(k_slot(s), &tm_k, fb, 0, n * kBlk, h, b);
          tma_load_4d(k_slot(s) + kHalfTile, &tm_k, fb, 64, n * kBlk, h, b);
          tma_load_4d(v_slot(s), &tm_v, fb, 0, n * kBlk, h, b);
          tma_load_4d(v_slot(s) + kHalfTile, &tm_v, fb, 64, n * kBlk, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);    // S = Q K^T
      constexpr uint32_t idesc_o = instr_desc_f16(fmt, 128, 128, 0, 1);   // O += P V   (V is MN-major)
      mbar_wait(smem_u32(&sm->q_full), 0, &g_lmk_status, kErrFwdMma);
      auto issue_s = [&](int j) {
        const int s = j % kFwdStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kFwdStages) & 1, &g_lmk_status, kErrFwdMma);
        if (j >= 2) mbar_wait(smem_u32(&sm->s_free[sb]), ((j / 2) & 1) ^ 1, &g_lmk_status, kErrFwdMma);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          // Q and K: two 64-column sub-tiles; a K-step of 16 elements is 32 bytes inside the swizzle atom
          const uint32_t qa = q_tile + (kk >> 2) * kTileBytes + (kk & 3) * 32;
          const uint32_t ka = k_slot(s) + (kk >> 2) * kHalfTile + (kk & 3) * 32;
          mma_f16_ss(tmem_s0 + sb * 64, smem_desc_sw128(qa, 16, 1024), smem_desc_sw128(ka, 16, 1024), idesc_s,
                     kk > 0);
        }
        mma_commit(smem_u32(&sm->s_full[sb]));
      };
      issue_s(0);
      bool o_started = false;
      for (int i = 0; i < total; ++i) {
        if (i + 1 < total) issue_s(i + 1);
        const int s = i % kFwdStages;
        mbar_wait(smem_u32(&sm->p_ready[s]), (i / kFwdStages) & 1, &g_lmk_status, kErrFwdMma);
        tc_fence_after();
        if (i >= n_lm_tiles) {
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk) {
            // P: [128 x 64] K-major tile in the K slot.  V: two [64 keys x 64 features] sub-tiles, MN-major:
            // 8-key groups 1024 B apart (SBO), the second 64-feature half 8192 B further (LBO); 16 keys = 2048 B.
            const uint32_t pa = k_slot(s) + kk * 32;
            const uint32_t va = v_slot(s) + kk * 2048;
            mma_f16_ss(tmem_o, smem_desc_sw128(pa, 16, 1024), smem_desc_sw128(va, kHalfTile, 1024), idesc_o,
                       (o_started || kk > 0) ? 1u : 0u);
          }
          o_started = true;
        }
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->o_full));
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax threads (row = tid)
    const int row = tid;
    const int half = row >> 6;
    const int own = own0 + half;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m2 = -INFINITY;   // maximum of the outer softmax, log2 domain
    float l = 0.f;
    for (int i = 0; i < total; ++i) {
      const int sb = i & 1, s = i % kFwdStages;
      mbar_wait(smem_u32(&sm->s_full[sb]), (i / 2) & 1, &g_lmk_status, kErrFwdSoftmax);
      tc_fence_after();
      uint32_t ra[32], rb[32];
      tmem_ld_32x32b_x32(tmem_s0 + sb * 64 + lane_base, ra);
      tmem_ld_32x32b_x32(tmem_s0 + sb * 64 + 32 + lane_base, rb);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->s_free[sb]));
      float sv[64];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        sv[j] = __uint_as_float(ra[j]) * scale_log2;
        sv[32 + j] = __uint_as_float(rb[j]) * scale_log2;
      }
      if (i < n_lm_tiles) {
        // landmark scores of blocks i*64 .. i*64+63; only blocks before the row's own block count
        const int first = i * 64;
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (first + j < own) m2 = fmaxf(m2, sv[j]);
      } else {
        const int n = n_last - (i - n_lm_tiles);
        uint32_t w[32];
        if (n > own) {
#pragma unroll
          for (int j = 0; j < 32; ++j) w[j] = 0u;
        } else if (n == own) {
          float mx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (j <= vis) mx = fmaxf(mx, sv[j]);
          m2 = fmaxf(m2, mx);
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            sv[j] = (j <= vis) ? ex2(sv[j] - m2) : 0.f;
            sum += sv[j];
          }
          l += sum;
#pragma unroll
          for (int j = 0; j < 32; ++j) w[j] = pack2<kBf16>(sv[2 * j], sv[2 * j + 1]);
        } else {
          const float lm = sv[63];
          float mx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 63; ++j) mx = fmaxf(mx, sv[j]);
          float den = 0.f;
#pragma unroll
          for (int j = 0; j < 63; ++j) {
            sv[j] = ex2(sv[j] - mx);
            den += sv[j];
          }
          const float el = ex2(lm - m2);
          l += el;
          const float wgt = el / den;
          sv[63] = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) w[j] = pack2<kBf16>(sv[2 * j] * wgt, sv[2 * j + 1] * wgt);
        }
        store_row_sw128(k_slot(s), row, w);
        fence_proxy_async_smem();
      }
      mbar_arrive(smem_u32(&sm->p_ready[s]));
    }
    // ------------------------------------------------------------------ epilogue
    mbar_wait(smem_u32(&sm->o_full), 0, &g_lmk_status, kErrFwdEpilogue);
    tc_fence_after();
    const float inv = 1.f / l;
    const int grow = t * kQTile + row;
    uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(o_ptr) + ((int64_t)bh * Lq + grow) * kD);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_o + c * 32 + lane_base, r);
      tmem_ld_wait();
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        uint4 pk;
        pk.x = pack2<kBf16>(__uint_as_float(r[8 * v4 + 0]) * inv, __uint_as_float(r[8 * v4 + 1]) * inv);
        pk.y = pack2<kBf16>(__uint_as_float(r[8 * v4 + 2]) * inv, __uint_as_float(r[8 * v4 + 3]) * inv);
        pk.z = pack2<kBf16>(__uint_as_float(r[8 * v4 + 4]) * inv, __uint_as_float(r[8 * v4 + 5]) * inv);
        pk.w = pack2<kBf16>(__uint_as_float(r[8 * v4 + 6]) * inv, __uint_as_float(r[8 * v4 + 7]) * inv);
        orow[c * 4 + v4] = pk;
      }
    }
    L_ptr[(int64_t)bh * Lq + grow] = l;
    M_ptr[(int64_t)bh * Lq + grow] = m2 * (1.f / kLog2e);
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}


// ---------------------------------------------------------------------------------------------- forward, two tiles
// Same algorithm with TWO adjacent 128-row query tiles per CTA (one CTA per SM): softmax warpgroup 0 owns tile A
// (rows 256u .. 256u+127), warpgroup 1 owns tile B (the next 128 rows).  Both tiles consume the same K/V stream, so
// every K/V block is fetched from L2 once per 256 query rows, and the two softmax pipelines overlap with each
// other and with the MMAs.  Tile A skips the two newest key blocks (they lie after its own blocks).
constexpr int kFwd2Stages = 4;
constexpr int kFwd2Threads = 320;
enum { kErrFwd2Producer = 111, kErrFwd2Mma = 112, kErrFwd2Softmax = 113, kErrFwd2Epilogue = 114 };

struct Fwd2Smem {
  uint64_t q_full;
  uint64_t full[kFwd2Stages];
  uint64_t empty[kFwd2Stages];
  uint64_t s_full[2][2];    // [tile][S buffer]
  uint64_t s_free[2][2];
  uint64_t p_ready[2];
  uint64_t p_free[2];
  uint64_t o_full;
  uint32_t tmem_base;
};

template <bool kBf16>
__global__ void __launch_bounds__(kFwd2Threads, 1)
sm100_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_klm,
                  void* __restrict__ o_ptr, float* __restrict__ L_ptr, float* __restrict__ M_ptr, int H, int Lq, int Lk,
                  int lm_box, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  auto q_tile = [&](int w) { return base + (uint32_t)w * 32768u; };
  auto k_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u; };
  auto v_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u + 16384u; };
  auto p_tile = [&](int w) { return base + 65536u + kFwd2Stages * 32768u + (uint32_t)w * 16384u; };
  Fwd2Smem* sm = reinterpret_cast<Fwd2Smem*>(smem_raw + (base - raw) + 65536u + kFwd2Stages * 32768u + 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_pairs = Lq / (2 * kQTile);
  const int u = n_pairs - 1 - (int)blockIdx.x;          // heaviest pairs first
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int own0_a = prefix_blocks + 4 * u;             // tile A: blocks own0_a, own0_a+1; tile B: +2, +3
  const int n_last = own0_a + 3;                        // newest block of the pair
  const int n_lm_tiles = (n_last + 63) / 64;            // landmarks 0 .. n_last-1
  const int total = n_lm_tiles + n_last + 1;
  // tile A takes part in item i unless it is one of the first two main items
  auto active = [&](int w, int i) { return w == 1 || i < n_lm_tiles || i >= n_lm_tiles + 2; };

  if (tid == 0) {
    mbar_init(smem_u32(&sm->q_full), 1);
    for (int s = 0; s < kFwd2Stages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
    }
    for (int w = 0; w < 2; ++w) {
      for (int s = 0; s < 2; ++s) {
        mbar_init(smem_u32(&sm->s_full[w][s]), 1);
        mbar_init(smem_u32(&sm->s_free[w][s]), 128);
      }
      mbar_init(smem_u32(&sm->p_ready[w]), 128);
      mbar_init(smem_u32(&sm->p_free[w]), 1);
    }
    mbar_init(smem_u32(&sm->o_full), 1);
    mbar_init_fence();
  }
  if (warp == 9) tmem_alloc(smem_u32(&sm->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  auto tmem_s = [&](int w, int sb) { return tmem + (uint32_t)(w * 128 + sb * 64); };
  auto tmem_o = [&](int w) { return tmem + 256u + (uint32_t)w * 128u; };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_klm);
      const uint32_t qb = smem_u32(&sm->q_full);
      mbar_arrive_expect_tx(qb, 4 * kTileBytes);
      for (int w = 0; w < 2; ++w) {
        tma_load_4d(q_tile(w), &tm_q, qb, 0, (2 * u + w) * kQTile, h, b);
        tma_load_4d(q_tile(w) + kTileBytes, &tm_q, qb, 64, (2 * u + w) * kQTile, h, b);
      }
      for (int i = 0; i < total; ++i) {
        const int s = i % kFwd2Stages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kFwd2Stages) & 1) ^ 1, &g_lmk_status, kErrFwd2Producer);
        const uint32_t fb = smem_u32(&sm->full[s]);
        if (i < n_lm_tiles) {
          mbar_arrive_expect_tx(fb, (uint32_t)lm_box * 256u);
          tma_load_5d(k_slot(s), &tm_klm, fb, 0, kBlk - 1, i * 64, h, b);
          tma_load_5d(k_slot(s) + kHalfTile, &tm_klm, fb, 64, kBlk - 1, i * 64, h, b);
        } else {
          const int n = n_last - (i - n_lm_tiles);
          mbar_arrive_expect_tx(fb, 2 * kTileBytes);
          tma_load_4d(k_slot(s), &tm_k, fb, 0, n * kBlk, h, b);
          tma_load_4d(k_slot(s) + kHalfTile, &tm_k, fb, 64, n * kBlk, h, b);
          tma_load_4d(v_slot(s), &tm_v, fb, 0, n * kBlk, h, b);
          tma_load_4d(v_slot(s) + kHalfTile, &tm_v, fb, 64, n * kBlk, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      constexpr uint32_t idesc_o = instr_desc_f16(fmt, 128, 128, 0, 1);
      mbar_wait(smem_u32(&sm->q_full), 0, &g_lmk_status, kErrFwd2Mma);
      int ks[2] = {0, 0};      // S MMAs issued per tile
      int kp[2] = {0, 0};      // items retired per tile
      auto issue_s = [&](int j) {
        const int s = j % kFwd2Stages;
        mbar_wait(smem_u32(&sm->full[s]), (j / kFwd2Stages) & 1, &g_lmk_status, kErrFwd2Mma);
        for (int w = 0; w < 2; ++w) {
          if (!active(w, j)) continue;
          const int k = ks[w]++, sb = k & 1;
          if (k >= 2) mbar_wait(smem_u32(&sm->s_free[w][sb]), ((k / 2) & 1) ^ 1, &g_lmk_status, kErrFwd2Mma);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t qa = q_tile(w) + (kk >> 2) * kTileBytes + (kk & 3) * 32;
            const uint32_t ka = k_slot(s) + (kk >> 2) * kHalfTile + (kk & 3) * 32;
            mma_f16_ss(tmem_s(w, sb), smem_desc_sw128(qa, 16, 1024), smem_desc_sw128(ka, 16, 1024), idesc_s, kk > 0);
          }
          mma_commit(smem_u32(&sm->s_full[w][sb]));
        }
      };
      issue_s(0);
      bool o_started[2] = {false, false};
      for (int i = 0; i < total; ++i) {
        if (i + 1 < total) issue_s(i + 1);
        const int s = i % kFwd2Stages;
        for (int w = 0; w < 2; ++w) {
          if (!active(w, i)) continue;
          const int k = kp[w]++;
          mbar_wait(smem_u32(&sm->p_ready[w]), k & 1, &g_lmk_status, kErrFwd2Mma);
          tc_fence_after();
          if (i >= n_lm_tiles) {
#pragma unroll
            for (int kk = 0; kk < kBlk / 16; ++kk)
              mma_f16_ss(tmem_o(w), smem_desc_sw128(p_tile(w) + kk * 32, 16, 1024),
                         smem_desc_sw128(v_slot(s) + kk * 2048, kHalfTile, 1024), idesc_o,
                         (o_started[w] || kk > 0) ? 1u : 0u);
            o_started[w] = true;
          }
          mma_commit(smem_u32(&sm->p_free[w]));
        }
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->o_full));
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int w = warp >> 2;                       // 0: tile A, 1: tile B
    const int row = tid & 127;
    const int half = row >> 6;
    const int own = own0_a + 2 * w + half;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    float m2 = -INFINITY, l = 0.f;
    int k = 0;
    for (int i = 0; i < total; ++i) {
      if (!active(w, i)) continue;
      const int sb = k & 1;
      mbar_wait(smem_u32(&sm->s_full[w][sb]), (k / 2) & 1, &g_lmk_status, kErrFwd2Softmax);
      tc_fence_after();
      float sv[64];
      {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(tmem_s(w, sb) + lane_base, ra);
        tmem_ld_32x32b_x32(tmem_s(w, sb) + 32 + lane_base, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = __uint_as_float(ra[j]);
          sv[32 + j] = __uint_as_float(rb[j]);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->s_free[w][sb]));
      uint32_t wgt[32];
      bool write_p = false;
      if (i < n_lm_tiles) {
        const int first = i * 64;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (first + j < own) mx = fmaxf(mx, sv[j]);
        m2 = fmaxf(m2, mx * scale_log2);
      } else {
        const int n = n_last - (i - n_lm_tiles);
        write_p = true;
        if (n > own) {
#pragma unroll
          for (int j = 0; j < 32; ++j) wgt[j] = 0u;
        } else if (n == own) {
          float mx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (j <= vis) mx = fmaxf(mx, sv[j]);
          m2 = fmaxf(m2, mx * scale_log2);
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            sv[j] = (j <= vis) ? ex2(fmaf(sv[j], scale_log2, -m2)) : 0.f;
            sum += sv[j];
          }
          l += sum;
#pragma unroll
          for (int j = 0; j < 32; ++j) wgt[j] = pack2<kBf16>(sv[2 * j], sv[2 * j + 1]);
        } else {
          float mx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 63; ++j) mx = fmaxf(mx, sv[j]);
          const float nmx = -mx * scale_log2;
          const float el = ex2(fmaf(sv[63], scale_log2, -m2));
          float den = 0.f;
#pragma unroll
          for (int j = 0; j < 63; ++j) {
            sv[j] = ex2(fmaf(sv[j], scale_log2, nmx));
            den += sv[j];
          }
          l += el;
          const float wg = __fdividef(el, den);
          sv[63] = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) wgt[j] = pack2<kBf16>(sv[2 * j] * wg, sv[2 * j + 1] * wg);
        }
      }
      if (k > 0) mbar_wait(smem_u32(&sm->p_free[w]), (k - 1) & 1, &g_lmk_status, kErrFwd2Softmax);
      if (write_p) {
        store_row_sw128(p_tile(w), row, wgt);
        fence_proxy_async_smem();
      }
      mbar_arrive(smem_u32(&sm->p_ready[w]));
      ++k;
    }
    // ------------------------------------------------------------------ epilogue
    mbar_wait(smem_u32(&sm->o_full), 0, &g_lmk_status, kErrFwd2Epilogue);
    tc_fence_after();
    const float inv = 1.f / l;
    const int grow = (2 * u + w) * kQTile + row;
    uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(o_ptr) + ((int64_t)bh * Lq + grow) * kD);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_o(w) + c * 32 + lane_base, r);
      tmem_ld_wait();
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        uint4 pk;
        pk.x = pack2<kBf16>(__uint_as_float(r[8 * v4 + 0]) * inv, __uint_as_float(r[8 * v4 + 1]) * inv);
        pk.y = pack2<kBf16>(__uint_as_float(r[8 * v4 + 2]) * inv, __uint_as_float(r[8 * v4 + 3]) * inv);
        pk.z = pack2<kBf16>(__uint_as_float(r[8 * v4 + 4]) * inv, __uint_as_float(r[8 * v4 + 5]) * inv);
        pk.w = pack2<kBf16>(__uint_as_float(r[8 * v4 + 6]) * inv, __uint_as_float(r[8 * v4 + 7]) * inv);
        orow[c * 4 + v4] = pk;
      }
    }
    L_ptr[(int64_t)bh * Lq + grow] = l;
    M_ptr[(int64_t)bh * Lq + grow] = m2 * (1.f / kLog2e);
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- backward: delta
template <bool kBf16>
__global__ void __launch_bounds__(256) sm100_delta_kernel(const uint2* __restrict__ o, const uint2* __restrict__ dO,
                                                          float* __restrict__ delta, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint2 a = o[row * 32 + lane], b = dO[row * 32 + lane];   // 4 elements per lane, 128 per row
  float acc;
  if (kBf16) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float2 a0 = __bfloat1622float2(pa[0]), a1 = __bfloat1622float2(pa[1]);
    float2 b0 = __bfloat1622float2(pb[0]), b1 = __bfloat1622float2(pb[1]);
    acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  } else {
    const __half2* pa = reinterpret_cast<const __half2*>(&a);
    const __half2* pb = reinterpret_cast<const __half2*>(&b);
    float2 a0 = __half22float2(pa[0]), a1 = __half22float2(pa[1]);
    float2 b0 = __half22float2(pb[0]), b1 = __half22float2(pb[1]);
    acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[row] = acc;
}

// Weights of one (query row, key block) pair from the raw scores S and dP = dO . V^T.
//   kind 0: block after the row's own block -> everything zero
//   kind 1: own block (causal, landmark hidden);  kind 2: earlier block (grouped)
// Outputs: ds[] (always) and p[] (when kNeedP) as fp32 in place of sv[] / dp[].
template <bool kNeedP>
__device__ __forceinline__ void bwd_weights(float (&sv)[64], float (&dp)[64], int kind, int vis, float scale_log2,
                                            float scale, float M2, float Linv, float delta) {
#pragma unroll
  for (int j = 0; j < 64; ++j) sv[j] *= scale_log2;
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < 64; ++j) sv[j] = dp[j] = 0.f;
  } else if (kind == 1) {
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      const float pj = (j <= vis) ? ex2(sv[j] - M2) * Linv : 0.f;
      dp[j] = pj * (dp[j] - delta) * scale;
      sv[j] = pj;
    }
  } else {
    const float lm = sv[63];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 63; ++j) mx = fmaxf(mx, sv[j]);
    float den = 0.f, nd = 0.f;
#pragma unroll
    for (int j = 0; j < 63; ++j) {
      sv[j] = ex2(sv[j] - mx);
      den += sv[j];
      nd = fmaf(sv[j], dp[j], nd);
    }
    const float rden = 1.f / den;
    nd *= rden;
    const float g = ex2(lm - M2) * Linv;
    const float w = g * rden;
#pragma unroll
    for (int j = 0; j < 63; ++j) {
      const float pj = sv[j] * w;
      dp[j] = pj * (dp[j] - nd) * scale;
      sv[j] = pj;
    }
    dp[63] = g * (nd - delta) * scale;
    sv[63] = 0.f;
  }
}

enum { kErrDkvProducer = 201, kErrDkvMma = 202, kErrDkvSoftmax = 203, kErrDkvEpilogue = 204,
       kErrDqProducer = 301, kErrDqMma = 302, kErrDqSoftmax = 303, kErrDqEpilogue = 304 };

// ---------------------------------------------------------------------------------------------- backward: dK, dV
constexpr int kDkvStages = 2;

struct DkvSmem {
  uint64_t kv_full;
  uint64_t full[kDkvStages];
  uint64_t empty[kDkvStages];
  uint64_t sdp_full[2];
  uint64_t sdp_free[2];
  uint64_t pds_ready;
  uint64_t pds_free;
  uint64_t acc_full;
  uint32_t tmem_base;
};

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 1)
sm100_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const float* __restrict__ L_ptr, const float* __restrict__ M_ptr,
                     const float* __restrict__ delta_ptr, void* __restrict__ dk_ptr, void* __restrict__ dv_ptr,
                     int H, int Lq, int Lk, float scale, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t k_tile = base, v_tile = base + 16384u;
  auto q_slot = [&](int s) { return base + 32768u + (uint32_t)s * 65536u; };
  auto do_slot = [&](int s) { return base + 32768u + (uint32_t)s * 65536u + 32768u; };
  const uint32_t p_tile = base + 32768u + kDkvStages * 65536u;
  const uint32_t ds_tile = p_tile + 16384u;
  DkvSmem* sm = reinterpret_cast<DkvSmem*>(smem_raw + (base - raw) + 32768u + kDkvStages * 65536u + 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x;                              // key block; low blocks see the most query tiles
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int n_tiles = Lq / kQTile;
  const int tq0 = n > prefix_blocks ? (n - prefix_blocks) / 2 : 0;
  const int n_items = n_tiles - tq0;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->kv_full), 1);
    for (int s = 0; s < kDkvStages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sm->sdp_full[s]), 1);
      mbar_init(smem_u32(&sm->sdp_free[s]), 128);
    }
    mbar_init(smem_u32(&sm->pds_ready), 128);
    mbar_init(smem_u32(&sm->pds_free), 1);
    mbar_init(smem_u32(&sm->acc_full), 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_u32(&sm->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dv = tmem + 256, tmem_dk = tmem + 320;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_do);
      const uint32_t kvb = smem_u32(&sm->kv_full);
      mbar_arrive_expect_tx(kvb, 2 * kTileBytes);
      tma_load_4d(k_tile, &tm_k, kvb, 0, n * kBlk, h, b);
      tma_load_4d(k_tile + kHalfTile, &tm_k, kvb, 64, n * kBlk, h, b);
      tma_load_4d(v_tile, &tm_v, kvb, 0, n * kBlk, h, b);
      tma_load_4d(v_tile + kHalfTile, &tm_v, kvb, 64, n * kBlk, h, b);
      for (int i = 0; i < n_items; ++i) {
        const int s = i % kDkvStages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kDkvStages) & 1) ^ 1, &g_lmk_status, kErrDkvProducer);
        const uint32_t fb = smem_u32(&sm->full[s]);
        const int r0 = (tq0 + i) * kQTile;
        mbar_arrive_expect_tx(fb, 4 * kTileBytes);
        tma_load_4d(q_slot(s), &tm_q, fb, 0, r0, h, b);
        tma_load_4d(q_slot(s) + kTileBytes, &tm_q, fb, 64, r0, h, b);
        tma_load_4d(do_slot(s), &tm_do, fb, 0, r0, h, b);
        tma_load_4d(do_slot(s) + kTileBytes, &tm_do, fb, 64, r0, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);   // S = Q K^T, dP = dO V^T
      constexpr uint32_t idesc_t = instr_desc_f16(fmt, 128, 64, 1, 1);   // dV^T += dO^T P, dK^T += Q^T dS
      mbar_wait(smem_u32(&sm->kv_full), 0, &g_lmk_status, kErrDkvMma);
      auto issue_sdp = [&](int j) {
        const int s = j % kDkvStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kDkvStages) & 1, &g_lmk_status, kErrDkvMma);
        if (j >= 2) mbar_wait(smem_u32(&sm->sdp_free[sb]), ((j / 2) & 1) ^ 1, &g_lmk_status, kErrDkvMma);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * kTileBytes + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          mma_f16_ss(tmem_s + sb * 64, smem_desc_sw128(q_slot(s) + off_a, 16, 1024),
                     smem_desc_sw128(k_tile + off_b, 16, 1024), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * kTileBytes + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          mma_f16_ss(tmem_dp + sb * 64, smem_desc_sw128(do_slot(s) + off_a, 16, 1024),
                     smem_desc_sw128(v_tile + off_b, 16, 1024), idesc_s, kk > 0);
        }
        mma_commit(smem_u32(&sm->sdp_full[sb]));
      };
      issue_sdp(0);
      for (int i = 0; i < n_items; ++i) {
        if (i + 1 < n_items) issue_sdp(i + 1);
        const int s = i % kDkvStages;
        mbar_wait(smem_u32(&sm->pds_ready), i & 1, &g_lmk_status, kErrDkvMma);
        tc_fence_after();
        // A = dO^T / Q^T: MN-major from the row-major [128 q x 128 d] tile (two 64-feature halves 16 KB apart);
        // B = P / dS: MN-major from the [128 q x 64 k] tile.  A K-step is 16 query rows = 2048 bytes.
#pragma unroll
        for (int kk = 0; kk < kQTile / 16; ++kk)
          mma_f16_ss(tmem_dv, smem_desc_sw128(do_slot(s) + kk * 2048, kTileBytes, 1024),
                     smem_desc_sw128(p_tile + kk * 2048, 16, 1024), idesc_t, (i > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kQTile / 16; ++kk)
          mma_f16_ss(tmem_dk, smem_desc_sw128(q_slot(s) + kk * 2048, kTileBytes, 1024),
                     smem_desc_sw128(ds_tile + kk * 2048, 16, 1024), idesc_t, (i > 0 || kk > 0) ? 1u : 0u);
        mma_commit(smem_u32(&sm->pds_free));
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->acc_full));
    }
    __syncwarp();
  } else {
    const int row = tid;
    const int half = row >> 6;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int i = 0; i < n_items; ++i) {
      const int sb = i & 1;
      const int tq = tq0 + i;
      const int own = prefix_blocks + 2 * tq + half;
      const int64_t grow = (int64_t)bh * Lq + tq * kQTile + row;
      const float M2 = M_ptr[grow] * kLog2e, Linv = 1.f / L_ptr[grow], delta = delta_ptr[grow];
      mbar_wait(smem_u32(&sm->sdp_full[sb]), (i / 2) & 1, &g_lmk_status, kErrDkvSoftmax);
      tc_fence_after();
      float sv[64], dp[64];
      {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(tmem_s + sb * 64 + lane_base, ra);
        tmem_ld_32x32b_x32(tmem_s + sb * 64 + 32 + lane_base, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = __uint_as_float(ra[j]);
          sv[32 + j] = __uint_as_float(rb[j]);
        }
        tmem_ld_32x32b_x32(tmem_dp + sb * 64 + lane_base, ra);
        tmem_ld_32x32b_x32(tmem_dp + sb * 64 + 32 + lane_base, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          dp[j] = __uint_as_float(ra[j]);
          dp[32 + j] = __uint_as_float(rb[j]);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->sdp_free[sb]));
      const int kind = n > own ? 0 : (n == own ? 1 : 2);
      bwd_weights<true>(sv, dp, kind, vis, scale_log2, scale, M2, Linv, delta);
      uint32_t wp[32], wd[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        wp[j] = pack2<kBf16>(sv[2 * j], sv[2 * j + 1]);
        wd[j] = pack2<kBf16>(dp[2 * j], dp[2 * j + 1]);
      }
      if (i > 0) mbar_wait(smem_u32(&sm->pds_free), (i - 1) & 1, &g_lmk_status, kErrDkvSoftmax);
      store_row_sw128(p_tile, row, wp);
      store_row_sw128(ds_tile, row, wd);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sm->pds_ready));
    }
    // epilogue: thread = feature d, TMEM column = key j  ->  dV[key][d], dK[key][d]
    mbar_wait(smem_u32(&sm->acc_full), 0, &g_lmk_status, kErrDkvEpilogue);
    tc_fence_after();
    uint16_t* dvp = reinterpret_cast<uint16_t*>(dv_ptr) + ((int64_t)bh * Lk + (int64_t)n * kBlk) * kD + row;
    uint16_t* dkp = reinterpret_cast<uint16_t*>(dk_ptr) + ((int64_t)bh * Lk + (int64_t)n * kBlk) * kD + row;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_dv + c * 32 + lane_base, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        dvp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(r[j]), 0.f) & 0xffffu);
      tmem_ld_32x32b_x32(tmem_dk + c * 32 + lane_base, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        dkp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(r[j]), 0.f) & 0xffffu);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- backward: dQ
constexpr int kDqStages = 3;

struct DqSmem {
  uint64_t qdo_full;
  uint64_t full[kDqStages];
  uint64_t empty[kDqStages];
  uint64_t ds_ready[kDqStages];
  uint64_t sdp_full[2];
  uint64_t sdp_free[2];
  uint64_t acc_full;
  uint32_t tmem_base;
};

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 1)
sm100_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const float* __restrict__ L_ptr, const float* __restrict__ M_ptr,
                    const float* __restrict__ delta_ptr, void* __restrict__ dq_ptr, int H, int Lq, int Lk,
                    float scale, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t q_tile = base, do_tile = base + 32768u;
  auto k_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u; };
  auto v_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u + 16384u; };   // V block, later dS
  DqSmem* sm = reinterpret_cast<DqSmem*>(smem_raw + (base - raw) + 65536u + kDqStages * 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQTile;
  const int t = n_tiles - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int own0 = prefix_blocks + 2 * t;
  const int n_last = own0 + 1;
  const int total = n_last + 1;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->qdo_full), 1);
    for (int s = 0; s < kDqStages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
      mbar_init(smem_u32(&sm->ds_ready[s]), 128);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&sm->sdp_full[s]), 1);
      mbar_init(smem_u32(&sm->sdp_free[s]), 128);
    }
    mbar_init(smem_u32(&sm->acc_full), 1);
    mbar_init_fence();
  }
  if (warp == 5) tmem_alloc(smem_u32(&sm->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dq = tmem + 256;

  if (warp == 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_do);
      const uint32_t qb = smem_u32(&sm->qdo_full);
      mbar_arrive_expect_tx(qb, 4 * kTileBytes);
      tma_load_4d(q_tile, &tm_q, qb, 0, t * kQTile, h, b);
      tma_load_4d(q_tile + kTileBytes, &tm_q, qb, 64, t * kQTile, h, b);
      tma_load_4d(do_tile, &tm_do, qb, 0, t * kQTile, h, b);
      tma_load_4d(do_tile + kTileBytes, &tm_do, qb, 64, t * kQTile, h, b);
      for (int i = 0; i < total; ++i) {
        const int s = i % kDqStages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kDqStages) & 1) ^ 1, &g_lmk_status, kErrDqProducer);
        const uint32_t fb = smem_u32(&sm->full[s]);
        const int n = n_last - i;
        mbar_arrive_expect_tx(fb, 2 * kTileBytes);
        tma_load_4d(k_slot(s), &tm_k, fb, 0, n * kBlk, h, b);
        tma_load_4d(k_slot(s) + kHalfTile, &tm_k, fb, 64, n * kBlk, h, b);
        tma_load_4d(v_slot(s), &tm_v, fb, 0, n * kBlk, h, b);
        tma_load_4d(v_slot(s) + kHalfTile, &tm_v, fb, 64, n * kBlk, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      constexpr uint32_t idesc_q = instr_desc_f16(fmt, 128, 128, 0, 1);   // dQ += dS K  (K is MN-major)
      mbar_wait(smem_u32(&sm->qdo_full), 0, &g_lmk_status, kErrDqMma);
      auto issue_sdp = [&](int j) {
        const int s = j % kDqStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kDqStages) & 1, &g_lmk_status, kErrDqMma);
        if (j >= 2) mbar_wait(smem_u32(&sm->sdp_free[sb]), ((j / 2) & 1) ^ 1, &g_lmk_status, kErrDqMma);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * kTileBytes + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          mma_f16_ss(tmem_s + sb * 64, smem_desc_sw128(q_tile + off_a, 16, 1024),
                     smem_desc_sw128(k_slot(s) + off_b, 16, 1024), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off_a = (kk >> 2) * kTileBytes + (kk & 3) * 32;
          const uint32_t off_b = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          mma_f16_ss(tmem_dp + sb * 64, smem_desc_sw128(do_tile + off_a, 16, 1024),
                     smem_desc_sw128(v_slot(s) + off_b, 16, 1024), idesc_s, kk > 0);
        }
        mma_commit(smem_u32(&sm->sdp_full[sb]));
      };
      issue_sdp(0);
      for (int i = 0; i < total; ++i) {
        if (i + 1 < total) issue_sdp(i + 1);
        const int s = i % kDqStages;
        mbar_wait(smem_u32(&sm->ds_ready[s]), (i / kDqStages) & 1, &g_lmk_status, kErrDqMma);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kBlk / 16; ++kk)
          mma_f16_ss(tmem_dq, smem_desc_sw128(v_slot(s) + kk * 32, 16, 1024),
                     smem_desc_sw128(k_slot(s) + kk * 2048, kHalfTile, 1024), idesc_q, (i > 0 || kk > 0) ? 1u : 0u);
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->acc_full));
    }
    __syncwarp();
  } else {
    const int row = tid;
    const int half = row >> 6;
    const int own = own0 + half;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int64_t grow = (int64_t)bh * Lq + t * kQTile + row;
    const float M2 = M_ptr[grow] * kLog2e, Linv = 1.f / L_ptr[grow], delta = delta_ptr[grow];
    for (int i = 0; i < total; ++i) {
      const int sb = i & 1, s = i % kDqStages;
      const int n = n_last - i;
      mbar_wait(smem_u32(&sm->sdp_full[sb]), (i / 2) & 1, &g_lmk_status, kErrDqSoftmax);
      tc_fence_after();
      float sv[64], dp[64];
      {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(tmem_s + sb * 64 + lane_base, ra);
        tmem_ld_32x32b_x32(tmem_s + sb * 64 + 32 + lane_base, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = __uint_as_float(ra[j]);
          sv[32 + j] = __uint_as_float(rb[j]);
        }
        tmem_ld_32x32b_x32(tmem_dp + sb * 64 + lane_base, ra);
        tmem_ld_32x32b_x32(tmem_dp + sb * 64 + 32 + lane_base, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          dp[j] = __uint_as_float(ra[j]);
          dp[32 + j] = __uint_as_float(rb[j]);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->sdp_free[sb]));
      const int kind = n > own ? 0 : (n == own ? 1 : 2);
      bwd_weights<false>(sv, dp, kind, vis, scale_log2, scale, M2, Linv, delta);
      uint32_t wd[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) wd[j] = pack2<kBf16>(dp[2 * j], dp[2 * j + 1]);
      store_row_sw128(v_slot(s), row, wd);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sm->ds_ready[s]));
    }
    mbar_wait(smem_u32(&sm->acc_full), 0, &g_lmk_status, kErrDqEpilogue);
    tc_fence_after();
    uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq_ptr) + grow * kD);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_dq + c * 32 + lane_base, r);
      tmem_ld_wait();
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        uint4 pk;
        pk.x = pack2<kBf16>(__uint_as_float(r[8 * v4 + 0]), __uint_as_float(r[8 * v4 + 1]));
        pk.y = pack2<kBf16>(__uint_as_float(r[8 * v4 + 2]), __uint_as_float(r[8 * v4 + 3]));
        pk.z = pack2<kBf16>(__uint_as_float(r[8 * v4 + 4]), __uint_as_float(r[8 * v4 + 5]));
        pk.w = pack2<kBf16>(__uint_as_float(r[8 * v4 + 6]), __uint_as_float(r[8 * v4 + 7]));
        orow[c * 4 + v4] = pk;
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Driver-API calls need the device's primary context current on the calling thread; autograd worker threads
// arrive here before any runtime call has bound it.  cudaSetDevice binds it without synchronising the device.
inline void bind_context() {
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaSetDevice(dev);
}

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [B, H, L, 128] tensor with element strides {b, h, row}; box = 64 features x `box_rows` rows, 128-byte swizzle
int make_map_4d(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3], int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[0] * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, dtype == LMK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with %d", (int)r);
  return LMK_OK;
}

// landmark keys: k viewed as [B, H, L/64, 64, 128]; box = 64 features x 1 row-in-block x 64 blocks
int make_map_landmarks(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3],
                       int lm_box) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[5] = {(cuuint64_t)kD, (cuuint64_t)kBlk, (cuuint64_t)(L / kBlk), (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[4] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[2] * 2 * kBlk, (cuuint64_t)st[1] * 2,
                           (cuuint64_t)st[0] * 2};
  cuuint32_t box[5] = {64, 1, (cuuint32_t)lm_box, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, dtype == LMK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled (landmarks) failed with %d", (int)r);
  return LMK_OK;
}

bool tma_ok(const void* p, const int64_t st[3]) {
  return ((uintptr_t)p % 16 == 0) && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0 && st[2] >= kD;
}

}  // namespace

bool attn_sm100_supported(int B, int H, int Lq, int Lk, int D, int block, int dtype) {
  return (dtype == LMK_BF16 || dtype == LMK_F16) && D == kD && block == kBlk && Lq >= kQTile && Lq % kQTile == 0 &&
         Lk % kBlk == 0 && Lk >= Lq && B >= 1 && H >= 1;
}

int attn_sm100_fwd(const AttnParams& p, int dtype, cudaStream_t st) {
  if (!tma_ok(p.q, p.qs) || !tma_ok(p.k, p.ks) || !tma_ok(p.v, p.vs))
    return fail(LMK_ERR_UNSUPPORTED, "tcgen05 path needs 16-byte aligned q/k/v with strides that are multiples of 8");
  bind_context();
  CUtensorMap tq, tk, tv, tl;
  int rc;
  if ((rc = make_map_4d(&tq, p.q, dtype, p.B, p.H, p.Lq, p.qs, kQTile)) != LMK_OK) return rc;
  if ((rc = make_map_4d(&tk, p.k, dtype, p.B, p.H, p.Lk, p.ks, kBlk)) != LMK_OK) return rc;
  if ((rc = make_map_4d(&tv, p.v, dtype, p.B, p.H, p.Lk, p.vs, kBlk)) != LMK_OK) return rc;
  const int lm_box = (p.Lk / kBlk) < 64 ? (p.Lk / kBlk) : 64;
  if ((rc = make_map_landmarks(&tl, p.k, dtype, p.B, p.H, p.Lk, p.ks, lm_box)) != LMK_OK) return rc;
  const float scale_log2 = p.scale * kLog2e;
  if (p.Lq % (2 * kQTile) == 0) {
    const size_t smem = 1024 + 65536 + kFwd2Stages * 32768 + 32768 + sizeof(Fwd2Smem);
    dim3 grid(p.Lq / (2 * kQTile), p.B * p.H);
    if (dtype == LMK_BF16) {
      LMK_CUDA(cudaFuncSetAttribute(sm100_fwd2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      sm100_fwd2_kernel<true><<<grid, kFwd2Threads, smem, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                lm_box, scale_log2);
    } else {
      LMK_CUDA(cudaFuncSetAttribute(sm100_fwd2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      sm100_fwd2_kernel<false><<<grid, kFwd2Threads, smem, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                 lm_box, scale_log2);
    }
  } else {
    const size_t smem = 1024 + 32768 + kFwdStages * 32768 + sizeof(FwdSmem);
    dim3 grid(p.Lq / kQTile, p.B * p.H);
    if (dtype == LMK_BF16) {
      LMK_CUDA(cudaFuncSetAttribute(sm100_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      sm100_fwd_kernel<true><<<grid, kFwdThreads, smem, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk, lm_box,
                                                              scale_log2);
    } else {
      LMK_CUDA(cudaFuncSetAttribute(sm100_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      sm100_fwd_kernel<false><<<grid, kFwdThreads, smem, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk, lm_box,
                                                               scale_log2);
    }
  }
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

int attn_sm100_bwd(const AttnParams& p, int dtype, cudaStream_t st) {
  if (!tma_ok(p.q, p.qs) || !tma_ok(p.k, p.ks) || !tma_ok(p.v, p.vs) || (uintptr_t)p.dO % 16 != 0)
    return fail(LMK_ERR_UNSUPPORTED, "tcgen05 path needs 16-byte aligned tensors with strides that are multiples of 8");
  if (p.Lk % kBlk != 0 || p.Lq % kQTile != 0)
    return fail(LMK_ERR_INVALID, "Backward supported only for full blocks");
  bind_context();
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  const int64_t dense[3] = {(int64_t)p.H * p.Lq * kD, (int64_t)p.Lq * kD, (int64_t)kD};
  if ((rc = make_map_4d(&tq, p.q, dtype, p.B, p.H, p.Lq, p.qs, kQTile)) != LMK_OK) return rc;
  if ((rc = make_map_4d(&tk, p.k, dtype, p.B, p.H, p.Lk, p.ks, kBlk)) != LMK_OK) return rc;
  if ((rc = make_map_4d(&tv, p.v, dtype, p.B, p.H, p.Lk, p.vs, kBlk)) != LMK_OK) return rc;
  if ((rc = make_map_4d(&tdo, p.dO, dtype, p.B, p.H, p.Lq, dense, kQTile)) != LMK_OK) return rc;
  float* delta = reinterpret_cast<float*>(p.workspace);
  const int64_t rows = (int64_t)p.B * p.H * p.Lq;
  const float scale_log2 = p.scale * kLog2e;
  const size_t smem_dkv = 1024 + 32768 + kDkvStages * 65536 + 32768 + sizeof(DkvSmem);
  const size_t smem_dq = 1024 + 65536 + kDqStages * 32768 + sizeof(DqSmem);
  dim3 grid_dkv(p.Lk / kBlk, p.B * p.H), grid_dq(p.Lq / kQTile, p.B * p.H);
#define LMK_BWD_LAUNCH(BF)                                                                                          \
  do {                                                                                                              \
    sm100_delta_kernel<BF><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(                                             \
        reinterpret_cast<const uint2*>(p.o), reinterpret_cast<const uint2*>(p.dO), delta, rows);                    \
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dkv_kernel<BF>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                  (int)smem_dkv));                                                                  \
    sm100_bwd_dkv_kernel<BF><<<grid_dkv, kFwdThreads, smem_dkv, st>>>(tq, tk, tv, tdo, p.L, p.M, delta, p.dk, p.dv, \
                                                                     p.H, p.Lq, p.Lk, p.scale, scale_log2);         \
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dq_kernel<BF>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                  (int)smem_dq));                                                                   \
    sm100_bwd_dq_kernel<BF><<<grid_dq, kFwdThreads, smem_dq, st>>>(tq, tk, tv, tdo, p.L, p.M, delta, p.dq, p.H,     \
                                                                   p.Lq, p.Lk, p.scale, scale_log2);                \
  } while (0)
  if (dtype == LMK_BF16) LMK_BWD_LAUNCH(true);
  else LMK_BWD_LAUNCH(false);
#undef LMK_BWD_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

size_t attn_sm100_bwd_workspace(int B, int H, int Lq, int, int) { return sizeof(float) * (size_t)B * H * Lq; }

int device_status(int* out, int clear) {
  int v = 0;
  LMK_CUDA(cudaDeviceSynchronize());
  LMK_CUDA(cudaMemcpyFromSymbol(&v, g_lmk_status, sizeof(int)));
  if (clear && v != 0) {
    int z = 0;
    LMK_CUDA(cudaMemcpyToSymbol(g_lmk_status, &z, sizeof(int)));
  }
  if (out) *out = v;
  return LMK_OK;
}

}  // namespace lmk
