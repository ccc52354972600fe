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
//      write them as bf16 into shared memory (128-byte swizzled, K-major), and O += P . V_n runs with V as an
//      MN-major operand straight from its row-major TMA tile.
//   3. Epilogue: O / l -> global, plus the statistics L = l, M = m the backward pass needs.
// When Lq is a multiple of 256 the paired kernel (sm100_fwd2_kernel) runs instead: two query tiles per CTA share every
// K/V tile, each with its own softmax warpgroup; P goes back into the TMEM columns its S came from and P . V takes it
// from there as the A operand (no shared-memory round trip); the exponentials are packed fp32 pairs, a quarter of them
// evaluated on the FMA pipe.
// Reference semantics: llama/ltriton/flash_landmark_attention.py:6-122.
//
// Backward is recompute-based and atomic-free (bit-reproducible), in two launches:
//   a. dQ (sm100_bwd_dq_kernel): persistent; a unit is (128 query rows, batch*head).  Its prologue computes
//      delta = rowsum(O * dO) from the O and dO tiles (:125-149, without the 1/L pre-scaling) and stores it for (b).
//      Then, per key block: S = Q K^T, dP = dO V^T -> dS (written over the V tile, which dP no longer needs) ->
//      dQ += dS K with K as an MN-major operand.  Two softmax warpgroups take alternate blocks.
//   b. dK/dV (sm100_bwd_dkv_kernel): persistent; a unit is a pair of adjacent key blocks of one head, held in shared
//      memory while the query tiles that see them stream through.  Per tile: S, dP of both blocks into TMEM (N = 128);
//      the softmax threads rebuild P and dS (bf16, [128 q x 64 k] swizzled tiles); dV^T += dO^T P and dK^T += Q^T dS accumulate
//      TRANSPOSED ([128 features x 64 keys], M = 128) so that every MMA keeps the full 128-lane shape; dO, Q, P and dS
//      are consumed as MN-major operands from their row-major tiles.
//   Per tile pair: earlier block  dS_j = g s_j (dP_j - nD) scale,  dS_landmark = g (nD - delta) scale,  P_j = g s_j,
//   with s = softmax inside the block, g = exp(l_n - M) / L, nD = sum_j s_j dP_j;  own block: p = exp(S - M) / L,
//   dS = p (dP - delta) scale.                                                                      (:152-305)
#include <atomic>
#include <mutex>
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

// Row reductions with four independent chains: one softmax thread has little other work in flight, so a single
// 63-deep dependent chain of max / add would expose the ALU latency on every step.
template <int N>
__device__ __forceinline__ float row_max(const float (&v)[64]) {
  float a = -INFINITY, b = -INFINITY, c = -INFINITY, d = -INFINITY;
#pragma unroll
  for (int j = 0; j + 3 < N; j += 4) {
    a = fmaxf(a, v[j]);
    b = fmaxf(b, v[j + 1]);
    c = fmaxf(c, v[j + 2]);
    d = fmaxf(d, v[j + 3]);
  }
#pragma unroll
  for (int j = N & ~3; j < N; ++j) a = fmaxf(a, v[j]);
  return fmaxf(fmaxf(a, b), fmaxf(c, d));
}
__device__ __forceinline__ float row_max_upto(const float (&v)[64], int last) {
  float a = -INFINITY, b = -INFINITY, c = -INFINITY, d = -INFINITY;
#pragma unroll
  for (int j = 0; j < 64; j += 4) {
    a = fmaxf(a, j <= last ? v[j] : -INFINITY);
    b = fmaxf(b, j + 1 <= last ? v[j + 1] : -INFINITY);
    c = fmaxf(c, j + 2 <= last ? v[j + 2] : -INFINITY);
    d = fmaxf(d, j + 3 <= last ? v[j + 3] : -INFINITY);
  }
  return fmaxf(fmaxf(a, b), fmaxf(c, d));
}
template <int N>
__device__ __forceinline__ float row_sum(const float (&v)[64]) {
  float a = 0.f, b = 0.f, c = 0.f, d = 0.f;
#pragma unroll
  for (int j = 0; j + 3 < N; j += 4) {
    a += v[j];
    b += v[j + 1];
    c += v[j + 2];
    d += v[j + 3];
  }
#pragma unroll
  for (int j = N & ~3; j < N; ++j) a += v[j];
  return (a + b) + (c + d);
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
  // grid = (batch*head, tile): consecutive CTAs are different heads of the same tile, heaviest tiles first, so the
  // hardware's in-order block dispatch is a longest-job-first schedule over the whole launch
  const int t = n_tiles - 1 - (int)blockIdx.y;
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
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
      // Q and K: two 64-column sub-tiles; a K-step of 16 elements is 32 bytes inside the swizzle atom
      const uint64_t dq = smem_desc_sw128(q_tile, 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(k_slot(0), 16, 1024);
      const uint64_t dv0 = smem_desc_sw128(v_slot(0), kHalfTile, 1024);
      auto issue_s = [&](int j) {
        const int s = j % kFwdStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kFwdStages) & 1, &g_lmk_status, kErrFwdMma);
        if (j >= 2) mbar_wait(smem_u32(&sm->s_free[sb]), ((j / 2) & 1) ^ 1, &g_lmk_status, kErrFwdMma);
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (uint32_t)s * 32768u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_s0 + sb * 64, desc_advance(dq, kmajor_step(kk, kTileBytes)),
                     desc_advance(dk, kmajor_step(kk, kHalfTile)), idesc_s, kk > 0);
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
          // P: [128 x 64] K-major tile in the K slot.  V: two [64 keys x 64 features] sub-tiles, MN-major:
          // 8-key groups 1024 B apart (SBO), the second 64-feature half 8192 B further (LBO); 16 keys = 2048 B.
          const uint64_t dp = desc_advance(dk0, (uint32_t)s * 32768u);
          const uint64_t dv = desc_advance(dv0, (uint32_t)s * 32768u);
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk)
            mma_f16_ss(tmem_o, desc_advance(dp, kk * 32), desc_advance(dv, kk * 2048), idesc_o,
                       (o_started || kk > 0) ? 1u : 0u);
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
constexpr int kFwd2Stages = 5;
constexpr int kFwd2Threads = 352;
enum { kErrFwd2Producer = 111, kErrFwd2Mma = 112, kErrFwd2Softmax = 113, kErrFwd2Epilogue = 114 };

// one in this many pairs of exponentials uses ex2_poly2 (measured at L = 8192: 2 -> 544 us, 4 -> 523, 8 -> 515, 64 -> 508;
// no difference at L = 2048: the special-function pipe is not what the forward kernel waits for)
constexpr int kFwdPolyEvery = 64;

struct Fwd2Smem {
  uint64_t q_full;
  uint64_t full[kFwd2Stages];
  uint64_t empty[kFwd2Stages];
  uint64_t s_full[2][2];    // [tile][S buffer]
  uint64_t s_free[2][2];
  uint64_t p_ready[2];
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
  Fwd2Smem* sm = reinterpret_cast<Fwd2Smem*>(smem_raw + (base - raw) + 65536u + kFwd2Stages * 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_pairs = Lq / (2 * kQTile);
  const int u = n_pairs - 1 - (int)blockIdx.y;          // heaviest pairs first, across all heads
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
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
        mbar_init(smem_u32(&sm->s_free[w][s]), 1);
      }
      mbar_init(smem_u32(&sm->p_ready[w]), 128);
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
  grid_dep_launch();      // a dependent kernel (the backward pass) may do its set-up while this grid drains

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
    // ------------------------------------------------------------------ MMA issuer 1: S = Q K^T
    // Two issuer threads keep the scalar bookkeeping between tcgen05.mma instructions short, and the S MMAs of the
    // next key block never queue behind a wait for the softmax of the current one.
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      mbar_wait(smem_u32(&sm->q_full), 0, &g_lmk_status, kErrFwd2Mma);
      const uint64_t dq0 = smem_desc_sw128(q_tile(0), 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(k_slot(0), 16, 1024);
      int ks[2] = {0, 0};
      int s = 0;
      uint32_t ph = 0;
      for (int j = 0; j < total; ++j) {
        mbar_wait(smem_u32(&sm->full[s]), ph, &g_lmk_status, kErrFwd2Mma);
        const uint64_t dk = desc_advance(dk0, (uint32_t)s * 32768u);
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          if (!active(w, j)) continue;
          const int k = ks[w]++, sb = k & 1;
          if (k >= 2) mbar_wait(smem_u32(&sm->s_free[w][sb]), ((k >> 1) & 1) ^ 1, &g_lmk_status, kErrFwd2Mma);
          tc_fence_after();
          const uint64_t dq = desc_advance(dq0, (uint32_t)w * 32768u);
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk)
            mma_f16_ss(tmem_s(w, sb), desc_advance(dq, kmajor_step(kk, kTileBytes)),
                       desc_advance(dk, kmajor_step(kk, kHalfTile)), idesc_s, kk > 0);
          mma_commit(smem_u32(&sm->s_full[w][sb]));
        }
        if (++s == kFwd2Stages) { s = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------------------------------ MMA issuer 2: O += P V
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_o = instr_desc_f16(fmt, 128, 128, 0, 1);
      const uint64_t dv0 = smem_desc_sw128(v_slot(0), kHalfTile, 1024);
      int kp[2] = {0, 0};
      bool o_started[2] = {false, false};
      int s = 0;
      for (int i = 0; i < total; ++i) {
        const uint64_t dv = desc_advance(dv0, (uint32_t)s * 32768u);
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          if (!active(w, i)) continue;
          const int k = kp[w]++;
          mbar_wait(smem_u32(&sm->p_ready[w]), k & 1, &g_lmk_status, kErrFwd2Mma);
          tc_fence_after();
          if (i >= n_lm_tiles) {
            // A = P straight from TMEM: the softmax threads wrote it over the first 32 columns of the S buffer it was
            // computed from (8 columns = 16 keys per K-step)
            const uint32_t tp = tmem_s(w, k & 1);
#pragma unroll
            for (int kk = 0; kk < kBlk / 16; ++kk)
              mma_f16_ts(tmem_o(w), tp + kk * 8, desc_advance(dv, kk * 2048), idesc_o,
                         (o_started[w] || kk > 0) ? 1u : 0u);
            o_started[w] = true;
          }
          mma_commit(smem_u32(&sm->s_free[w][k & 1]));      // the S / P buffer may take the next S product
        }
        // the stage is free once both P V products are done; each of them waited for its S product to be read
        mma_commit(smem_u32(&sm->empty[s]));
        if (++s == kFwd2Stages) s = 0;
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
      uint32_t wgt[32];
      bool write_p = false;
      if (i < n_lm_tiles) {
        m2 = fmaxf(m2, row_max_upto(sv, own - 1 - i * 64) * scale_log2);
      } else {
        const int n = n_last - (i - n_lm_tiles);
        write_p = true;
        if (n > own) {
#pragma unroll
          for (int j = 0; j < 32; ++j) wgt[j] = 0u;
        } else if (n == own) {
          m2 = fmaxf(m2, row_max_upto(sv, vis) * scale_log2);
#pragma unroll
          for (int j = 0; j < 64; ++j) sv[j] = (j <= vis) ? ex2(fmaf(sv[j], scale_log2, -m2)) : 0.f;
          l += row_sum<64>(sv);
#pragma unroll
          for (int j = 0; j < 32; ++j) wgt[j] = pack2<kBf16>(sv[2 * j], sv[2 * j + 1]);
        } else {
          const float nmx = -row_max<63>(sv) * scale_log2;
          const float el = ex2(fmaf(sv[63], scale_log2, -m2));
          const uint64_t c2 = pk2(scale_log2, scale_log2), n2 = pk2(nmx, nmx);
          uint64_t sp[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint64_t x = fma2(pk2(sv[2 * j], sv[2 * j + 1]), c2, n2);
            if (j % kFwdPolyEvery == 1) {
              sp[j] = ex2_poly2(x);       // a share of the exponentials runs on the FMA pipe
            } else {
              float a, b;
              upk2(x, a, b);
              sp[j] = pk2(ex2(a), j == 31 ? 0.f : ex2(b));
            }
          }
          uint64_t s0 = sp[0], s1 = sp[1], s2 = sp[2], s3 = sp[3];
#pragma unroll
          for (int j = 4; j < 32; j += 4) {
            s0 = add2(s0, sp[j]);
            s1 = add2(s1, sp[j + 1]);
            s2 = add2(s2, sp[j + 2]);
            s3 = add2(s3, sp[j + 3]);
          }
          float dl, dh;
          upk2(add2(add2(s0, s1), add2(s2, s3)), dl, dh);
          l += el;
          const float wg = __fdividef(el, dl + dh);
          const uint64_t w2 = pk2(wg, wg);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float a, b;
            upk2(mul2(sp[j], w2), a, b);
            wgt[j] = pack2<kBf16>(a, b);
          }
        }
      }
      if (write_p) {
        tmem_st_32x32b_x32(tmem_s(w, sb) + lane_base, wgt);     // P replaces S in place; the P V product reads it there
        tmem_st_wait();
      }
      tc_fence_before();
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

// ---------------------------------------------------------------------------------------------- backward
// One (query row, key block) pair of the backward pass, in packed fp32 pairs and within 168 registers per thread (so
// that two softmax warpgroups fit next to the three single-thread roles).
//   kind 0: block after the row's own block -> zeros;  kind 1: own block (causal, landmark hidden);
//   kind 2: earlier block (grouped).
// Writes the P row (kNeedP) into p_dst and the dS row into ds_dst ([128 x 64] 128B-swizzled tiles), arrives on
// `free_bar` once the TMEM buffer has been read for the last time, and calls wait_dst() before the first store.
// one in this many pairs of exponentials uses ex2_poly2 (measured: 3 % faster than "never" at L = 8192, equal at 2048)
constexpr int kBwdPolyEvery = 4;

struct NoHook {
  __device__ __forceinline__ void operator()() const {}
};

// packed (bf16 or f16) pair -> packed fp32 pair
template <bool kBf16>
__device__ __forceinline__ uint64_t unpack2(uint32_t w) {
  if (kBf16) return pk2u(w << 16, w & 0xffff0000u);
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  return pk2(f.x, f.y);
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2p(uint64_t v) {
  float lo, hi;
  upk2(v, lo, hi);
  return pack2<kBf16>(lo, hi);
}

// M2L = (row max + log(row sum)) * log2(e): exp2(s * c - M2L) is the outer-softmax probability.
// S and dP are each read from TMEM once and held as packed pairs; dP's buffer is released (free_bar) as soon as it is
// in registers, before the reductions, so the next dP product can start early.
template <bool kBf16, bool kNeedP, typename WaitFn, typename AfterSFn = NoHook, typename BeforeDpFn = NoHook,
          typename BetweenFn = NoHook>
__device__ __forceinline__ void bwd_item(uint32_t ts, uint32_t tdp, uint32_t free_bar, int kind, int vis, float c,
                                         float scale, float M2L, float delta, uint32_t p_dst, uint32_t ds_dst, int row,
                                         WaitFn wait_dst, AfterSFn after_s = AfterSFn(),
                                         BeforeDpFn before_dp = BeforeDpFn(),
                                         BetweenFn between_stores = BetweenFn()) {
  uint64_t sp[32];      // the row as packed pairs: S, then P
  uint64_t dp[32];      // dP, then dS
  float nmx = 0.f, lm2 = 0.f;
  {
    uint32_t ra[32], rb[32];
    tmem_ld_32x32b_x32(ts, ra);
    tmem_ld_32x32b_x32(ts + 32, rb);
    tmem_ld_wait();
    if (kind == 2) {
      float sv[64];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        sv[j] = __uint_as_float(ra[j]);
        sv[32 + j] = __uint_as_float(rb[j]);
      }
      nmx = -row_max<63>(sv) * c;
      lm2 = sv[63] * c;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sp[j] = pk2u(ra[2 * j], ra[2 * j + 1]);
      sp[16 + j] = pk2u(rb[2 * j], rb[2 * j + 1]);
    }
  }
  after_s();      // S is in registers: a caller with separate S / dP buffers releases the S buffer here
  float sub = delta, lm_ds = 0.f, pscale = 1.f;
  const uint64_t c2 = pk2(c, c);
  uint64_t s0 = 0ull, s1 = 0ull, s2 = 0ull, s3 = 0ull;
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) sp[j] = 0ull;
  } else if (kind == 1) {
    const uint64_t m2 = pk2(-M2L, -M2L);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float a, b;
      upk2(fma2(sp[j], c2, m2), a, b);
      sp[j] = pk2(2 * j <= vis ? ex2(a) : 0.f, 2 * j + 1 <= vis ? ex2(b) : 0.f);
    }
  } else {
    const uint64_t n2 = pk2(nmx, nmx);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint64_t x = fma2(sp[j], c2, n2);
      if (j % kBwdPolyEvery == 1) {
        sp[j] = ex2_poly2(x);         // a share of the exponentials runs on the FMA pipe
      } else {
        float a, b;
        upk2(x, a, b);
        sp[j] = pk2(ex2(a), j == 31 ? 0.f : ex2(b));
      }
    }
    s0 = sp[0], s1 = sp[1], s2 = sp[2], s3 = sp[3];
#pragma unroll
    for (int j = 4; j < 32; j += 4) {
      s0 = add2(s0, sp[j]);
      s1 = add2(s1, sp[j + 1]);
      s2 = add2(s2, sp[j + 2]);
      s3 = add2(s3, sp[j + 3]);
    }
  }
  before_dp();    // a caller with separate S / dP buffers waits for dP only now, after the exponentials
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) dp[j] = 0ull;
  } else {
    uint32_t ra[32], rb[32];
    tmem_ld_32x32b_x32(tdp, ra);
    tmem_ld_32x32b_x32(tdp + 32, rb);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      dp[j] = pk2u(ra[2 * j], ra[2 * j + 1]);
      dp[16 + j] = pk2u(rb[2 * j], rb[2 * j + 1]);
    }
  }
  tc_fence_before();
  mbar_arrive(free_bar);
  if (kind == 2) {
    uint64_t n0 = 0ull, n1 = 0ull, n2a = 0ull, n3 = 0ull;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      n0 = fma2(sp[j], dp[j], n0);
      n1 = fma2(sp[j + 1], dp[j + 1], n1);
      n2a = fma2(sp[j + 2], dp[j + 2], n2a);
      n3 = fma2(sp[j + 3], dp[j + 3], n3);
    }
    float dl, dh, ql, qh;
    upk2(add2(add2(s0, s1), add2(s2, s3)), dl, dh);
    upk2(add2(add2(n0, n1), add2(n2a, n3)), ql, qh);
    const float rden = __fdividef(1.f, dl + dh);
    const float nd = (ql + qh) * rden;
    const float g = ex2(lm2 - M2L);
    const float w = g * rden;
    if (kNeedP) {
      const uint64_t w2 = pk2(w, w);
#pragma unroll
      for (int j = 0; j < 32; ++j) sp[j] = mul2(sp[j], w2);
    } else {
      pscale = w;       // P itself is not stored: its row factor is folded into the dS coefficients below
    }
    sub = nd;
    lm_ds = g * (nd - delta) * scale;
  }
  // dS = P * (dP - sub) * scale = P * fma(dP, scale, -sub * scale)
  const float sc = scale * pscale;
  const uint64_t sc2 = pk2(sc, sc);
  const float nss = -sub * sc;
  const uint64_t nss2 = pk2(nss, nss);
  uint32_t wd[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float d0, d1;
    upk2(mul2(sp[j], fma2(dp[j], sc2, nss2)), d0, d1);
    if (j == 31 && kind == 2) d1 = lm_ds;
    wd[j] = pack2<kBf16>(d0, d1);
  }
  if (kNeedP) {
    uint32_t wp[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) wp[j] = pack2p<kBf16>(sp[j]);
    wait_dst();
    store_row_sw128(p_dst, row, wp);
    between_stores();   // the P tile and the dS tile are handed over separately
    store_row_sw128(ds_dst, row, wd);
  } else {
    wait_dst();
    store_row_sw128(ds_dst, row, wd);
  }
}

enum { kErrDkvProducer = 201, kErrDkvMma = 202, kErrDkvSoftmax = 203, kErrDkvEpilogue = 204,
       kErrDqProducer = 301, kErrDqMma = 302, kErrDqSoftmax = 303, kErrDqEpilogue = 304 };

// ---------------------------------------------------------------------------------------------- backward: dK, dV
// Thread roles (both backward kernels): warps 0-3 and 4-7 are two softmax warpgroups that take alternate items
// (the backward pass carries no state from one item to the next), warp 8 issues TMA loads, warp 9 issues the
// S / dP MMAs and owns the TMEM allocation, warp 10 issues the accumulating MMAs.  Two issuer threads keep the
// products of the next item from queueing behind a wait for the current one.  (Registers are granted to 4 warps at
// a time, so 9 to 12 warps all leave 168 registers per thread.)
constexpr int kBwdGroups = 2;                       // softmax warpgroups (items are dealt round-robin)
constexpr int kBwdThreads = (kBwdGroups * 4 + 3) * 32;
constexpr int kSdpBufs = 2;                         // S / dP buffers in TMEM of the dQ kernel: 2 x (64 + 64) columns
constexpr int kDkvStages = 2;

struct DkvSmem {
  uint64_t kv_full;
  uint64_t kv_empty;
  uint64_t full[kDkvStages];
  uint64_t empty[kDkvStages];
  uint64_t s_full;          // S of both blocks (one N = 128 product)
  uint64_t s_free;          // both warpgroups hold S in registers
  uint64_t dp_full;
  uint64_t dp_free;         // both warpgroups have read dP for the last time
  uint64_t p_ready;         // the P tile / the dS tile are handed over separately, so that one warpgroup's stores
  uint64_t ds_ready;        // overlap the other one's accumulating MMAs
  uint64_t p_free[2];       // [g]: the dV MMAs of warpgroup g's latest item have read the P tile
  uint64_t ds_free[2];      // [g]: likewise the dK MMAs and the dS tile
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
};

// Persistent; a work unit is a PAIR of adjacent 64-key blocks (a = 2c, b = 2c+1) of one (batch, head).  Both blocks
// stay in shared memory while the unit streams the query tiles that see them, so each 64 KB Q/dO tile is fetched from
// L2 once per 128 keys, and S / dP of the two blocks are single N = 128 products.  Warpgroup 0 rebuilds P and dS for
// block a, warpgroup 1 for block b; they share a single P/dS tile pair (a writer waits until the accumulating MMAs of
// the item written before have read it), which settles them half an item apart.
// CTA c takes units w = round * grid + c with the direction alternating per round (snake), heaviest pairs first.
// Loads, S/dP products and the softmax of the next unit start while the accumulators of the current one are drained.
template <bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1)
sm100_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const float* __restrict__ L_ptr, const float* __restrict__ M_ptr,
                     const float* __restrict__ delta_ptr, void* __restrict__ dk_ptr, void* __restrict__ dv_ptr,
                     int H, int BH, int Lq, int Lk, float scale, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  // K of the pair as one [128 keys x 128 d] K-major operand: 64-feature sub-tile c at c * 16 KB, block g's 64 rows at
  // g * 8 KB inside it; V likewise, 32 KB further
  const uint32_t k_pair = base, v_pair = base + 32768u;
  auto q_slot = [&](int s) { return base + 65536u + (uint32_t)s * 65536u; };
  auto do_slot = [&](int s) { return base + 65536u + (uint32_t)s * 65536u + 32768u; };
  const uint32_t p_tile = base + 65536u + kDkvStages * 65536u;
  const uint32_t ds_tile = p_tile + 16384u;
  DkvSmem* sm = reinterpret_cast<DkvSmem*>(smem_raw + (base - raw) + 65536u + kDkvStages * 65536u + 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int n_tiles = Lq / kQTile;
  const int n_blocks = Lk / kBlk;
  const int n_pairs = (n_blocks + 1) / 2;
  const int n_units = n_pairs * BH;
  auto unit_of = [&](int r) {
    const int c = (r & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    return r * (int)gridDim.x + c;
  };
  auto unit_tq0 = [&](int pair) { return 2 * pair > prefix_blocks ? (2 * pair - prefix_blocks) / 2 : 0; };

  if (tid == 0) {
    mbar_init(smem_u32(&sm->kv_full), 1);
    mbar_init(smem_u32(&sm->kv_empty), 1);
    for (int s = 0; s < kDkvStages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
    }
    mbar_init(smem_u32(&sm->s_full), 1);
    mbar_init(smem_u32(&sm->s_free), 256);
    mbar_init(smem_u32(&sm->dp_full), 1);
    mbar_init(smem_u32(&sm->dp_free), 256);
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&sm->acc_full[g]), 1);
      mbar_init(smem_u32(&sm->acc_empty[g]), 128);
    }
    mbar_init(smem_u32(&sm->p_ready), 128);
    mbar_init(smem_u32(&sm->ds_ready), 128);
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&sm->p_free[g]), 1);
      mbar_init(smem_u32(&sm->ds_free[g]), 1);
    }
    mbar_init_fence();
  }
  if (warp == kBwdGroups * 4 + 1) tmem_alloc(smem_u32(&sm->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  auto tmem_s = [&](int g) { return tmem + (uint32_t)g * 64u; };
  auto tmem_dp = [&](int g) { return tmem + 128u + (uint32_t)g * 64u; };
  auto tmem_dv = [&](int g) { return tmem + 256u + (uint32_t)g * 128u; };
  auto tmem_dk = [&](int g) { return tmem + 320u + (uint32_t)g * 128u; };

  if (warp == kBwdGroups * 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_do);
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int pair = w / BH, bh = w - pair * BH, b = bh / H, h = bh - b * H;
        const int tq0 = unit_tq0(pair), n_items = n_tiles - tq0;
        const uint32_t kvb = smem_u32(&sm->kv_full);
        mbar_wait(smem_u32(&sm->kv_empty), (u & 1) ^ 1, &g_lmk_status, kErrDkvProducer);
        mbar_arrive_expect_tx(kvb, 4 * kTileBytes);
        for (int g = 0; g < 2; ++g) {       // a block past the end of the sequence reads as zeros
          const int r0 = (2 * pair + g) * kBlk;
          tma_load_4d(k_pair + g * kHalfTile, &tm_k, kvb, 0, r0, h, b);
          tma_load_4d(k_pair + kTileBytes + g * kHalfTile, &tm_k, kvb, 64, r0, h, b);
          tma_load_4d(v_pair + g * kHalfTile, &tm_v, kvb, 0, r0, h, b);
          tma_load_4d(v_pair + kTileBytes + g * kHalfTile, &tm_v, kvb, 64, r0, h, b);
        }
        for (int i = 0; i < n_items; ++i, ++it) {
          const int s = it % kDkvStages;
          mbar_wait(smem_u32(&sm->empty[s]), ((it / kDkvStages) & 1) ^ 1, &g_lmk_status, kErrDkvProducer);
          const uint32_t fb = smem_u32(&sm->full[s]);
          const int r0 = (tq0 + i) * kQTile;
          mbar_arrive_expect_tx(fb, 4 * kTileBytes);
          tma_load_4d(q_slot(s), &tm_q, fb, 0, r0, h, b);
          tma_load_4d(q_slot(s) + kTileBytes, &tm_q, fb, 64, r0, h, b);
          tma_load_4d(do_slot(s), &tm_do, fb, 0, r0, h, b);
          tma_load_4d(do_slot(s) + kTileBytes, &tm_do, fb, 64, r0, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == kBwdGroups * 4 + 1) {
    // S = Q K^T and dP = dO V^T for both blocks of the pair at once (N = 128: full-rate MMAs), one query tile at a
    // time.  S has its own full / free barriers: the warpgroups hold S in registers early in an item, so the next S
    // product runs while they are still busy with dP.
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 128, 0, 0);
      const uint64_t dk0 = smem_desc_sw128(k_pair, 16, 1024), dv0 = smem_desc_sw128(v_pair, 16, 1024);
      const uint64_t dq0 = smem_desc_sw128(q_slot(0), 16, 1024), ddo0 = smem_desc_sw128(do_slot(0), 16, 1024);
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int n_items = n_tiles - unit_tq0(w / BH);
        mbar_wait(smem_u32(&sm->kv_full), u & 1, &g_lmk_status, kErrDkvMma);
        for (int i = 0; i < n_items; ++i, ++it) {
          const int s = it % kDkvStages;
          mbar_wait(smem_u32(&sm->full[s]), (it / kDkvStages) & 1, &g_lmk_status, kErrDkvMma);
          const uint64_t dq = desc_advance(dq0, (uint32_t)s * 65536u), ddo = desc_advance(ddo0, (uint32_t)s * 65536u);
          if (it >= 1) mbar_wait(smem_u32(&sm->s_free), (it & 1) ^ 1, &g_lmk_status, kErrDkvMma);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk)
            mma_f16_ss(tmem_s(0), desc_advance(dq, kmajor_step(kk, kTileBytes)),
                       desc_advance(dk0, kmajor_step(kk, kTileBytes)), idesc_s, kk > 0);
          mma_commit(smem_u32(&sm->s_full));
          if (it >= 1) mbar_wait(smem_u32(&sm->dp_free), (it & 1) ^ 1, &g_lmk_status, kErrDkvMma);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk)
            mma_f16_ss(tmem_dp(0), desc_advance(ddo, kmajor_step(kk, kTileBytes)),
                       desc_advance(dv0, kmajor_step(kk, kTileBytes)), idesc_s, kk > 0);
          mma_commit(smem_u32(&sm->dp_full));
        }
        mma_commit(smem_u32(&sm->kv_empty));      // K / V tiles may be replaced once these products are done
      }
    }
    __syncwarp();
  } else if (warp == kBwdGroups * 4 + 2) {
    // dV_g^T += dO^T P and dK_g^T += Q^T dS.  A = dO^T / Q^T: MN-major view of the row-major [128 q x 128 d] tile (second
    // 64-feature half 16 KB further); B = P / dS: MN-major view of the [128 q x 64 k] tile; a K-step is 16 query rows
    // = 2048 bytes.
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_t = instr_desc_f16(fmt, 128, 64, 1, 1);
      const uint64_t dq0t = smem_desc_sw128(q_slot(0), kTileBytes, 1024);
      const uint64_t ddo0t = smem_desc_sw128(do_slot(0), kTileBytes, 1024);
      const uint64_t dpt = smem_desc_sw128(p_tile, 16, 1024), ddst = smem_desc_sw128(ds_tile, 16, 1024);
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int n_items = n_tiles - unit_tq0(w / BH);
        for (int i = 0; i < n_items; ++i, ++it) {
          const int s = it % kDkvStages;
          const uint64_t ddot = desc_advance(ddo0t, (uint32_t)s * 65536u), dqt = desc_advance(dq0t, (uint32_t)s * 65536u);
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            // item j = 2 * it + g of the single P/dS tile pair
            mbar_wait(smem_u32(&sm->p_ready), g, &g_lmk_status, kErrDkvMma);
            if (i == 0) mbar_wait(smem_u32(&sm->acc_empty[g]), (u & 1) ^ 1, &g_lmk_status, kErrDkvMma);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kQTile / 16; ++kk)
              mma_f16_ss(tmem_dv(g), desc_advance(ddot, kk * 2048), desc_advance(dpt, kk * 2048), idesc_t,
                         (i > 0 || kk > 0) ? 1u : 0u);
            mma_commit(smem_u32(&sm->p_free[g]));
            mbar_wait(smem_u32(&sm->ds_ready), g, &g_lmk_status, kErrDkvMma);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kQTile / 16; ++kk)
              mma_f16_ss(tmem_dk(g), desc_advance(dqt, kk * 2048), desc_advance(ddst, kk * 2048), idesc_t,
                         (i > 0 || kk > 0) ? 1u : 0u);
            mma_commit(smem_u32(&sm->ds_free[g]));
          }
          mma_commit(smem_u32(&sm->empty[s]));
        }
        mma_commit(smem_u32(&sm->acc_full[0]));
        mma_commit(smem_u32(&sm->acc_full[1]));
      }
    }
    __syncwarp();
  } else {
    const int g = warp >> 2;                       // warpgroup g owns block g of every pair
    const int row = tid & 127;
    const int half = row >> 6;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int it = 0, u = 0;
    for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
      const int pair = w / BH, bh = w - pair * BH;
      const int n = 2 * pair + g;
      const int tq0 = unit_tq0(pair), n_items = n_tiles - tq0;
      // the row statistics of the next item are fetched one item ahead, so their latency is never exposed
      const int64_t grow0 = (int64_t)bh * Lq + tq0 * kQTile + row;
      if (u == 0) grid_dep_wait();     // delta comes from the dQ kernel, which may still be running (see the launch)
      float nM = M_ptr[grow0], nL = L_ptr[grow0], nDelta = delta_ptr[grow0];
      for (int i = 0; i < n_items; ++i, ++it) {
        const int tq = tq0 + i;
        const int own = prefix_blocks + 2 * tq + half;
        const float M2L = fmaf(nM, kLog2e, __log2f(nL)), delta = nDelta;
        if (i + 1 < n_items) {
          const int64_t grow = (int64_t)bh * Lq + (tq + 1) * kQTile + row;
          nM = M_ptr[grow];
          nL = L_ptr[grow];
          nDelta = delta_ptr[grow];
        }
        mbar_wait(smem_u32(&sm->s_full), it & 1, &g_lmk_status, kErrDkvSoftmax);
        tc_fence_after();
        const int kind = n > own ? 0 : (n == own ? 1 : 2);
        bwd_item<kBf16, true>(tmem_s(g) + lane_base, tmem_dp(g) + lane_base, smem_u32(&sm->dp_free), kind, vis,
                              scale_log2, scale, M2L, delta, p_tile, ds_tile, row, [&]() {
                                // The single P/dS tile pair is written in the order a, b, a, b, ...: before writing,
                                // the accumulating MMAs of the OTHER warpgroup's latest item must have read it.  Each
                                // warpgroup is the only waiter on the other one's barriers and sees every phase.
                                const int prev = 2 * it + g - 1;          // item written just before this one
                                if (prev >= 0)
                                  mbar_wait(smem_u32(&sm->p_free[1 - g]), (prev >> 1) & 1, &g_lmk_status,
                                            kErrDkvSoftmax);
                              },
                              [&]() {
                                tc_fence_before();
                                mbar_arrive(smem_u32(&sm->s_free));
                              },
                              [&]() {
                                mbar_wait(smem_u32(&sm->dp_full), it & 1, &g_lmk_status, kErrDkvSoftmax);
                                tc_fence_after();
                              },
                              [&]() {
                                fence_proxy_async_smem();
                                mbar_arrive(smem_u32(&sm->p_ready));
                                const int prev = 2 * it + g - 1;
                                if (prev >= 0)
                                  mbar_wait(smem_u32(&sm->ds_free[1 - g]), (prev >> 1) & 1, &g_lmk_status,
                                            kErrDkvSoftmax);
                              });
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&sm->ds_ready));
      }
      // epilogue: each warpgroup drains its own block; thread = feature d, TMEM column = key j -> dV[key][d], dK[key][d]
      mbar_wait(smem_u32(&sm->acc_full[g]), u & 1, &g_lmk_status, kErrDkvEpilogue);
      tc_fence_after();
      uint32_t rv[2][32], rk[2][32];
      tmem_ld_32x32b_x32(tmem_dv(g) + lane_base, rv[0]);
      tmem_ld_32x32b_x32(tmem_dv(g) + 32 + lane_base, rv[1]);
      tmem_ld_32x32b_x32(tmem_dk(g) + lane_base, rk[0]);
      tmem_ld_32x32b_x32(tmem_dk(g) + 32 + lane_base, rk[1]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->acc_empty[g]));     // the next unit may start accumulating into this block's columns
      if (n < n_blocks) {
        uint16_t* dvp = reinterpret_cast<uint16_t*>(dv_ptr) + ((int64_t)bh * Lk + (int64_t)n * kBlk) * kD + row;
        uint16_t* dkp = reinterpret_cast<uint16_t*>(dk_ptr) + ((int64_t)bh * Lk + (int64_t)n * kBlk) * kD + row;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            dvp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(rv[c][j]), 0.f) & 0xffffu);
            dkp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(rk[c][j]), 0.f) & 0xffffu);
          }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kBwdGroups * 4 + 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- backward: dQ
constexpr int kDqStages = 4;
// The dQ kernel has a fourth single-thread role: S = Q K^T and dP = dO V^T are issued by two different threads.  With
// the A operand in TMEM an N = 64 product needs only 32 clk of the tensor pipe, but one thread cannot issue such
// instructions faster than one per ~45 clk; two issuers together reach the pipe's rate (measured with an issue-rate
// microbenchmark: 44.7 clk per instruction from one thread, 32 clk per instruction from two).
constexpr int kDqThreads = kBwdThreads + 32;

struct DqSmem {
  uint64_t qdo_full;
  uint64_t ops_ready;       // the unit's Q and dO rows sit in TMEM (written by the softmax warpgroups)
  uint64_t ops_free;        // the S / dP products of the unit have read them
  uint64_t delta_read;      // both softmax warpgroups are done with the Q, dO and O tiles in shared memory
  uint64_t full[kDqStages];
  uint64_t empty[kDqStages];
  uint64_t ds_ready[kDqStages];
  uint64_t sdp_full[kSdpBufs];
  uint64_t sdp_free[kSdpBufs];
  uint64_t acc_full[2];     // per draining warpgroup (the one that took the unit's last item)
  uint64_t acc_empty;
  uint32_t tmem_base;
};

// Persistent: one CTA per SM walks through the units (128 query rows, batch*head), heaviest tiles first, dealt to the
// CTAs in a snake.  The K/V stream, the S/dP products and the softmax of the next unit start while dQ of the current
// unit is drained by one warpgroup (the two warpgroups alternate); only the unit's first accumulating MMA waits for
// the drain.  All barrier phases derive from counters that run across units.
template <bool kBf16>
__global__ void __launch_bounds__(kDqThreads, 1)
sm100_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_o, const float* __restrict__ L_ptr,
                    const float* __restrict__ M_ptr, float* __restrict__ delta_ptr, void* __restrict__ dq_ptr, int H,
                    int BH, int Lq, int Lk, float scale, float scale_log2) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t q_tile = base, do_tile = base + 32768u;
  auto k_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u; };
  auto v_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u + 16384u; };   // V block, later dS
  const uint32_t o_tile = base + 65536u + kDqStages * 32768u;      // forward output tile, only for delta
  DqSmem* sm = reinterpret_cast<DqSmem*>(smem_raw + (base - raw) + 65536u + kDqStages * 32768u + 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQTile;
  const int prefix_blocks = (Lk - Lq) / kBlk;
  const int n_units = n_tiles * BH;
  auto unit_of = [&](int r) {
    const int c = (r & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    return r * (int)gridDim.x + c;
  };
  // unit w -> query tile (heaviest = last tile first) and number of key blocks it sees
  auto unit_tile = [&](int w) { return n_tiles - 1 - w / BH; };
  auto unit_items = [&](int t) { return prefix_blocks + 2 * t + 2; };

  if (tid == 0) {
    mbar_init(smem_u32(&sm->qdo_full), 1);
    mbar_init(smem_u32(&sm->ops_ready), 256);
    mbar_init(smem_u32(&sm->ops_free), 2);          // the S issuer and the dP issuer
    mbar_init(smem_u32(&sm->delta_read), 256);
    for (int s = 0; s < kDqStages; ++s) {
      mbar_init(smem_u32(&sm->full[s]), 1);
      mbar_init(smem_u32(&sm->empty[s]), 1);
      mbar_init(smem_u32(&sm->ds_ready[s]), 128);
    }
    for (int s = 0; s < kSdpBufs; ++s) {
      mbar_init(smem_u32(&sm->sdp_full[s]), 2);     // S product done + dP product done
      mbar_init(smem_u32(&sm->sdp_free[s]), 128);
    }
    mbar_init(smem_u32(&sm->acc_full[0]), 1);
    mbar_init(smem_u32(&sm->acc_full[1]), 1);
    mbar_init(smem_u32(&sm->acc_empty), 128);
    mbar_init_fence();
  }
  if (warp == kBwdGroups * 4 + 1) tmem_alloc(smem_u32(&sm->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  // TMEM: S buffers [0,128), dP buffers [128,256), dQ [256,384), Q rows [384,448), dO rows [448,512).  Q and dO are the
  // A operands of S = Q K^T and dP = dO V^T for every key block of the unit: held in TMEM they are not re-read from
  // shared memory 2 x 32 KB per block (half of the kernel's shared-memory operand traffic), and their shared-memory
  // tiles are free for the next unit's loads as soon as the prologue has copied them.
  const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dq = tmem + 256, tmem_q = tmem + 384, tmem_do = tmem + 448;
  // Everything above (barriers, TMEM) overlapped the tail of the kernel before this one in the stream; any of this
  // kernel's inputs may come from it, so nothing is read from global memory before this point.  The dK/dV kernel that
  // follows may start its CTAs as SMs free up: it only depends on this kernel for `delta`.
  grid_dep_wait();
  grid_dep_launch();

  if (warp == kBwdGroups * 4) {
    if (lane == 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_do);
      prefetch_tensormap(&tm_o);
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int t = unit_tile(w), bh = w % BH, b = bh / H, h = bh - b * H;
        const int total = unit_items(t), n_last = total - 1;
        const uint32_t qb = smem_u32(&sm->qdo_full);
        mbar_wait(smem_u32(&sm->delta_read), (u & 1) ^ 1, &g_lmk_status, kErrDqProducer);
        mbar_arrive_expect_tx(qb, 6 * kTileBytes);
        tma_load_4d(o_tile, &tm_o, qb, 0, t * kQTile, h, b);
        tma_load_4d(o_tile + kTileBytes, &tm_o, qb, 64, t * kQTile, h, b);
        tma_load_4d(q_tile, &tm_q, qb, 0, t * kQTile, h, b);
        tma_load_4d(q_tile + kTileBytes, &tm_q, qb, 64, t * kQTile, h, b);
        tma_load_4d(do_tile, &tm_do, qb, 0, t * kQTile, h, b);
        tma_load_4d(do_tile + kTileBytes, &tm_do, qb, 64, t * kQTile, h, b);
        for (int i = 0; i < total; ++i, ++it) {
          const int s = it % kDqStages;
          mbar_wait(smem_u32(&sm->empty[s]), ((it / kDqStages) & 1) ^ 1, &g_lmk_status, kErrDqProducer);
          const uint32_t fb = smem_u32(&sm->full[s]);
          const int n = n_last - i;
          mbar_arrive_expect_tx(fb, 2 * kTileBytes);
          tma_load_4d(k_slot(s), &tm_k, fb, 0, n * kBlk, h, b);
          tma_load_4d(k_slot(s) + kHalfTile, &tm_k, fb, 64, n * kBlk, h, b);
          tma_load_4d(v_slot(s), &tm_v, fb, 0, n * kBlk, h, b);
          tma_load_4d(v_slot(s) + kHalfTile, &tm_v, fb, 64, n * kBlk, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == kBwdGroups * 4 + 1 || warp == kBwdGroups * 4 + 3) {
    // warp +1 issues S = Q K^T, warp +3 issues dP = dO V^T; both walk through the same items and wait for the same
    // barriers (each is a waiter of its own on full / sdp_free / ops_ready and sees every phase)
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      const bool is_s = warp == kBwdGroups * 4 + 1;
      const uint64_t db0 = smem_desc_sw128(is_s ? k_slot(0) : v_slot(0), 16, 1024);
      const uint32_t t_out = is_s ? tmem_s : tmem_dp, t_a = is_s ? tmem_q : tmem_do;
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int total = unit_items(unit_tile(w));
        mbar_wait(smem_u32(&sm->ops_ready), u & 1, &g_lmk_status, kErrDqMma);
        for (int i = 0; i < total; ++i, ++it) {
          const int s = it % kDqStages, sb = it % kSdpBufs;
          mbar_wait(smem_u32(&sm->full[s]), (it / kDqStages) & 1, &g_lmk_status, kErrDqMma);
          if (it >= kSdpBufs)
            mbar_wait(smem_u32(&sm->sdp_free[sb]), ((it / kSdpBufs) & 1) ^ 1, &g_lmk_status, kErrDqMma);
          tc_fence_after();
          const uint64_t db = desc_advance(db0, (uint32_t)s * 32768u);
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk)      // A from TMEM: 8 columns = 16 features per K-step
            mma_f16_ts(t_out + sb * 64, t_a + kk * 8, desc_advance(db, kmajor_step(kk, kHalfTile)), idesc_s, kk > 0);
          mma_commit(smem_u32(&sm->sdp_full[sb]));
        }
        mma_commit(smem_u32(&sm->ops_free));        // the next unit's Q / dO rows may be written
      }
    }
    __syncwarp();
  } else if (warp == kBwdGroups * 4 + 2) {
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_q = instr_desc_f16(fmt, 128, 128, 0, 1);   // dQ += dS K  (K is MN-major)
      const uint64_t dv0 = smem_desc_sw128(v_slot(0), 16, 1024);
      const uint64_t dk0t = smem_desc_sw128(k_slot(0), kHalfTile, 1024);
      int it = 0, u = 0;
      for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
        const int total = unit_items(unit_tile(w));
        for (int i = 0; i < total; ++i, ++it) {
          const int s = it % kDqStages;
          mbar_wait(smem_u32(&sm->ds_ready[s]), (it / kDqStages) & 1, &g_lmk_status, kErrDqMma);
          if (i == 0) mbar_wait(smem_u32(&sm->acc_empty), (u & 1) ^ 1, &g_lmk_status, kErrDqMma);
          tc_fence_after();
          const uint64_t dds = desc_advance(dv0, (uint32_t)s * 32768u), dkt = desc_advance(dk0t, (uint32_t)s * 32768u);
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk)
            mma_f16_ss(tmem_dq, desc_advance(dds, kk * 32), desc_advance(dkt, kk * 2048), idesc_q,
                       (i > 0 || kk > 0) ? 1u : 0u);
          mma_commit(smem_u32(&sm->empty[s]));
        }
        mma_commit(smem_u32(&sm->acc_full[(it - 1) & 1]));     // drained by the warpgroup that took the last item
      }
    }
    __syncwarp();
  } else {
    const int g = warp >> 2;                       // warpgroup: items with (running item count) % 2 == g
    const int row = tid & 127;
    const int half = row >> 6;
    const int vis = min(row & 63, kBlk - 2);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int it0 = 0, u = 0, drains = 0;
    // dQ of a unit is drained by the warpgroup that took its last item, but only after that warpgroup has done the
    // prologue of the NEXT unit: the last dQ product queues behind the next unit's first S / dP products, so an
    // immediate drain would just wait for it.  (The next unit's first dQ product needs its first dS, far later.)
    int64_t drain_row = -1;
    auto drain = [&]() {
      mbar_wait(smem_u32(&sm->acc_full[g]), drains & 1, &g_lmk_status, kErrDqEpilogue);
      ++drains;
      tc_fence_after();
      uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq_ptr) + drain_row * kD);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_dq + c * 32 + lane_base, r);
        tmem_ld_wait();
        if (c == 3) {
          tc_fence_before();
          mbar_arrive(smem_u32(&sm->acc_empty));     // the next unit may start accumulating
        }
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
      drain_row = -1;
    };
    // the row statistics of the next unit are fetched while the current one runs, so their latency is never exposed
    float nM = 0.f, nL = 1.f;
    {
      const int w0 = unit_of(0);
      if (w0 < n_units) {
        const int64_t g0 = (int64_t)(w0 % BH) * Lq + unit_tile(w0) * kQTile + row;
        nM = M_ptr[g0];
        nL = L_ptr[g0];
      }
    }
    for (int w = unit_of(0); w < n_units; w = unit_of(++u)) {
      const int t = unit_tile(w), bh = w % BH;
      const int own = prefix_blocks + 2 * t + half;
      const int total = unit_items(t), n_last = total - 1;
      const int64_t grow = (int64_t)bh * Lq + t * kQTile + row;
      const float M2L = fmaf(nM, kLog2e, __log2f(nL));
      {
        const int wn = unit_of(u + 1);
        if (wn < n_units) {
          const int64_t gn = (int64_t)(wn % BH) * Lq + unit_tile(wn) * kQTile + row;
          nM = M_ptr[gn];
          nL = L_ptr[gn];
        }
      }
      // delta = rowsum(O * dO), straight from the swizzled tiles (one row per thread, 16-byte chunks); warpgroup 0
      // also publishes it for the dK/dV kernel, which runs after this one
      mbar_wait(smem_u32(&sm->qdo_full), u & 1, &g_lmk_status, kErrDqSoftmax);
      float delta = 0.f;
      uint32_t opw[2][32];      // this thread's row of the operand its warpgroup moves to TMEM (0: Q, 1: dO)
#pragma unroll
      for (int sub = 0; sub < 2; ++sub)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t off = (uint32_t)sub * kTileBytes + (uint32_t)row * 128u + (uint32_t)((c ^ (row & 7)) << 4);
          uint32_t ov[4], gv[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(ov[0]), "=r"(ov[1]), "=r"(ov[2]), "=r"(ov[3]) : "r"(o_tile + off));
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(gv[0]), "=r"(gv[1]), "=r"(gv[2]), "=r"(gv[3]) : "r"(do_tile + off));
          if (g == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) opw[sub][4 * c + e] = gv[e];
          } else {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(opw[sub][4 * c]), "=r"(opw[sub][4 * c + 1]), "=r"(opw[sub][4 * c + 2]),
                           "=r"(opw[sub][4 * c + 3]) : "r"(q_tile + off));
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 fo, fg;
            if (kBf16) {
              fo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov[e]));
              fg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv[e]));
            } else {
              fo = __half22float2(*reinterpret_cast<const __half2*>(&ov[e]));
              fg = __half22float2(*reinterpret_cast<const __half2*>(&gv[e]));
            }
            delta = fmaf(fo.x, fg.x, delta);
            delta = fmaf(fo.y, fg.y, delta);
          }
        }
      mbar_arrive(smem_u32(&sm->delta_read));       // the shared-memory tiles may take the next unit's rows
      // row -> TMEM lane, 32-bit word j (two features) -> column j: the layout of a K-major A operand
      mbar_wait(smem_u32(&sm->ops_free), (u & 1) ^ 1, &g_lmk_status, kErrDqSoftmax);
      tc_fence_after();
      {
        const uint32_t dst = (g == 0 ? tmem_q : tmem_do) + lane_base;
        tmem_st_32x32b_x32(dst, opw[0]);
        tmem_st_32x32b_x32(dst + 32, opw[1]);
        tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sm->ops_ready));
      if (g == 0) delta_ptr[grow] = delta;
      if (drain_row >= 0) drain();
      for (int i = (it0 + g) & 1; i < total; i += kBwdGroups) {
        const int it = it0 + i;
        const int s = it % kDqStages, sb = it % kSdpBufs;
        const int n = n_last - i;
        mbar_wait(smem_u32(&sm->sdp_full[sb]), (it / kSdpBufs) & 1, &g_lmk_status, kErrDqSoftmax);
        tc_fence_after();
        const int kind = n > own ? 0 : (n == own ? 1 : 2);
        // dS replaces the V tile of this stage, which dP = dO V^T has finished reading
        bwd_item<kBf16, false>(tmem_s + sb * 64 + lane_base, tmem_dp + sb * 64 + lane_base,
                               smem_u32(&sm->sdp_free[sb]), kind, vis, scale_log2, scale, M2L, delta, 0u,
                               v_slot(s), row, []() {});
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&sm->ds_ready[s]));
      }
      it0 += total;
      if (g == ((it0 - 1) & 1)) drain_row = grow;
    }
    if (drain_row >= 0) drain();
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kBwdGroups * 4 + 1) {
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

// Tensor maps are cached: a training loop calls with the same few (pointer, shape, strides) again and again, and
// encoding five or six maps per call is a noticeable part of the host time of a 50 us kernel.  The key holds
// everything the encoding depends on, so a hit is always valid (a map describes addresses, not contents); the table
// is small, shared by all threads and replaced round-robin.
struct MapKey {
  const void* ptr;
  int kind, dtype, B, H, L, box;
  int64_t st[3];
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && kind == o.kind && dtype == o.dtype && B == o.B && H == o.H && L == o.L && box == o.box &&
           st[0] == o.st[0] && st[1] == o.st[1] && st[2] == o.st[2];
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  std::mutex mu;
  MapKey keys[kMapCacheSize];
  CUtensorMap maps[kMapCacheSize];
  int used = 0, next = 0;
};
MapCache& map_cache() {
  static MapCache c;
  return c;
}

template <typename EncodeFn>
int cached_map(CUtensorMap* m, const MapKey& key, EncodeFn encode) {
  MapCache& c = map_cache();
  {
    std::lock_guard<std::mutex> lock(c.mu);
    for (int i = 0; i < c.used; ++i)
      if (c.keys[i] == key) {
        *m = c.maps[i];
        return LMK_OK;
      }
  }
  const int rc = encode(m);
  if (rc != LMK_OK) return rc;
  std::lock_guard<std::mutex> lock(c.mu);
  const int slot = c.used < kMapCacheSize ? c.used++ : (c.next++ % kMapCacheSize);
  c.keys[slot] = key;
  c.maps[slot] = *m;
  return LMK_OK;
}

// [B, H, L, 128] tensor with element strides {b, h, row}; box = 64 features x `box_rows` rows, 128-byte swizzle
int make_map_4d(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3], int box_rows) {
  const MapKey key{ptr, 4, dtype, B, H, L, box_rows, {st[0], st[1], st[2]}};
  return cached_map(m, key, [&](CUtensorMap* out) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[0] * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(out, dtype == LMK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with %d", (int)r);
    return (int)LMK_OK;
  });
}

// landmark keys: k viewed as [B, H, L/64, 64, 128]; box = 64 features x 1 row-in-block x 64 blocks
int make_map_landmarks(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3],
                       int lm_box) {
  const MapKey key{ptr, 5, dtype, B, H, L, lm_box, {st[0], st[1], st[2]}};
  return cached_map(m, key, [&](CUtensorMap* out) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[5] = {(cuuint64_t)kD, (cuuint64_t)kBlk, (cuuint64_t)(L / kBlk), (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[4] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[2] * 2 * kBlk, (cuuint64_t)st[1] * 2,
                             (cuuint64_t)st[0] * 2};
    cuuint32_t box[5] = {64, 1, (cuuint32_t)lm_box, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = enc(out, dtype == LMK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled (landmarks) failed with %d", (int)r);
    return (int)LMK_OK;
  });
}

// Per-device launch facts, looked up once: the SM count and the opt-in to large dynamic shared memory for every kernel
// of this file (the attribute is a property of the function on a device, not of a launch).
constexpr int kMaxDevices = 64;
struct DeviceFacts {
  bool ready = false;
  int n_sm = 0;
};
constexpr size_t kSmemFwd2 = 1024 + 65536 + kFwd2Stages * 32768 + sizeof(Fwd2Smem);
constexpr size_t kSmemFwd = 1024 + 32768 + kFwdStages * 32768 + sizeof(FwdSmem);
constexpr size_t kSmemDkv = 1024 + 65536 + kDkvStages * 65536 + 32768 + sizeof(DkvSmem);
constexpr size_t kSmemDq = 1024 + 65536 + kDqStages * 32768 + 32768 + sizeof(DqSmem);

int device_facts(const DeviceFacts** out) {
  static std::mutex mu;
  static DeviceFacts facts[kMaxDevices];
  int dev = 0;
  LMK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(LMK_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  DeviceFacts& f = facts[dev];
  if (!f.ready) {
    LMK_CUDA(cudaDeviceGetAttribute(&f.n_sm, cudaDevAttrMultiProcessorCount, dev));
    const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    LMK_CUDA(cudaFuncSetAttribute(sm100_fwd2_kernel<true>, attr, (int)kSmemFwd2));
    LMK_CUDA(cudaFuncSetAttribute(sm100_fwd2_kernel<false>, attr, (int)kSmemFwd2));
    LMK_CUDA(cudaFuncSetAttribute(sm100_fwd_kernel<true>, attr, (int)kSmemFwd));
    LMK_CUDA(cudaFuncSetAttribute(sm100_fwd_kernel<false>, attr, (int)kSmemFwd));
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dq_kernel<true>, attr, (int)kSmemDq));
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dq_kernel<false>, attr, (int)kSmemDq));
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dkv_kernel<true>, attr, (int)kSmemDkv));
    LMK_CUDA(cudaFuncSetAttribute(sm100_bwd_dkv_kernel<false>, attr, (int)kSmemDkv));
    f.ready = true;
  }
  *out = &f;
  return LMK_OK;
}

// Upper bound on the CTAs of the persistent backward kernels; 0 = one per SM.  Only the tests lower it (to make every
// CTA walk through several work units at small sizes).
std::atomic<int> g_max_ctas{0};

// A tensor the TMA unit can address: 16-byte aligned base, positive strides that are multiples of 16 bytes
// (an expanded view has stride 0), rows at least one head apart.
bool tma_ok(const void* p, const int64_t st[3]) {
  return ((uintptr_t)p % 16 == 0) && st[0] > 0 && st[1] > 0 && st[0] % 8 == 0 && st[1] % 8 == 0 && st[2] % 8 == 0 &&
         st[2] >= kD;
}

}  // namespace

bool attn_sm100_supported(int B, int H, int Lq, int Lk, int D, int block, int dtype) {
  return (dtype == LMK_BF16 || dtype == LMK_F16) && D == kD && block == kBlk && Lq >= kQTile && Lq % kQTile == 0 &&
         Lk % kBlk == 0 && Lk >= Lq && B >= 1 && H >= 1;
}

bool attn_sm100_operands_ok(const AttnParams& p, bool backward) {
  if (!tma_ok(p.q, p.qs) || !tma_ok(p.k, p.ks) || !tma_ok(p.v, p.vs)) return false;
  if (backward && ((uintptr_t)p.dO % 16 != 0 || (uintptr_t)p.o % 16 != 0)) return false;
  return true;
}

void attn_sm100_set_max_ctas(int n) { g_max_ctas.store(n > 0 ? n : 0); }

int tensor_map_4d(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3], int box_rows) {
  bind_context();
  return make_map_4d(m, ptr, dtype, B, H, L, st, box_rows);
}
bool tensor_map_operand_ok(const void* p, const int64_t st[3]) { return tma_ok(p, st); }

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
  const DeviceFacts* facts = nullptr;
  if ((rc = device_facts(&facts)) != LMK_OK) return rc;
  if (p.Lq % (2 * kQTile) == 0) {
    dim3 grid(p.B * p.H, p.Lq / (2 * kQTile));
    if (dtype == LMK_BF16)
      sm100_fwd2_kernel<true><<<grid, kFwd2Threads, kSmemFwd2, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                     lm_box, scale_log2);
    else
      sm100_fwd2_kernel<false><<<grid, kFwd2Threads, kSmemFwd2, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                      lm_box, scale_log2);
  } else {
    dim3 grid(p.B * p.H, p.Lq / kQTile);
    if (dtype == LMK_BF16)
      sm100_fwd_kernel<true><<<grid, kFwdThreads, kSmemFwd, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                  lm_box, scale_log2);
    else
      sm100_fwd_kernel<false><<<grid, kFwdThreads, kSmemFwd, st>>>(tq, tk, tv, tl, p.o, p.L, p.M, p.H, p.Lq, p.Lk,
                                                                   lm_box, scale_log2);
  }
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

int attn_sm100_bwd(const AttnParams& p, int dtype, cudaStream_t st) {
  if (!tma_ok(p.q, p.qs) || !tma_ok(p.k, p.ks) || !tma_ok(p.v, p.vs) || (uintptr_t)p.dO % 16 != 0 ||
      (uintptr_t)p.o % 16 != 0)
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
  const float scale_log2 = p.scale * kLog2e;
  const size_t smem_dkv = kSmemDkv, smem_dq = kSmemDq;
  CUtensorMap to;
  if ((rc = make_map_4d(&to, p.o, dtype, p.B, p.H, p.Lq, dense, kQTile)) != LMK_OK) return rc;
  const DeviceFacts* facts = nullptr;
  if ((rc = device_facts(&facts)) != LMK_OK) return rc;
  int n_sm = facts->n_sm;
  const int cap = g_max_ctas.load();
  if (cap >= 1 && cap < n_sm) n_sm = cap;
  const int dkv_units = ((p.Lk / kBlk + 1) / 2) * p.B * p.H;
  const int dq_units = (p.Lq / kQTile) * p.B * p.H;
  dim3 grid_dkv(dkv_units < n_sm ? dkv_units : n_sm), grid_dq(dq_units < n_sm ? dq_units : n_sm);
  // Both launches can carry the programmatic-stream-serialization attribute.  The dQ kernel waits for the kernel before it
  // right after its set-up (only the set-up overlaps).  The dK/dV kernel reads q, k, v, dO, L, M, which were complete
  // before the dQ kernel started, and `delta`, which the dQ kernel writes: its loads and S / dP products start on
  // every SM the dQ kernel has left, and only its softmax threads wait (griddepcontrol.wait) before they read delta.
  // The attribute is only attached while the stream is being captured into a CUDA graph: there it becomes a programmatic
  // edge that costs nothing per replay, whereas an eager launch that carries launch attributes takes a slower path
  // through the driver (measured: ~50 us more host time per call, which makes a 0.2 ms step host-bound).
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  LMK_CUDA(cudaStreamIsCapturing(st, &capturing));
  const unsigned n_attrs = capturing == cudaStreamCaptureStatusActive ? 1u : 0u;
  cudaLaunchConfig_t cfg_dq = {}, cfg_dkv = {};
  cfg_dq.gridDim = grid_dq;  cfg_dq.blockDim = dim3(kDqThreads);  cfg_dq.dynamicSmemBytes = smem_dq;  cfg_dq.stream = st;
  cfg_dq.attrs = pdl;  cfg_dq.numAttrs = n_attrs;
  cfg_dkv.gridDim = grid_dkv;  cfg_dkv.blockDim = dim3(kBwdThreads);  cfg_dkv.dynamicSmemBytes = smem_dkv;
  cfg_dkv.stream = st;  cfg_dkv.attrs = pdl;  cfg_dkv.numAttrs = n_attrs;
  const float* Lc = p.L;
  const float* Mc = p.M;
  const float* deltac = delta;
  const int BH = p.B * p.H;
#define LMK_BWD_LAUNCH(BF)                                                                                          \
  do {                                                                                                              \
    LMK_CUDA(cudaLaunchKernelEx(&cfg_dq, sm100_bwd_dq_kernel<BF>, tq, tk, tv, tdo, to, Lc, Mc, delta, p.dq, p.H, BH, \
                                p.Lq, p.Lk, p.scale, scale_log2));                                                  \
    LMK_CUDA(cudaLaunchKernelEx(&cfg_dkv, sm100_bwd_dkv_kernel<BF>, tq, tk, tv, tdo, Lc, Mc, deltac, p.dk, p.dv,    \
                                p.H, BH, p.Lq, p.Lk, p.scale, scale_log2));                                         \
  } while (0)
  if (dtype == LMK_BF16) LMK_BWD_LAUNCH(true);
  else LMK_BWD_LAUNCH(false);
#undef LMK_BWD_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

size_t attn_sm100_bwd_workspace(int B, int H, int Lq, int, int) { return sizeof(float) * (size_t)B * H * Lq; }

// Device address of the status word on the current device, for kernels compiled in other translation units.
int* device_status_word() {
  int* ptr = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_lmk_status) != cudaSuccess) return nullptr;
  return ptr;
}

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
