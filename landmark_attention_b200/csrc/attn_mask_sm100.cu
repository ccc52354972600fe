// Fused landmark attention for ARBITRARY landmark positions (sm_100a: TMA + tcgen05 + TMEM).
//
// This is the attention of lm_benchmark's CausalSelfAttention.forward (lm_benchmark/models/landmark.py:196-236) with
// its mask block (:210-224) and grouped softmax (:37-119) folded into the kernels: the landmark flags arrive as one
// byte per (batch row, key) -- is_mem [B, Lk] -- and group ids are derived inside the kernel, so no [B,H,Lq,Lk] score,
// mask or probability tensor ever exists.  Landmarks may sit anywhere (training windows are cut at random offsets,
// optim/utils.py:21-26, with a landmark after every 50 tokens: groups of 51 keys that straddle the 64-key tiles).
//
// Semantics for the query at key position p (p = Lk - Lq + row), with c(j) = number of landmarks strictly before j:
//   own section  = non-landmark keys j <= p with c(j) == c(p)              (the keys of the query's unfinished group)
//   group g < c(p) = non-landmark keys with c(j) == g, closed by landmark l_g (the last key of the group, l_g < p)
//   outer softmax over {score(l_g) : g < c(p)} U {score(j) : j in own section}  -> G_g, P_j (own section)
//   P_j = G_g * softmax_inside_group_g(score)_j for j in group g; landmark keys themselves carry no value weight;
//   a query that is itself a landmark does not see its own key; rows with nothing visible give 0.
//
// Shape contract: bf16 / fp16, head dim 128, Lq a multiple of 128, Lk and Lk - Lq multiples of 64, at most
// kMaxGroups landmarks visible to any query, Lk <= 64 * kMaxKeyTiles.
//
// Forward (sm100_mask_fwd_kernel), one CTA per (128 query rows, batch*head), two passes over the visible key tiles:
//   pass 1: S = Q K^T per 64-key tile; every softmax thread (= query row) walks its row once, keeping an online
//           (max, sum) of the open group and of the outer softmax; when the walk meets a landmark the group is closed:
//           A_g = max_g + log2(sum_g) - score(l_g)  (log2 domain) is stored per (row, group).  After the last tile
//           R = max_outer + log2(sum_outer) is known and every probability is exp2(x_j - A_g - R) (own section: A = 0):
//   pass 2: S again, P = exp2(x - z) written as 16-bit over the K tile, O += P V.  O needs no rescaling or final division.
//   A [B*H, G, Lq] and R [B*H, Lq] are kept for the backward pass.
// Backward:
//   sm100_mask_bwd_dq_kernel, CTA per (128 query rows, batch*head): delta = rowsum(O * dO); pass 1 accumulates
//     T_g = sum_{j in g} P_j dP_j and stores nD_g = T_g / G_g per (row, group); pass 2 forms
//     dS_j = P_j (dP_j - nD_g) scale (group g), P_j (dP_j - delta) scale (own section), G_g (nD_g - delta) scale (landmark l_g)
//     and accumulates dQ += dS K.
//   sm100_mask_bwd_dkv_kernel, CTA per (64-key tile, batch*head) streaming the query tiles that see it: rebuilds P and dS
//     from A, R, nD, delta and accumulates dV^T += dO^T P, dK^T += Q^T dS (transposed accumulators, M = 128).
// The same identities as the regular-pattern kernels in attn_sm100.cu apply (see there for the derivation).
#include <mutex>
#include "common.cuh"
#include "attn_params.h"
#include "sm100_ptx.cuh"

namespace lmk {
namespace {

using namespace ptx;

constexpr int kD = 128;
constexpr int kKT = 64;                  // keys per tile
constexpr int kQT = 128;                 // query rows per tile
constexpr int kMaxGroups = 64;           // closed groups per query row the kernels keep statistics for
constexpr int kMaxKeyTiles = 512;        // Lk <= 32768
constexpr uint32_t kTile = 16384;        // [128 x 64] 16-bit tile
constexpr uint32_t kHalf = 8192;         // [64 x 64] 16-bit tile
constexpr float kLog2e = 1.4426950408889634f;

enum { kErrMaskFwd = 401, kErrMaskDq = 411, kErrMaskDkv = 421, kErrMaskGroups = 431 };

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

// Tiles written by the softmax threads are [128 x 64] 16-bit, K-major, with the 128-byte swizzle.
// 16 consecutive keys (8 packed words) of one row of such a tile: 16-byte chunks 2c and 2c+1 of the row
__device__ __forceinline__ void store_row16_sw128(uint32_t tile_base, int row, int c, const uint32_t (&w)[8]) {
  const uint32_t row_addr = tile_base + row * 128;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t addr = row_addr + (((2 * c + h) ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * h]), "r"(w[4 * h + 1]),
                 "r"(w[4 * h + 2]), "r"(w[4 * h + 3])
                 : "memory");
  }
}

// The softmax threads walk a 64-key tile in four chunks of 16 keys loaded from TMEM inside a runtime loop: the code of
// one chunk (a branch-free path for chunks without a landmark, a per-key path otherwise) stays resident in the
// instruction cache and the row needs 16 registers instead of 64.

// ---------------------------------------------------------------------------------------------- landmark bookkeeping
// kmask[t] bit j = key 64 t + j of batch row b is a landmark; gbase[t] = landmarks before tile t.  Built by the
// four softmax warps from the byte flags; n_kt tiles (the ones at or below the CTA's diagonal).
__device__ __forceinline__ void build_masks(const uint8_t* __restrict__ is_mem_row, int n_kt, uint64_t* kmask,
                                            int* gbase, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  for (int t = warp; t < n_kt; t += 4) {
    const unsigned lo = __ballot_sync(0xffffffffu, is_mem_row[t * kKT + lane] != 0);
    const unsigned hi = __ballot_sync(0xffffffffu, is_mem_row[t * kKT + 32 + lane] != 0);
    if (lane == 0) kmask[t] = (uint64_t)lo | ((uint64_t)hi << 32);
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (tid == 0) {
    int run = 0;
    for (int t = 0; t < n_kt; ++t) {
      gbase[t] = run;
      run += __popcll(kmask[t]);
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// per-row view of one key tile: which local keys the row sees and which landmark (if any) is its own key
struct RowTile {
  int lim;        // local keys 0..lim are visible (-1: none, 63: all)
  int own;        // local index of the row's own key in this tile, or -1
};
__device__ __forceinline__ RowTile row_tile(int kt, int kd, int jl_own) {
  RowTile r;
  r.lim = kt < kd ? 63 : (kt == kd ? jl_own : -1);
  r.own = kt == kd ? jl_own : -1;
  return r;
}

// online (max, sum) in the log2 domain
struct Online {
  float m, s;
  __device__ __forceinline__ void reset() { m = -INFINITY; s = 0.f; }
  __device__ __forceinline__ void add(float x) {           // x finite
    const float mn = fmaxf(m, x);
    s = s * ex2(m - mn) + ex2(x - mn);
    m = mn;
  }
  __device__ __forceinline__ void add4(float a, float b, float c, float d) {   // -inf entries are skipped
    const float mn = fmaxf(fmaxf(m, fmaxf(a, b)), fmaxf(c, d));
    const float ms = mn == -INFINITY ? 0.f : mn;
    s = s * ex2(m - ms) + (ex2(a - ms) + ex2(b - ms)) + (ex2(c - ms) + ex2(d - ms));
    m = mn;
  }
  __device__ __forceinline__ void merge(float m2, float s2) {                  // s2 > 0, m2 finite
    const float mn = fmaxf(m, m2);
    s = s * ex2(m - mn) + s2 * ex2(m2 - mn);
    m = mn;
  }
};

// ---------------------------------------------------------------------------------------------- forward
constexpr int kMfStages = 2;      // 2 stages + statistics sized for the launch keep two CTAs on an SM at training shapes
constexpr int kMfThreads = 192;

struct MfSmem {
  uint64_t q_full;
  uint64_t full[kMfStages];
  uint64_t empty[kMfStages];
  uint64_t p_ready[kMfStages];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t o_full;
  uint32_t tmem_base;
};

// dynamic shared memory of the forward kernel for G groups and n_kt key tiles (n_kt rounded up to an even count)
__host__ __device__ constexpr size_t mf_smem_bytes(int G, int n_kt) {
  return 1024 + 32768 + kMfStages * 32768 + (size_t)G * kQT * 4 + (size_t)((n_kt + 1) & ~1) * 12 + sizeof(MfSmem);
}

template <bool kBf16>
__global__ void __launch_bounds__(kMfThreads, 2)
sm100_mask_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const uint8_t* __restrict__ is_mem, int64_t is_mem_stride,
                      void* __restrict__ o_ptr, float* __restrict__ R_ptr, float* __restrict__ A_ptr, int H, int Lq,
                      int Lk, int G, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t q_tile = base;
  auto k_slot = [&](int s) { return base + 32768u + (uint32_t)s * 32768u; };       // K tile, later P
  auto v_slot = [&](int s) { return base + 32768u + (uint32_t)s * 32768u + 16384u; };
  const int kt_cap = (Lk / kKT + 1) & ~1;                                           // entries of the two tables below
  float* Asm = reinterpret_cast<float*>(gen + 32768 + kMfStages * 32768);           // [G][128]
  uint64_t* kmask = reinterpret_cast<uint64_t*>(Asm + (size_t)G * kQT);
  int* gbase = reinterpret_cast<int*>(kmask + kt_cap);
  MfSmem* sm = reinterpret_cast<MfSmem*>(gbase + kt_cap);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQT;
  const int t = n_tiles - 1 - (int)blockIdx.y;          // heaviest tiles first
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
  const int pos0 = (Lk - Lq) + t * kQT;                 // key position of row 0 (a multiple of 64)
  const int n_kt = pos0 / kKT + 2;                      // key tiles 0 .. diagonal
  const int total = 2 * n_kt;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->q_full), 1);
    for (int s = 0; s < kMfStages; ++s) {
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
      const uint32_t qb = smem_u32(&sm->q_full);
      mbar_arrive_expect_tx(qb, 2 * kTile);
      tma_load_4d(q_tile, &tm_q, qb, 0, t * kQT, h, b);
      tma_load_4d(q_tile + kTile, &tm_q, qb, 64, t * kQT, h, b);
      for (int i = 0; i < total; ++i) {
        const int s = i % kMfStages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kMfStages) & 1) ^ 1, status, kErrMaskFwd);
        const uint32_t fb = smem_u32(&sm->full[s]);
        const int kt = i < n_kt ? i : i - n_kt;
        if (i < n_kt) {
          mbar_arrive_expect_tx(fb, kTile);
          tma_load_4d(k_slot(s), &tm_k, fb, 0, kt * kKT, h, b);
          tma_load_4d(k_slot(s) + kHalf, &tm_k, fb, 64, kt * kKT, h, b);
        } else {
          mbar_arrive_expect_tx(fb, 2 * kTile);
          tma_load_4d(k_slot(s), &tm_k, fb, 0, kt * kKT, h, b);
          tma_load_4d(k_slot(s) + kHalf, &tm_k, fb, 64, kt * kKT, h, b);
          tma_load_4d(v_slot(s), &tm_v, fb, 0, kt * kKT, h, b);
          tma_load_4d(v_slot(s) + kHalf, &tm_v, fb, 64, kt * kKT, h, b);
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
      mbar_wait(smem_u32(&sm->q_full), 0, status, kErrMaskFwd + 1);
      const uint64_t dq = smem_desc_sw128(q_tile, 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(k_slot(0), 16, 1024);
      const uint64_t dv0 = smem_desc_sw128(v_slot(0), kHalf, 1024);
      auto issue_s = [&](int j) {
        const int s = j % kMfStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kMfStages) & 1, status, kErrMaskFwd + 1);
        if (j >= 2) mbar_wait(smem_u32(&sm->s_free[sb]), ((j / 2) & 1) ^ 1, status, kErrMaskFwd + 1);
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (uint32_t)s * 32768u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_s0 + sb * 64, desc_advance(dq, kmajor_step(kk, kTile)),
                     desc_advance(dk, kmajor_step(kk, kHalf)), idesc_s, kk > 0);
        mma_commit(smem_u32(&sm->s_full[sb]));
      };
      issue_s(0);
      bool o_started = false;
      for (int i = 0; i < total; ++i) {
        if (i + 1 < total) issue_s(i + 1);
        const int s = i % kMfStages;
        mbar_wait(smem_u32(&sm->p_ready[s]), (i / kMfStages) & 1, status, kErrMaskFwd + 1);
        tc_fence_after();
        if (i >= n_kt) {
          const uint64_t dp = desc_advance(dk0, (uint32_t)s * 32768u);
          const uint64_t dv = desc_advance(dv0, (uint32_t)s * 32768u);
#pragma unroll
          for (int kk = 0; kk < kKT / 16; ++kk)
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
    build_masks(is_mem + (int64_t)b * is_mem_stride, n_kt, kmask, gbase, tid);
    const int pos = pos0 + row;
    const int kd = pos / kKT, jl_own = pos % kKT;
    // landmarks strictly before the row's own position = number of closed groups the row sees
    const int c_row = gbase[kd] + __popcll(kmask[kd] & ((1ull << jl_own) - 1ull));
    if (c_row > G) atomicCAS(status, 0, kErrMaskGroups);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    Online grp, outer;
    grp.reset();
    outer.reset();
    float R = INFINITY;
    for (int i = 0; i < total; ++i) {
      const int sb = i & 1, s = i % kMfStages;
      const int kt = i < n_kt ? i : i - n_kt;
      mbar_wait(smem_u32(&sm->s_full[sb]), (i / 2) & 1, status, kErrMaskFwd + 2);
      tc_fence_after();
      const RowTile rt = row_tile(kt, kd, jl_own);
      const uint64_t mask = kmask[kt];
      int g = gbase[kt];
      const uint32_t ts = tmem_s0 + sb * 64 + lane_base;
      auto zof = [&](int gg) { return gg < c_row ? Asm[(gg < G ? gg : G - 1) * kQT + row] + R : R; };
      float z = i < n_kt ? 0.f : zof(g);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float sv[16];
        {
          uint32_t xr[16];
          tmem_ld_32x32b_x16(ts + c * 16, xr);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) sv[e] = __uint_as_float(xr[e]) * scale_log2;
        }
        if (c == 3) {                 // the S buffer has been read for the last time
          tc_fence_before();
          mbar_arrive(smem_u32(&sm->s_free[sb]));
        }
        const uint32_t m16 = (uint32_t)(mask >> (16 * c)) & 0xffffu;      // uniform
        const int j0 = 16 * c;
        if (i < n_kt) {
          // ---------------- pass 1: statistics
          if (m16 == 0u) {
#pragma unroll
            for (int e = 0; e < 16; e += 4)
              grp.add4(j0 + e <= rt.lim ? sv[e] : -INFINITY, j0 + e + 1 <= rt.lim ? sv[e + 1] : -INFINITY,
                       j0 + e + 2 <= rt.lim ? sv[e + 2] : -INFINITY, j0 + e + 3 <= rt.lim ? sv[e + 3] : -INFINITY);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j = j0 + e;
              if ((m16 >> e) & 1u) {                          // landmark (uniform)
                if (j <= rt.lim && j != rt.own) {             // it closes group g for this row
                  const float A = grp.s > 0.f ? grp.m + __log2f(grp.s) - sv[e] : INFINITY;
                  if (g < G) Asm[g * kQT + row] = A;
                  outer.add(sv[e]);
                  grp.reset();
                }
                ++g;
              } else if (j <= rt.lim) {
                grp.add(sv[e]);
              }
            }
          }
        } else {
          // ---------------- pass 2: probabilities
          uint32_t w[8];
          if (m16 == 0u) {
#pragma unroll
            for (int e = 0; e < 16; e += 2)
              w[e / 2] = pack2<kBf16>(j0 + e <= rt.lim ? ex2(sv[e] - z) : 0.f,
                                      j0 + e + 1 <= rt.lim ? ex2(sv[e + 1] - z) : 0.f);
          } else {
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              float p[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if ((m16 >> (e + h)) & 1u) {                  // landmark keys carry no weight; next group starts
                  p[h] = 0.f;
                  ++g;
                  z = zof(g);
                } else {
                  p[h] = j0 + e + h <= rt.lim ? ex2(sv[e + h] - z) : 0.f;
                }
              }
              w[e / 2] = pack2<kBf16>(p[0], p[1]);
            }
          }
          store_row16_sw128(k_slot(s), row, c, w);
        }
      }
      if (i == n_kt - 1) {
        // the open group is the row's own section: its keys enter the outer softmax directly
        if (grp.s > 0.f) outer.merge(grp.m, grp.s);
        R = outer.s > 0.f ? outer.m + __log2f(outer.s) : INFINITY;
      }
      if (i >= n_kt) fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sm->p_ready[s]));
    }
    // statistics for the backward pass: R per row, A per (group, row) for the groups the row sees
    R_ptr[(int64_t)bh * Lq + t * kQT + row] = R;
    {
      const int ng = c_row < G ? c_row : G;
      float* Ag = A_ptr + (int64_t)bh * G * Lq + t * kQT + row;
      for (int g = 0; g < ng; ++g) Ag[(int64_t)g * Lq] = Asm[g * kQT + row];
    }
    // ------------------------------------------------------------------ epilogue
    mbar_wait(smem_u32(&sm->o_full), 0, status, kErrMaskFwd + 3);
    tc_fence_after();
    const int grow = t * kQT + row;
    uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(o_ptr) + ((int64_t)bh * Lq + grow) * kD);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_o + c * 32 + lane_base, r);
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
    tmem_dealloc(tmem, 256);
  }
}


// ---------------------------------------------------------------------------------------------- backward: dQ (+ nD)
constexpr int kMqStages = 2;
constexpr int kMqThreads = 192;

struct MqSmem {
  uint64_t qdo_full;
  uint64_t full[kMqStages];
  uint64_t empty[kMqStages];
  uint64_t ds_ready[kMqStages];
  uint64_t sdp_full[2];
  uint64_t sdp_free[2];
  uint64_t acc_full;
  uint32_t tmem_base;
};

__host__ __device__ constexpr size_t mq_smem_bytes(int G) {
  return 1024 + 65536 + kMqStages * 32768 + (size_t)2 * G * kQT * 4 + kMaxKeyTiles * 12 + sizeof(MqSmem);
}

// 16 bytes of 16-bit values times 16 bytes of 16-bit values, accumulated in fp32
template <bool kBf16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 fa, fb;
    if (kBf16) {
      fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[e]));
      fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[e]));
    } else {
      fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[e]));
      fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[e]));
    }
    acc = fmaf(fa.x, fb.x, acc);
    acc = fmaf(fa.y, fb.y, acc);
  }
  return acc;
}

template <bool kBf16>
__global__ void __launch_bounds__(kMqThreads, 1)
sm100_mask_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                         const uint8_t* __restrict__ is_mem, int64_t is_mem_stride, const void* __restrict__ o_ptr,
                         const void* __restrict__ do_ptr, const float* __restrict__ R_ptr,
                         const float* __restrict__ A_ptr, float* __restrict__ delta_ptr, float* __restrict__ nD_ptr,
                         void* __restrict__ dq_ptr, int H, int Lq, int Lk, int G, float scale, float scale_log2,
                         int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t q_tile = base, do_tile = base + 32768u;
  auto k_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u; };
  auto v_slot = [&](int s) { return base + 65536u + (uint32_t)s * 32768u + 16384u; };   // V tile, later dS
  float* Asm = reinterpret_cast<float*>(gen + 65536 + kMqStages * 32768);                // [G][128]
  float* nDsm = Asm + (size_t)G * kQT;                                                   // [G][128]
  uint64_t* kmask = reinterpret_cast<uint64_t*>(nDsm + (size_t)G * kQT);
  int* gbase = reinterpret_cast<int*>(kmask + kMaxKeyTiles);
  MqSmem* sm = reinterpret_cast<MqSmem*>(gbase + kMaxKeyTiles);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQT;
  const int t = n_tiles - 1 - (int)blockIdx.y;
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
  const int pos0 = (Lk - Lq) + t * kQT;
  const int n_kt = pos0 / kKT + 2;
  const int total = 2 * n_kt;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->qdo_full), 1);
    for (int s = 0; s < kMqStages; ++s) {
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
      mbar_arrive_expect_tx(qb, 4 * kTile);
      tma_load_4d(q_tile, &tm_q, qb, 0, t * kQT, h, b);
      tma_load_4d(q_tile + kTile, &tm_q, qb, 64, t * kQT, h, b);
      tma_load_4d(do_tile, &tm_do, qb, 0, t * kQT, h, b);
      tma_load_4d(do_tile + kTile, &tm_do, qb, 64, t * kQT, h, b);
      for (int i = 0; i < total; ++i) {
        const int s = i % kMqStages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kMqStages) & 1) ^ 1, status, kErrMaskDq);
        const uint32_t fb = smem_u32(&sm->full[s]);
        const int kt = i < n_kt ? i : i - n_kt;
        mbar_arrive_expect_tx(fb, 2 * kTile);
        tma_load_4d(k_slot(s), &tm_k, fb, 0, kt * kKT, h, b);
        tma_load_4d(k_slot(s) + kHalf, &tm_k, fb, 64, kt * kKT, h, b);
        tma_load_4d(v_slot(s), &tm_v, fb, 0, kt * kKT, h, b);
        tma_load_4d(v_slot(s) + kHalf, &tm_v, fb, 64, kt * kKT, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      constexpr uint32_t idesc_q = instr_desc_f16(fmt, 128, 128, 0, 1);   // dQ += dS K  (K is MN-major)
      mbar_wait(smem_u32(&sm->qdo_full), 0, status, kErrMaskDq + 1);
      const uint64_t dq = smem_desc_sw128(q_tile, 16, 1024), ddo = smem_desc_sw128(do_tile, 16, 1024);
      const uint64_t dk0 = smem_desc_sw128(k_slot(0), 16, 1024), dv0 = smem_desc_sw128(v_slot(0), 16, 1024);
      const uint64_t dk0t = smem_desc_sw128(k_slot(0), kHalf, 1024);
      auto issue_sdp = [&](int j) {
        const int s = j % kMqStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kMqStages) & 1, status, kErrMaskDq + 1);
        if (j >= 2) mbar_wait(smem_u32(&sm->sdp_free[sb]), ((j / 2) & 1) ^ 1, status, kErrMaskDq + 1);
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (uint32_t)s * 32768u), dv = desc_advance(dv0, (uint32_t)s * 32768u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_s + sb * 64, desc_advance(dq, kmajor_step(kk, kTile)), desc_advance(dk, kmajor_step(kk, kHalf)),
                     idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_dp + sb * 64, desc_advance(ddo, kmajor_step(kk, kTile)),
                     desc_advance(dv, kmajor_step(kk, kHalf)), idesc_s, kk > 0);
        mma_commit(smem_u32(&sm->sdp_full[sb]));
      };
      issue_sdp(0);
      bool started = false;
      for (int i = 0; i < total; ++i) {
        if (i + 1 < total) issue_sdp(i + 1);
        const int s = i % kMqStages;
        mbar_wait(smem_u32(&sm->ds_ready[s]), (i / kMqStages) & 1, status, kErrMaskDq + 1);
        tc_fence_after();
        if (i >= n_kt) {
          const uint64_t dds = desc_advance(dv0, (uint32_t)s * 32768u), dkt = desc_advance(dk0t, (uint32_t)s * 32768u);
#pragma unroll
          for (int kk = 0; kk < kKT / 16; ++kk)
            mma_f16_ss(tmem_dq, desc_advance(dds, kk * 32), desc_advance(dkt, kk * 2048), idesc_q,
                       (started || kk > 0) ? 1u : 0u);
          started = true;
        }
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->acc_full));
    }
    __syncwarp();
  } else {
    const int row = tid;
    build_masks(is_mem + (int64_t)b * is_mem_stride, n_kt, kmask, gbase, tid);
    const int pos = pos0 + row;
    const int kd = pos / kKT, jl_own = pos % kKT;
    const int c_row = gbase[kd] + __popcll(kmask[kd] & ((1ull << jl_own) - 1ull));
    const int ng = c_row < G ? c_row : G;
    const int64_t grow = (int64_t)bh * Lq + t * kQT + row;
    const float R = R_ptr[grow];
    {
      const float* Ag = A_ptr + (int64_t)bh * G * Lq + t * kQT + row;
      for (int g = 0; g < ng; ++g) Asm[g * kQT + row] = Ag[(int64_t)g * Lq];
    }
    // delta = rowsum(O * dO) from global memory (each thread its own row)
    float delta = 0.f;
    {
      const uint4* orow = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(o_ptr) + grow * kD);
      const uint4* grw = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(do_ptr) + grow * kD);
#pragma unroll 4
      for (int c = 0; c < kD / 8; ++c) delta = dot8<kBf16>(orow[c], grw[c], delta);
    }
    delta_ptr[grow] = delta;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    auto zof = [&](int gg) { return gg < c_row ? Asm[(gg < G ? gg : G - 1) * kQT + row] + R : R; };
    float T = 0.f;
    for (int i = 0; i < total; ++i) {
      const int sb = i & 1, s = i % kMqStages;
      const int kt = i < n_kt ? i : i - n_kt;
      mbar_wait(smem_u32(&sm->sdp_full[sb]), (i / 2) & 1, status, kErrMaskDq + 2);
      tc_fence_after();
      const RowTile rt = row_tile(kt, kd, jl_own);
      const uint64_t mask = kmask[kt];
      int g = gbase[kt];
      float z = zof(g);
      float sub = (i >= n_kt && g < c_row) ? nDsm[(g < G ? g : G - 1) * kQT + row] : delta;
      const uint32_t ts = tmem_s + sb * 64 + lane_base, td = tmem_dp + sb * 64 + lane_base;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float xv[16], dp[16];
        {
          uint32_t xr[16], dr[16];
          tmem_ld_32x32b_x16(ts + c * 16, xr);
          tmem_ld_32x32b_x16(td + c * 16, dr);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            xv[e] = __uint_as_float(xr[e]) * scale_log2;
            dp[e] = __uint_as_float(dr[e]);
          }
        }
        if (c == 3) {                 // S and dP have been read for the last time
          tc_fence_before();
          mbar_arrive(smem_u32(&sm->sdp_free[sb]));
        }
        const uint32_t m16 = (uint32_t)(mask >> (16 * c)) & 0xffffu;      // uniform
        const int j0 = 16 * c;
        if (i < n_kt) {
          // ---------------- pass 1: nD_g = (sum_{j in g} P_j dP_j) / G_g for every closed group
          if (m16 == 0u) {
            float t0 = 0.f, t1 = 0.f;                          // two chains instead of one 16-deep dependency
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              t0 = fmaf(j0 + e <= rt.lim ? ex2(xv[e] - z) : 0.f, dp[e], t0);
              t1 = fmaf(j0 + e + 1 <= rt.lim ? ex2(xv[e + 1] - z) : 0.f, dp[e + 1], t1);
            }
            T += t0 + t1;
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j = j0 + e;
              if ((m16 >> e) & 1u) {
                if (j <= rt.lim && j != rt.own) {
                  const float Gp = ex2(xv[e] - R);
                  const float nd = Gp > 0.f ? __fdividef(T, Gp) : 0.f;
                  if (g < G) nDsm[g * kQT + row] = nd;
                  T = 0.f;
                }
                ++g;
                z = zof(g);
              } else if (j <= rt.lim) {
                T = fmaf(ex2(xv[e] - z), dp[e], T);
              }
            }
          }
        } else {
          // ---------------- pass 2: dS
          uint32_t w[8];
          if (m16 == 0u) {
#pragma unroll
            for (int e = 0; e < 16; e += 2)
              w[e / 2] = pack2<kBf16>(j0 + e <= rt.lim ? ex2(xv[e] - z) * (dp[e] - sub) * scale : 0.f,
                                      j0 + e + 1 <= rt.lim ? ex2(xv[e + 1] - z) * (dp[e + 1] - sub) * scale : 0.f);
          } else {
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              float d[2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int j = j0 + e + h;
                if ((m16 >> (e + h)) & 1u) {
                  // landmark l_g: dS = G_g (nD_g - delta) scale when it closes a group for this row (then sub = nD_g)
                  d[h] = (j <= rt.lim && j != rt.own) ? ex2(xv[e + h] - R) * (sub - delta) * scale : 0.f;
                  ++g;
                  z = zof(g);
                  sub = g < c_row ? nDsm[(g < G ? g : G - 1) * kQT + row] : delta;
                } else {
                  d[h] = j <= rt.lim ? ex2(xv[e + h] - z) * (dp[e + h] - sub) * scale : 0.f;
                }
              }
              w[e / 2] = pack2<kBf16>(d[0], d[1]);
            }
          }
          store_row16_sw128(v_slot(s), row, c, w);
        }
      }
      if (i >= n_kt) fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sm->ds_ready[s]));
    }
    {
      float* ndg = nD_ptr + (int64_t)bh * G * Lq + t * kQT + row;
      for (int g = 0; g < ng; ++g) ndg[(int64_t)g * Lq] = nDsm[g * kQT + row];
    }
    mbar_wait(smem_u32(&sm->acc_full), 0, status, kErrMaskDq + 3);
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

// ---------------------------------------------------------------------------------------------- backward: dK, dV
constexpr int kMkStages = 2;
constexpr int kMkThreads = 192;

struct MkSmem {
  uint64_t kv_full;
  uint64_t full[kMkStages];
  uint64_t empty[kMkStages];
  uint64_t sdp_full[2];
  uint64_t sdp_free[2];
  uint64_t pds_ready;
  uint64_t pds_free;
  uint64_t acc_full;
  uint32_t tmem_base;
  uint64_t mask;          // landmark bits of this key tile
  int g0;                 // landmarks before the tile
  int next_lm;            // position of the first landmark at or after the end of the tile (INT_MAX: none)
  int cnt[4];
};

constexpr size_t kMkSmemBytes = 1024 + 32768 + kMkStages * 65536 + 32768 + sizeof(MkSmem);

template <bool kBf16>
__global__ void __launch_bounds__(kMkThreads, 1)
sm100_mask_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                          const uint8_t* __restrict__ is_mem, int64_t is_mem_stride, const float* __restrict__ R_ptr,
                          const float* __restrict__ A_ptr, const float* __restrict__ delta_ptr,
                          const float* __restrict__ nD_ptr, void* __restrict__ dk_ptr, void* __restrict__ dv_ptr,
                          int H, int Lq, int Lk, int G, float scale, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t k_tile = base, v_tile = base + 16384u;
  auto q_slot = [&](int s) { return base + 32768u + (uint32_t)s * 65536u; };
  auto do_slot = [&](int s) { return base + 32768u + (uint32_t)s * 65536u + 32768u; };
  const uint32_t p_tile = base + 32768u + kMkStages * 65536u;
  const uint32_t ds_tile = p_tile + 16384u;
  MkSmem* sm = reinterpret_cast<MkSmem*>(smem_raw + (base - raw) + 32768u + kMkStages * 65536u + 32768u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = Lq / kQT;
  const int kt = blockIdx.y;                            // early key tiles are seen by the most query tiles
  const int bh = blockIdx.x, b = bh / H, h = bh - b * H;
  const int prefix = Lk - Lq;
  const int k0 = kt * kKT;
  const int t_first = k0 > prefix ? (k0 - prefix) / kQT : 0;
  const int n_items = n_tiles - t_first;

  if (tid == 0) {
    mbar_init(smem_u32(&sm->kv_full), 1);
    for (int s = 0; s < kMkStages; ++s) {
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
    if (lane == 0 && n_items > 0) {
      prefetch_tensormap(&tm_q);
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
      prefetch_tensormap(&tm_do);
      const uint32_t kvb = smem_u32(&sm->kv_full);
      mbar_arrive_expect_tx(kvb, 2 * kTile);
      tma_load_4d(k_tile, &tm_k, kvb, 0, k0, h, b);
      tma_load_4d(k_tile + kHalf, &tm_k, kvb, 64, k0, h, b);
      tma_load_4d(v_tile, &tm_v, kvb, 0, k0, h, b);
      tma_load_4d(v_tile + kHalf, &tm_v, kvb, 64, k0, h, b);
      for (int i = 0; i < n_items; ++i) {
        const int s = i % kMkStages;
        mbar_wait(smem_u32(&sm->empty[s]), ((i / kMkStages) & 1) ^ 1, status, kErrMaskDkv);
        const uint32_t fb = smem_u32(&sm->full[s]);
        const int r0 = (t_first + i) * kQT;
        mbar_arrive_expect_tx(fb, 4 * kTile);
        tma_load_4d(q_slot(s), &tm_q, fb, 0, r0, h, b);
        tma_load_4d(q_slot(s) + kTile, &tm_q, fb, 64, r0, h, b);
        tma_load_4d(do_slot(s), &tm_do, fb, 0, r0, h, b);
        tma_load_4d(do_slot(s) + kTile, &tm_do, fb, 64, r0, h, b);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0 && n_items > 0) {
      constexpr uint32_t fmt = kBf16 ? 1u : 0u;
      constexpr uint32_t idesc_s = instr_desc_f16(fmt, 128, 64, 0, 0);
      constexpr uint32_t idesc_t = instr_desc_f16(fmt, 128, 64, 1, 1);
      const uint64_t dk = smem_desc_sw128(k_tile, 16, 1024), dv = smem_desc_sw128(v_tile, 16, 1024);
      const uint64_t dq0 = smem_desc_sw128(q_slot(0), 16, 1024), ddo0 = smem_desc_sw128(do_slot(0), 16, 1024);
      const uint64_t dq0t = smem_desc_sw128(q_slot(0), kTile, 1024), ddo0t = smem_desc_sw128(do_slot(0), kTile, 1024);
      const uint64_t dpt = smem_desc_sw128(p_tile, 16, 1024), ddst = smem_desc_sw128(ds_tile, 16, 1024);
      mbar_wait(smem_u32(&sm->kv_full), 0, status, kErrMaskDkv + 1);
      auto issue_sdp = [&](int j) {
        const int s = j % kMkStages, sb = j & 1;
        mbar_wait(smem_u32(&sm->full[s]), (j / kMkStages) & 1, status, kErrMaskDkv + 1);
        if (j >= 2) mbar_wait(smem_u32(&sm->sdp_free[sb]), ((j / 2) & 1) ^ 1, status, kErrMaskDkv + 1);
        tc_fence_after();
        const uint64_t dq = desc_advance(dq0, (uint32_t)s * 65536u), ddo = desc_advance(ddo0, (uint32_t)s * 65536u);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_s + sb * 64, desc_advance(dq, kmajor_step(kk, kTile)), desc_advance(dk, kmajor_step(kk, kHalf)),
                     idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          mma_f16_ss(tmem_dp + sb * 64, desc_advance(ddo, kmajor_step(kk, kTile)),
                     desc_advance(dv, kmajor_step(kk, kHalf)), idesc_s, kk > 0);
        mma_commit(smem_u32(&sm->sdp_full[sb]));
      };
      issue_sdp(0);
      for (int i = 0; i < n_items; ++i) {
        if (i + 1 < n_items) issue_sdp(i + 1);
        const int s = i % kMkStages;
        mbar_wait(smem_u32(&sm->pds_ready), i & 1, status, kErrMaskDkv + 1);
        tc_fence_after();
        const uint64_t ddot = desc_advance(ddo0t, (uint32_t)s * 65536u), dqt = desc_advance(dq0t, (uint32_t)s * 65536u);
        // dV^T += dO^T P and dK^T += Q^T dS: A = MN-major view of the row-major [128 q x 128 d] tile, B = MN-major view
        // of the [128 q x 64 k] tile; a K-step is 16 query rows = 2048 bytes
#pragma unroll
        for (int kk = 0; kk < kQT / 16; ++kk)
          mma_f16_ss(tmem_dv, desc_advance(ddot, kk * 2048), desc_advance(dpt, kk * 2048), idesc_t,
                     (i > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kQT / 16; ++kk)
          mma_f16_ss(tmem_dk, desc_advance(dqt, kk * 2048), desc_advance(ddst, kk * 2048), idesc_t,
                     (i > 0 || kk > 0) ? 1u : 0u);
        mma_commit(smem_u32(&sm->pds_free));
        mma_commit(smem_u32(&sm->empty[s]));
      }
      mma_commit(smem_u32(&sm->acc_full));
    }
    __syncwarp();
  } else {
    const int row = tid;
    const uint8_t* im = is_mem + (int64_t)b * is_mem_stride;
    // landmark bits of this tile, landmarks before it, first landmark after it
    {
      const unsigned lo = __ballot_sync(0xffffffffu, im[k0 + lane] != 0);
      const unsigned hi = __ballot_sync(0xffffffffu, im[k0 + 32 + lane] != 0);
      int c = 0;
      for (int j = tid; j < k0; j += 128) c += im[j] != 0;
      c = (int)warp_sum((float)c);
      if (lane == 0) sm->cnt[warp] = c;
      if (tid == 0) sm->mask = (uint64_t)lo | ((uint64_t)hi << 32);
      if (warp == 0) {
        int found = 0x7fffffff;
        for (int j0 = k0 + kKT; j0 < Lk && found == 0x7fffffff; j0 += 32) {
          const unsigned bal = __ballot_sync(0xffffffffu, j0 + lane < Lk && im[j0 + lane] != 0);
          if (bal) found = j0 + __ffs(bal) - 1;
        }
        if (lane == 0) sm->next_lm = found;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (tid == 0) sm->g0 = sm->cnt[0] + sm->cnt[1] + sm->cnt[2] + sm->cnt[3];
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const uint64_t mask = sm->mask;
    const int g0 = sm->g0, next_lm = sm->next_lm;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // position of the landmark that closes the group open at local key j (uniform)
    auto closing = [&](int from) {
      const uint64_t rest = from >= 64 ? 0ull : (mask >> from) << from;
      return rest ? k0 + (__ffsll((long long)rest) - 1) : next_lm;
    };
    // closing landmark of the e-th group that meets the tile (uniform), for the first four groups
    const int n_grp = __popcll(mask) + 1;
    int lm_of[4];
    {
      uint64_t rest = mask;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        lm_of[e] = rest ? k0 + (__ffsll((long long)rest) - 1) : next_lm;
        rest &= rest - 1;
      }
    }
    for (int i = 0; i < n_items; ++i) {
      const int sb = i & 1;
      const int tq = t_first + i;
      const int64_t grow = (int64_t)bh * Lq + tq * kQT + row;
      const int pos = prefix + tq * kQT + row;
      const float R = R_ptr[grow], delta = delta_ptr[grow];
      const int lim = pos - k0 >= 63 ? 63 : pos - k0;      // local keys 0..lim are visible (negative: none)
      const int own = pos - k0;                            // local index of the row's own key (may lie outside)
      const float* Arow = A_ptr + (int64_t)bh * G * Lq + tq * kQT + row;
      const float* Nrow = nD_ptr + (int64_t)bh * G * Lq + tq * kQT + row;
      // group g is closed for this row when its landmark lies before the row's position
      auto zof = [&](int gg, int lmpos, float& sub) {
        if (lmpos < pos && gg < G) {
          sub = Nrow[(int64_t)gg * Lq];
          return Arow[(int64_t)gg * Lq] + R;
        }
        sub = delta;
        return R;
      };
      // The statistics of the first four groups that meet this tile are fetched up front, all loads in flight at once
      // and overlapped with the wait for S / dP (a fetch at every group change would put a global-memory round trip
      // into the row walk each time); tiles with more groups fetch the rest on demand.
      float zq[4], sq[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        zq[e] = R;
        sq[e] = delta;
        if (e < n_grp) zq[e] = zof(g0 + e, lm_of[e], sq[e]);
      }
      int g = g0, gi = 0;
      int lmpos = lm_of[0];
      float sub = sq[0];
      float z = zq[0];
      mbar_wait(smem_u32(&sm->sdp_full[sb]), (i / 2) & 1, status, kErrMaskDkv + 2);
      tc_fence_after();
      // the P / dS tiles are free once the accumulating products of the previous item have read them
      if (i >= 1) mbar_wait(smem_u32(&sm->pds_free), (i - 1) & 1, status, kErrMaskDkv + 2);
      const uint32_t ts = tmem_s + sb * 64 + lane_base, td = tmem_dp + sb * 64 + lane_base;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float xv[16], dp[16];
        {
          uint32_t xr[16], dr[16];
          tmem_ld_32x32b_x16(ts + c * 16, xr);
          tmem_ld_32x32b_x16(td + c * 16, dr);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            xv[e] = __uint_as_float(xr[e]) * scale_log2;
            dp[e] = __uint_as_float(dr[e]);
          }
        }
        if (c == 3) {
          tc_fence_before();
          mbar_arrive(smem_u32(&sm->sdp_free[sb]));
        }
        const uint32_t m16 = (uint32_t)(mask >> (16 * c)) & 0xffffu;      // uniform
        const int j0 = 16 * c;
        uint32_t wp[8], wd[8];
        if (m16 == 0u) {
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float p0 = j0 + e <= lim ? ex2(xv[e] - z) : 0.f;
            const float p1 = j0 + e + 1 <= lim ? ex2(xv[e + 1] - z) : 0.f;
            wp[e / 2] = pack2<kBf16>(p0, p1);
            wd[e / 2] = pack2<kBf16>(p0 * (dp[e] - sub) * scale, p1 * (dp[e + 1] - sub) * scale);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            float p[2], d[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = j0 + e + h;
              if ((m16 >> (e + h)) & 1u) {
                p[h] = 0.f;
                d[h] = (j <= lim && j != own) ? ex2(xv[e + h] - R) * (sub - delta) * scale : 0.f;
                ++g;
                ++gi;
                if (gi < 4) {
                  z = gi == 1 ? zq[1] : (gi == 2 ? zq[2] : zq[3]);
                  sub = gi == 1 ? sq[1] : (gi == 2 ? sq[2] : sq[3]);
                } else {
                  lmpos = closing(j + 1);
                  z = zof(g, lmpos, sub);
                }
              } else {
                const float pj = j <= lim ? ex2(xv[e + h] - z) : 0.f;
                p[h] = pj;
                d[h] = pj * (dp[e + h] - sub) * scale;
              }
            }
            wp[e / 2] = pack2<kBf16>(p[0], p[1]);
            wd[e / 2] = pack2<kBf16>(d[0], d[1]);
          }
        }
        store_row16_sw128(p_tile, row, c, wp);
        store_row16_sw128(ds_tile, row, c, wd);
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&sm->pds_ready));
    }
    // epilogue: thread = feature d (TMEM lane), column = key -> dV[key][d], dK[key][d]
    if (n_items > 0) {
      mbar_wait(smem_u32(&sm->acc_full), 0, status, kErrMaskDkv + 3);
      tc_fence_after();
      uint32_t rv[2][32], rk[2][32];
      tmem_ld_32x32b_x32(tmem_dv + lane_base, rv[0]);
      tmem_ld_32x32b_x32(tmem_dv + 32 + lane_base, rv[1]);
      tmem_ld_32x32b_x32(tmem_dk + lane_base, rk[0]);
      tmem_ld_32x32b_x32(tmem_dk + 32 + lane_base, rk[1]);
      tmem_ld_wait();
      uint16_t* dvp = reinterpret_cast<uint16_t*>(dv_ptr) + ((int64_t)bh * Lk + k0) * kD + row;
      uint16_t* dkp = reinterpret_cast<uint16_t*>(dk_ptr) + ((int64_t)bh * Lk + k0) * kD + row;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          dvp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(rv[c][j]), 0.f) & 0xffffu);
          dkp[(int64_t)(c * 32 + j) * kD] = (uint16_t)(pack2<kBf16>(__uint_as_float(rk[c][j]), 0.f) & 0xffffu);
        }
    } else {
      // no query row sees this tile (only possible for tiles past the last query): zero gradients
      uint16_t* dvp = reinterpret_cast<uint16_t*>(dv_ptr) + ((int64_t)bh * Lk + k0) * kD + row;
      uint16_t* dkp = reinterpret_cast<uint16_t*>(dk_ptr) + ((int64_t)bh * Lk + k0) * kD + row;
      for (int j = 0; j < kKT; ++j) {
        dvp[(int64_t)j * kD] = 0;
        dkp[(int64_t)j * kD] = 0;
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
struct MaskFacts {
  bool ready = false;
};

int mask_kernel_attributes() {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static MaskFacts facts[kMaxDevices];
  int dev = 0;
  LMK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(LMK_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!facts[dev].ready) {
    const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_fwd_kernel<true>, attr, (int)mf_smem_bytes(kMaxGroups, kMaxKeyTiles)));
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_fwd_kernel<false>, attr, (int)mf_smem_bytes(kMaxGroups, kMaxKeyTiles)));
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_bwd_dq_kernel<true>, attr, (int)mq_smem_bytes(kMaxGroups)));
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_bwd_dq_kernel<false>, attr, (int)mq_smem_bytes(kMaxGroups)));
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_bwd_dkv_kernel<true>, attr, (int)kMkSmemBytes));
    LMK_CUDA(cudaFuncSetAttribute(sm100_mask_bwd_dkv_kernel<false>, attr, (int)kMkSmemBytes));
    facts[dev].ready = true;
  }
  return LMK_OK;
}

}  // namespace

bool attn_mask_sm100_supported(int B, int H, int Lq, int Lk, int D, int dtype) {
  return (dtype == LMK_BF16 || dtype == LMK_F16) && D == kD && Lq >= kQT && Lq % kQT == 0 && Lk % kKT == 0 &&
         Lk >= Lq && (Lk - Lq) % kKT == 0 && Lk <= kKT * kMaxKeyTiles && B >= 1 && H >= 1;
}

int attn_mask_sm100_max_groups() { return kMaxGroups; }

int attn_mask_sm100_fwd(const AttnParams& p, const uint8_t* is_mem, int64_t is_mem_stride, float* R, float* A, int G,
                        int dtype, cudaStream_t st) {
  if (!tensor_map_operand_ok(p.q, p.qs) || !tensor_map_operand_ok(p.k, p.ks) || !tensor_map_operand_ok(p.v, p.vs))
    return fail(LMK_ERR_UNSUPPORTED, "masked attention needs 16-byte aligned q/k/v with strides that are multiples of 8");
  if (G < 1 || G > kMaxGroups) return fail(LMK_ERR_UNSUPPORTED, "max_groups must be in 1..%d (got %d)", kMaxGroups, G);
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = tensor_map_4d(&tq, p.q, dtype, p.B, p.H, p.Lq, p.qs, kQT)) != LMK_OK) return rc;
  if ((rc = tensor_map_4d(&tk, p.k, dtype, p.B, p.H, p.Lk, p.ks, kKT)) != LMK_OK) return rc;
  if ((rc = tensor_map_4d(&tv, p.v, dtype, p.B, p.H, p.Lk, p.vs, kKT)) != LMK_OK) return rc;
  if ((rc = mask_kernel_attributes()) != LMK_OK) return rc;
  int* status = device_status_word();
  if (!status) return fail(LMK_ERR_CUDA, "cannot resolve the device status word");
  const float scale_log2 = p.scale * kLog2e;
  dim3 grid(p.B * p.H, p.Lq / kQT);
  const size_t smem = mf_smem_bytes(G, p.Lk / kKT);
  if (dtype == LMK_BF16)
    sm100_mask_fwd_kernel<true><<<grid, kMfThreads, smem, st>>>(tq, tk, tv, is_mem, is_mem_stride, p.o, R, A, p.H, p.Lq,
                                                                 p.Lk, G, scale_log2, status);
  else
    sm100_mask_fwd_kernel<false><<<grid, kMfThreads, smem, st>>>(tq, tk, tv, is_mem, is_mem_stride, p.o, R, A, p.H, p.Lq,
                                                                  p.Lk, G, scale_log2, status);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

size_t attn_mask_sm100_bwd_workspace(int B, int H, int Lq, int G) {
  return sizeof(float) * ((size_t)B * H * Lq + (size_t)B * H * G * Lq);      // delta, nD
}

int attn_mask_sm100_bwd(const AttnParams& p, const uint8_t* is_mem, int64_t is_mem_stride, const float* R,
                        const float* A, int G, int dtype, cudaStream_t st) {
  if (!tensor_map_operand_ok(p.q, p.qs) || !tensor_map_operand_ok(p.k, p.ks) || !tensor_map_operand_ok(p.v, p.vs) ||
      (uintptr_t)p.dO % 16 != 0 || (uintptr_t)p.o % 16 != 0)
    return fail(LMK_ERR_UNSUPPORTED, "masked attention needs 16-byte aligned tensors with strides that are multiples of 8");
  if (G < 1 || G > kMaxGroups) return fail(LMK_ERR_UNSUPPORTED, "max_groups must be in 1..%d (got %d)", kMaxGroups, G);
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  const int64_t dense[3] = {(int64_t)p.H * p.Lq * kD, (int64_t)p.Lq * kD, (int64_t)kD};
  if ((rc = tensor_map_4d(&tq, p.q, dtype, p.B, p.H, p.Lq, p.qs, kQT)) != LMK_OK) return rc;
  if ((rc = tensor_map_4d(&tk, p.k, dtype, p.B, p.H, p.Lk, p.ks, kKT)) != LMK_OK) return rc;
  if ((rc = tensor_map_4d(&tv, p.v, dtype, p.B, p.H, p.Lk, p.vs, kKT)) != LMK_OK) return rc;
  if ((rc = tensor_map_4d(&tdo, p.dO, dtype, p.B, p.H, p.Lq, dense, kQT)) != LMK_OK) return rc;
  if ((rc = mask_kernel_attributes()) != LMK_OK) return rc;
  int* status = device_status_word();
  if (!status) return fail(LMK_ERR_CUDA, "cannot resolve the device status word");
  float* delta = reinterpret_cast<float*>(p.workspace);
  float* nD = delta + (size_t)p.B * p.H * p.Lq;
  const float scale_log2 = p.scale * kLog2e;
  dim3 grid_q(p.B * p.H, p.Lq / kQT), grid_k(p.B * p.H, p.Lk / kKT);
  const size_t smem_q = mq_smem_bytes(G);
#define LMK_MASK_BWD(BF)                                                                                                \
  do {                                                                                                                  \
    sm100_mask_bwd_dq_kernel<BF><<<grid_q, kMqThreads, smem_q, st>>>(tq, tk, tv, tdo, is_mem, is_mem_stride, p.o, p.dO,  \
                                                                     R, A, delta, nD, p.dq, p.H, p.Lq, p.Lk, G,         \
                                                                     p.scale, scale_log2, status);                      \
    sm100_mask_bwd_dkv_kernel<BF><<<grid_k, kMkThreads, kMkSmemBytes, st>>>(tq, tk, tv, tdo, is_mem, is_mem_stride, R,  \
                                                                           A, delta, nD, p.dk, p.dv, p.H, p.Lq, p.Lk,   \
                                                                           G, p.scale, scale_log2, status);             \
  } while (0)
  if (dtype == LMK_BF16) LMK_MASK_BWD(true);
  else LMK_MASK_BWD(false);
#undef LMK_MASK_BWD
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

}  // namespace lmk
