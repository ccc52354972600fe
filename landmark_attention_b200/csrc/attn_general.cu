// General-path fused landmark attention: CUDA-core kernels with fp32 accumulation.
//
// These kernels cover every dtype (fp32 / fp16 / bf16), any head dim <= 128 that is a multiple of 32, any
// landmark block size in [2, 128], a key prefix (Lk > Lq) and, in the forward pass, a ragged last block.
// They are the path for fp32 inputs (where bf16 tensor-core products would miss the 1e-4 tolerance) and
// for shapes the tcgen05 kernels do not take.
//
// Math (same quantities as the reference Triton kernels, llama/ltriton/flash_landmark_attention.py):
//   query row at key position p, own block b = p / block.
//   earlier block n < b : l_n = s[block-1] (landmark score), st = softmax(s[0..block-2]) inside the block,
//                         outer online softmax over l_n; weight of key j = st_j * exp(l_n - m) / L      (:47-86)
//   own block n == b    : plain causal softmax terms exp(s_j - m) / L for j <= min(p - b*block, block-2) (:88-113)
// The accumulator is kept un-normalised and divided by L once at the end.
#include "common.cuh"
#include "attn_params.h"

namespace lmk {

namespace {

constexpr int kChunk = 32;          // keys staged in shared memory at a time
constexpr int kFwdWarps = 4;
constexpr int kRowsPerWarp = 4;
constexpr int kFwdRows = kFwdWarps * kRowsPerWarp;   // 16 query rows per CTA

template <typename T>
__device__ __forceinline__ void load_rows_f32(float* dst, int ld, const T* src, int64_t row_stride, int row0,
                                              int nrows, int row_limit, int D, int tid, int nthreads) {
  for (int i = tid; i < nrows * D; i += nthreads) {
    int r = i / D, d = i - r * D;
    int row = row0 + r;
    dst[r * ld + d] = row < row_limit ? to_f32(src[(int64_t)row * row_stride + d]) : 0.f;
  }
}

// dot products of one staged key row (lane = key) against kRowsPerWarp query rows
template <int R>
__device__ __forceinline__ void dot_rows(const float* __restrict__ krow, const float* __restrict__ qrows, int D,
                                         float (&s)[R]) {
#pragma unroll
  for (int r = 0; r < R; ++r) s[r] = 0.f;
  for (int d = 0; d < D; d += 4) {
    float k0 = krow[d], k1 = krow[d + 1], k2 = krow[d + 2], k3 = krow[d + 3];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float4 qv = *reinterpret_cast<const float4*>(qrows + r * D + d);
      s[r] = fmaf(qv.x, k0, s[r]);
      s[r] = fmaf(qv.y, k1, s[r]);
      s[r] = fmaf(qv.z, k2, s[r]);
      s[r] = fmaf(qv.w, k3, s[r]);
    }
  }
}

// ---------------------------------------------------------------------------------------------- forward
template <typename T>
__global__ void __launch_bounds__(kFwdWarps * 32) general_fwd_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, DP = D + 1, blk = p.block;
  const int blkpad = (blk + 31) & ~31;
  float* Qs = smem;                       // [16][D]
  float* KVs = Qs + kFwdRows * D;         // [32][D+1]
  float* Sb = KVs + kChunk * DP;          // [16][blkpad]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int q0 = blockIdx.x * kFwdRows;
  const int prefix = p.Lk - p.Lq;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];

  load_rows_f32(Qs, D, qp, p.qs[2], q0, kFwdRows, p.Lq, D, tid, blockDim.x);

  int own[kRowsPerWarp], vis[kRowsPerWarp];
  bool valid[kRowsPerWarp];
  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][4];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = q0 + warp * kRowsPerWarp + r;
    valid[r] = row < p.Lq;
    int pos = prefix + row;
    own[r] = pos / blk;
    int loc = pos - own[r] * blk;
    vis[r] = min(loc, blk - 2);
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[r][e] = 0.f;
  }
  const int last_row = min(q0 + kFwdRows, p.Lq) - 1;
  const int own_last = (prefix + last_row) / blk;
  const float* qrows = Qs + warp * kRowsPerWarp * D;
  float* srows = Sb + warp * kRowsPerWarp * blkpad;

  for (int n = 0; n <= own_last; ++n) {
    const int key0 = n * blk;
    const int nkeys = min(blk, p.Lk - key0);
    // pass A: scores of the whole block into shared memory
    for (int c0 = 0; c0 < nkeys; c0 += kChunk) {
      __syncthreads();
      load_rows_f32(KVs, DP, kp, p.ks[2], key0 + c0, kChunk, key0 + nkeys, D, tid, blockDim.x);
      __syncthreads();
      float s[kRowsPerWarp];
      dot_rows<kRowsPerWarp>(KVs + lane * DP, qrows, D, s);
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r)
        srows[r * blkpad + c0 + lane] = (c0 + lane < nkeys) ? s[r] * p.scale : -INFINITY;
    }
    __syncwarp();
    // per-row weights, written back in place
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float* sr = srows + r * blkpad;
      if (!valid[r] || n > own[r]) {
        for (int j = lane; j < blkpad; j += 32) sr[j] = 0.f;
      } else if (n < own[r]) {
        float lm = sr[blk - 1];
        float mx = -INFINITY;
        for (int j = lane; j < blk - 1; j += 32) mx = fmaxf(mx, sr[j]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int j = lane; j < blk - 1; j += 32) den += expf(sr[j] - mx);
        den = warp_sum(den);
        float m_new = fmaxf(m[r], lm);
        float sc = expf(m[r] - m_new);
        float el = expf(lm - m_new);
        l[r] = l[r] * sc + el;
        m[r] = m_new;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] *= sc;
        float w = el / den;
        __syncwarp();
        for (int j = lane; j < blkpad; j += 32) sr[j] = (j < blk - 1) ? expf(sr[j] - mx) * w : 0.f;
      } else {
        float mx = -INFINITY;
        for (int j = lane; j <= vis[r]; j += 32) mx = fmaxf(mx, sr[j]);
        mx = warp_max(mx);
        float m_new = fmaxf(m[r], mx);
        float sc = expf(m[r] - m_new);
        float sum = 0.f;
        __syncwarp();
        for (int j = lane; j < blkpad; j += 32) {
          float pj = (j <= vis[r]) ? expf(sr[j] - m_new) : 0.f;
          sr[j] = pj;
          sum += pj;
        }
        sum = warp_sum(sum);
        l[r] = l[r] * sc + sum;
        m[r] = m_new;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] *= sc;
      }
    }
    __syncwarp();
    // pass B: acc += P V
    for (int c0 = 0; c0 < nkeys; c0 += kChunk) {
      __syncthreads();
      load_rows_f32(KVs, DP, vp, p.vs[2], key0 + c0, kChunk, key0 + nkeys, D, tid, blockDim.x);
      __syncthreads();
      const int jn = min(kChunk, nkeys - c0);
      for (int j = 0; j < jn; ++j) {
        float vv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) vv[e] = (lane + 32 * e < D) ? KVs[j * DP + lane + 32 * e] : 0.f;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
          float pj = srows[r * blkpad + c0 + j];
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[r][e] = fmaf(pj, vv[e], acc[r][e]);
        }
      }
    }
  }

  T* op = reinterpret_cast<T*>(p.o) + ((int64_t)bh * p.Lq) * D;
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = q0 + warp * kRowsPerWarp + r;
    if (!valid[r]) continue;
    float inv = 1.f / l[r];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (lane + 32 * e < D) op[(int64_t)row * D + lane + 32 * e] = from_f32<T>(acc[r][e] * inv);
    if (lane == 0) {
      p.L[(int64_t)bh * p.Lq + row] = l[r];
      p.M[(int64_t)bh * p.Lq + row] = m[r];
    }
  }
}

// ---------------------------------------------------------------------------------------------- backward: dQ
// Same tiling as the forward kernel.  Also produces delta = rowsum(O * dO) for the dK/dV kernel.
template <typename T>
__global__ void __launch_bounds__(kFwdWarps * 32) general_bwd_dq_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, DP = D + 1, blk = p.block;
  const int blkpad = (blk + 31) & ~31;
  float* Qs = smem;                        // [16][D]
  float* dOs = Qs + kFwdRows * D;          // [16][D]
  float* Ks = dOs + kFwdRows * D;          // [32][D+1]
  float* Vs = Ks + kChunk * DP;            // [32][D+1]
  float* Sb = Vs + kChunk * DP;            // [16][blkpad]  scores, then dS
  float* Pb = Sb + kFwdRows * blkpad;      // [16][blkpad]  dP

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int q0 = blockIdx.x * kFwdRows;
  const int prefix = p.Lk - p.Lq;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const T* op = reinterpret_cast<const T*>(p.o) + ((int64_t)bh * p.Lq) * D;
  const T* dop = reinterpret_cast<const T*>(p.dO) + ((int64_t)bh * p.Lq) * D;

  load_rows_f32(Qs, D, qp, p.qs[2], q0, kFwdRows, p.Lq, D, tid, blockDim.x);
  load_rows_f32(dOs, D, dop, (int64_t)D, q0, kFwdRows, p.Lq, D, tid, blockDim.x);
  __syncthreads();

  int own[kRowsPerWarp], vis[kRowsPerWarp];
  bool valid[kRowsPerWarp];
  float Mr[kRowsPerWarp], Linv[kRowsPerWarp], delta[kRowsPerWarp], dq[kRowsPerWarp][4];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = q0 + warp * kRowsPerWarp + r;
    valid[r] = row < p.Lq;
    int pos = prefix + row;
    own[r] = pos / blk;
    vis[r] = min(pos - own[r] * blk, blk - 2);
    Mr[r] = valid[r] ? p.M[(int64_t)bh * p.Lq + row] : 0.f;
    Linv[r] = valid[r] ? 1.f / p.L[(int64_t)bh * p.Lq + row] : 0.f;
    float dsum = 0.f;
    if (valid[r])
      for (int d = lane; d < D; d += 32)
        dsum += to_f32(op[(int64_t)row * D + d]) * dOs[(warp * kRowsPerWarp + r) * D + d];
    delta[r] = warp_sum(dsum);
    if (valid[r] && lane == 0) p.delta[(int64_t)bh * p.Lq + row] = delta[r];
#pragma unroll
    for (int e = 0; e < 4; ++e) dq[r][e] = 0.f;
  }
  const int last_row = min(q0 + kFwdRows, p.Lq) - 1;
  const int own_last = (prefix + last_row) / blk;
  const float* qrows = Qs + warp * kRowsPerWarp * D;
  const float* dorows = dOs + warp * kRowsPerWarp * D;
  float* srows = Sb + warp * kRowsPerWarp * blkpad;
  float* prows = Pb + warp * kRowsPerWarp * blkpad;

  for (int n = 0; n <= own_last; ++n) {
    const int key0 = n * blk;
    for (int c0 = 0; c0 < blk; c0 += kChunk) {
      __syncthreads();
      load_rows_f32(Ks, DP, kp, p.ks[2], key0 + c0, kChunk, key0 + blk, D, tid, blockDim.x);
      load_rows_f32(Vs, DP, vp, p.vs[2], key0 + c0, kChunk, key0 + blk, D, tid, blockDim.x);
      __syncthreads();
      float s[kRowsPerWarp], dp[kRowsPerWarp];
      dot_rows<kRowsPerWarp>(Ks + lane * DP, qrows, D, s);
      dot_rows<kRowsPerWarp>(Vs + lane * DP, dorows, D, dp);
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        bool in = c0 + lane < blk;
        srows[r * blkpad + c0 + lane] = in ? s[r] * p.scale : -INFINITY;
        prows[r * blkpad + c0 + lane] = in ? dp[r] : 0.f;
      }
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float* sr = srows + r * blkpad;
      const float* pr = prows + r * blkpad;
      if (!valid[r] || n > own[r]) {
        for (int j = lane; j < blkpad; j += 32) sr[j] = 0.f;
      } else if (n < own[r]) {
        float lm = sr[blk - 1];
        float mx = -INFINITY;
        for (int j = lane; j < blk - 1; j += 32) mx = fmaxf(mx, sr[j]);
        mx = warp_max(mx);
        float den = 0.f, nD = 0.f;
        for (int j = lane; j < blk - 1; j += 32) {
          float e = expf(sr[j] - mx);
          den += e;
          nD += e * pr[j];
        }
        den = warp_sum(den);
        nD = warp_sum(nD) / den;
        float g = expf(lm - Mr[r]) * Linv[r];
        float w = g / den;
        __syncwarp();
        for (int j = lane; j < blkpad; j += 32) {
          float ds;
          if (j < blk - 1) ds = expf(sr[j] - mx) * w * (pr[j] - nD);
          else if (j == blk - 1) ds = g * (nD - delta[r]);
          else ds = 0.f;
          sr[j] = ds * p.scale;
        }
      } else {
        for (int j = lane; j < blkpad; j += 32) {
          float ds = 0.f;
          if (j <= vis[r]) ds = expf(sr[j] - Mr[r]) * Linv[r] * (pr[j] - delta[r]);
          sr[j] = ds * p.scale;
        }
      }
    }
    __syncwarp();
    for (int c0 = 0; c0 < blk; c0 += kChunk) {
      __syncthreads();
      load_rows_f32(Ks, DP, kp, p.ks[2], key0 + c0, kChunk, key0 + blk, D, tid, blockDim.x);
      __syncthreads();
      const int jn = min(kChunk, blk - c0);
      for (int j = 0; j < jn; ++j) {
        float kk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) kk[e] = (lane + 32 * e < D) ? Ks[j * DP + lane + 32 * e] : 0.f;
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
          float ds = srows[r * blkpad + c0 + j];
#pragma unroll
          for (int e = 0; e < 4; ++e) dq[r][e] = fmaf(ds, kk[e], dq[r][e]);
        }
      }
    }
  }
  T* dqp = reinterpret_cast<T*>(p.dq) + ((int64_t)bh * p.Lq) * D;
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = q0 + warp * kRowsPerWarp + r;
    if (!valid[r]) continue;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (lane + 32 * e < D) dqp[(int64_t)row * D + lane + 32 * e] = from_f32<T>(dq[r][e]);
  }
}

// ---------------------------------------------------------------------------------------------- backward: dK, dV
// One CTA per (key block, batch*head); 16 warps.  Phase 1 recomputes the weights of a tile of 32 query rows
// against the whole key block (lane = key); phase 2 accumulates dK/dV with each warp owning a slice of the keys
// (lane = feature), so no atomics are needed and the result is bit-reproducible.
constexpr int kDkvWarps = 16;
constexpr int kDkvRows = 32;
constexpr int kMaxKeysPerWarp = 8;   // block <= 128
constexpr int kMaxKeysPerLane = 4;   // block <= 128

template <typename T>
__global__ void __launch_bounds__(kDkvWarps * 32) general_bwd_dkv_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, DP = D + 1, blk = p.block;
  const int blkpad = (blk + 31) & ~31;
  float* Ks = smem;                         // [blk][D+1]
  float* Vs = Ks + blk * DP;                // [blk][D+1]
  float* Qs = Vs + blk * DP;                // [32][D]
  float* dOs = Qs + kDkvRows * D;           // [32][D]
  float* Pb = dOs + kDkvRows * D;           // [32][blkpad]
  float* dSb = Pb + kDkvRows * blkpad;      // [32][blkpad]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = blockIdx.x;
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int prefix = p.Lk - p.Lq;
  const int key0 = n * blk;
  const T* qp = reinterpret_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
  const T* kp = reinterpret_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
  const T* vp = reinterpret_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
  const T* dop = reinterpret_cast<const T*>(p.dO) + ((int64_t)bh * p.Lq) * D;

  load_rows_f32(Ks, DP, kp, p.ks[2], key0, blk, p.Lk, D, tid, blockDim.x);
  load_rows_f32(Vs, DP, vp, p.vs[2], key0, blk, p.Lk, D, tid, blockDim.x);

  const int kpw = (blk + kDkvWarps - 1) / kDkvWarps;
  const int kpl = blkpad / 32;
  float dk[kMaxKeysPerWarp][4], dv[kMaxKeysPerWarp][4];
#pragma unroll
  for (int i = 0; i < kMaxKeysPerWarp; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;

  const int r_start = max(0, key0 - prefix);
  for (int t0 = (r_start / kDkvRows) * kDkvRows; t0 < p.Lq; t0 += kDkvRows) {
    __syncthreads();
    load_rows_f32(Qs, D, qp, p.qs[2], t0, kDkvRows, p.Lq, D, tid, blockDim.x);
    load_rows_f32(dOs, D, dop, (int64_t)D, t0, kDkvRows, p.Lq, D, tid, blockDim.x);
    __syncthreads();
    // phase 1: two rows per warp
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int r = warp * 2 + rr;
      const int row = t0 + r;
      const int pos = prefix + row;
      const int own = pos / blk;
      float* prow = Pb + r * blkpad;
      float* dsrow = dSb + r * blkpad;
      if (row >= p.Lq || own < n) {
        for (int j = lane; j < blkpad; j += 32) prow[j] = dsrow[j] = 0.f;
        continue;
      }
      const float Mr = p.M[(int64_t)bh * p.Lq + row];
      const float Linv = 1.f / p.L[(int64_t)bh * p.Lq + row];
      const float delta = p.delta[(int64_t)bh * p.Lq + row];
      float s[kMaxKeysPerLane], dp[kMaxKeysPerLane];
#pragma unroll
      for (int c = 0; c < kMaxKeysPerLane; ++c) {
        s[c] = -INFINITY;
        dp[c] = 0.f;
        int j = lane + 32 * c;
        if (c < kpl && j < blk) {
          float a[1], bb[1];
          dot_rows<1>(Ks + j * DP, Qs + r * D, D, a);
          dot_rows<1>(Vs + j * DP, dOs + r * D, D, bb);
          s[c] = a[0] * p.scale;
          dp[c] = bb[0];
        }
      }
      if (own > n) {
        // landmark score lives in lane (blk-1)%32, slot (blk-1)/32
        const int lslot = (blk - 1) >> 5, llane = (blk - 1) & 31;
        float lm = 0.f;
#pragma unroll
        for (int c = 0; c < kMaxKeysPerLane; ++c)
          if (c == lslot) lm = __shfl_sync(0xffffffffu, s[c], llane);
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < kMaxKeysPerLane; ++c)
          if (lane + 32 * c < blk - 1) mx = fmaxf(mx, s[c]);
        mx = warp_max(mx);
        float e[kMaxKeysPerLane], den = 0.f, nD = 0.f;
#pragma unroll
        for (int c = 0; c < kMaxKeysPerLane; ++c) {
          e[c] = (lane + 32 * c < blk - 1) ? expf(s[c] - mx) : 0.f;
          den += e[c];
          nD += e[c] * dp[c];
        }
        den = warp_sum(den);
        nD = warp_sum(nD) / den;
        const float g = expf(lm - Mr) * Linv;
        const float w = g / den;
#pragma unroll
        for (int c = 0; c < kMaxKeysPerLane; ++c) {
          int j = lane + 32 * c;
          if (c < kpl) {
            float pj = e[c] * w;
            float ds = pj * (dp[c] - nD);
            if (j == blk - 1) ds = g * (nD - delta);
            if (j >= blk) ds = 0.f;
            prow[j] = pj;
            dsrow[j] = ds * p.scale;
          }
        }
      } else {
        const int vis = min(pos - own * blk, blk - 2);
#pragma unroll
        for (int c = 0; c < kMaxKeysPerLane; ++c) {
          int j = lane + 32 * c;
          if (c < kpl) {
            float pj = (j <= vis) ? expf(s[c] - Mr) * Linv : 0.f;
            prow[j] = pj;
            dsrow[j] = pj * (dp[c] - delta) * p.scale;
          }
        }
      }
    }
    __syncthreads();
    // phase 2
    for (int r = 0; r < kDkvRows; ++r) {
      float qv[4], dov[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qv[e] = (lane + 32 * e < D) ? Qs[r * D + lane + 32 * e] : 0.f;
        dov[e] = (lane + 32 * e < D) ? dOs[r * D + lane + 32 * e] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < kMaxKeysPerWarp; ++i) {
        int j = warp * kpw + i;
        if (i < kpw && j < blk) {
          float pj = Pb[r * blkpad + j], ds = dSb[r * blkpad + j];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            dv[i][e] = fmaf(pj, dov[e], dv[i][e]);
            dk[i][e] = fmaf(ds, qv[e], dk[i][e]);
          }
        }
      }
    }
  }
  T* dkp = reinterpret_cast<T*>(p.dk) + ((int64_t)bh * p.Lk) * D;
  T* dvp = reinterpret_cast<T*>(p.dv) + ((int64_t)bh * p.Lk) * D;
#pragma unroll
  for (int i = 0; i < kMaxKeysPerWarp; ++i) {
    int j = warp * kpw + i;
    if (i < kpw && j < blk) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (lane + 32 * e < D) {
          dkp[(int64_t)(key0 + j) * D + lane + 32 * e] = from_f32<T>(dk[i][e]);
          dvp[(int64_t)(key0 + j) * D + lane + 32 * e] = from_f32<T>(dv[i][e]);
        }
    }
  }
}

template <typename T>
int launch_fwd(const AttnParams& p, cudaStream_t st) {
  const int blkpad = (p.block + 31) & ~31;
  size_t smem = sizeof(float) * ((size_t)kFwdRows * p.D + (size_t)kChunk * (p.D + 1) + (size_t)kFwdRows * blkpad);
  LMK_CUDA(cudaFuncSetAttribute(general_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((p.Lq + kFwdRows - 1) / kFwdRows, p.B * p.H);
  general_fwd_kernel<T><<<grid, kFwdWarps * 32, smem, st>>>(p);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

template <typename T>
int launch_bwd(const AttnParams& p, cudaStream_t st) {
  const int blkpad = (p.block + 31) & ~31;
  size_t smem1 = sizeof(float) * ((size_t)2 * kFwdRows * p.D + (size_t)2 * kChunk * (p.D + 1) +
                                  (size_t)2 * kFwdRows * blkpad);
  LMK_CUDA(cudaFuncSetAttribute(general_bwd_dq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
  dim3 grid1((p.Lq + kFwdRows - 1) / kFwdRows, p.B * p.H);
  general_bwd_dq_kernel<T><<<grid1, kFwdWarps * 32, smem1, st>>>(p);
  LMK_CUDA(cudaGetLastError());
  size_t smem2 = sizeof(float) * ((size_t)2 * p.block * (p.D + 1) + (size_t)2 * kDkvRows * p.D +
                                  (size_t)2 * kDkvRows * blkpad);
  LMK_CUDA(cudaFuncSetAttribute(general_bwd_dkv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2));
  dim3 grid2(p.Lk / p.block, p.B * p.H);
  general_bwd_dkv_kernel<T><<<grid2, kDkvWarps * 32, smem2, st>>>(p);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

}  // namespace

int attn_general_fwd(const AttnParams& p, int dtype, cudaStream_t st) {
  switch (dtype) {
    case LMK_F32: return launch_fwd<float>(p, st);
    case LMK_F16: return launch_fwd<__half>(p, st);
    default: return launch_fwd<__nv_bfloat16>(p, st);
  }
}

int attn_general_bwd(const AttnParams& p, int dtype, cudaStream_t st) {
  switch (dtype) {
    case LMK_F32: return launch_bwd<float>(p, st);
    case LMK_F16: return launch_bwd<__half>(p, st);
    default: return launch_bwd<__nv_bfloat16>(p, st);
  }
}

size_t attn_general_bwd_workspace(int B, int H, int Lq) { return sizeof(float) * (size_t)B * H * Lq; }

}  // namespace lmk
