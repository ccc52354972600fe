// Inference-time landmark retrieval: landmark scores, per-row top-k, and the gather of the selected KV blocks.
//
// Reference call sites: LlamaAttention.forward cache branch (llama/llama_mem.py:357-398, 408-410) and
// MemLMCacheStorage.retrieve_for_query (lm_benchmark/models/caches/mem_cache.py:51-98).  Both rotate cached keys at
// "slot" positions: the newest top_k blocks occupy slots 1..top_k, every older block shares slot 0.
#include <type_traits>
#include "common.cuh"
#include "scores_sm100.h"

namespace lmk {
namespace {

__host__ __device__ __forceinline__ int logical_age(int phys, int ring_start, int n) {
  int l = phys - ring_start;
  return l < 0 ? l + n : l;
}
// slot of a block given its logical age index (0 = oldest)
__host__ __device__ __forceinline__ int slot_of(int logical, int n, int top_k) {
  int first_recent = n - top_k;
  return logical >= first_recent ? logical - first_recent + 1 : 0;
}

// One rotary output element computed the way torch computes `x*cos + rotate_half(x)*sin` in dtype T:
// each product and the sum are rounded to T (no fused multiply-add).
template <typename T>
__device__ __forceinline__ float rotary_elem(float x, float partner_signed, float c, float s) {
  float a = to_f32(from_f32<T>(__fmul_rn(x, c)));
  float b = to_f32(from_f32<T>(__fmul_rn(partner_signed, s)));
  return to_f32(from_f32<T>(__fadd_rn(a, b)));
}

// Two rotary outputs at once with the same rounding steps; 16-bit types use the packed float2 -> x2 conversions, which
// halves the work on the conversion pipe (the gather kernel is otherwise limited by it, not by HBM).
template <typename T>
__device__ __forceinline__ void rotary_pair(float x0, float x1, float p0, float p1, float c0, float c1, float s0,
                                            float s1, T& o0, T& o1) {
  o0 = from_f32<T>(rotary_elem<T>(x0, p0, c0, s0));
  o1 = from_f32<T>(rotary_elem<T>(x1, p1, c1, s1));
}
template <>
__device__ __forceinline__ void rotary_pair<__nv_bfloat16>(float x0, float x1, float p0, float p1, float c0, float c1,
                                                           float s0, float s1, __nv_bfloat16& o0, __nv_bfloat16& o1) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(__fmul_rn(x0, c0), __fmul_rn(x1, c1));
  const __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(p0, s0), __fmul_rn(p1, s1));
  const __nv_bfloat162 r = __floats2bfloat162_rn(__fadd_rn(__low2float(a), __low2float(b)),
                                                 __fadd_rn(__high2float(a), __high2float(b)));
  o0 = __low2bfloat16(r);
  o1 = __high2bfloat16(r);
}
template <>
__device__ __forceinline__ void rotary_pair<__half>(float x0, float x1, float p0, float p1, float c0, float c1, float s0,
                                                    float s1, __half& o0, __half& o1) {
  const __half2 a = __floats2half2_rn(__fmul_rn(x0, c0), __fmul_rn(x1, c1));
  const __half2 b = __floats2half2_rn(__fmul_rn(p0, s0), __fmul_rn(p1, s1));
  const __half2 r = __floats2half2_rn(__fadd_rn(__low2float(a), __low2float(b)),
                                      __fadd_rn(__high2float(a), __high2float(b)));
  o0 = __low2half(r);
  o1 = __high2half(r);
}

// ------------------------------------------------------------------------------------------- landmark scores
constexpr int kScTile = 32;

template <typename T>
__global__ void __launch_bounds__(128) landmark_scores_kernel(const T* __restrict__ q, const T* __restrict__ kc,
                                                              lmk_cache_desc desc, const T* __restrict__ cos_t,
                                                              const T* __restrict__ sin_t, int n_pos, int rotary,
                                                              float* __restrict__ scores, int H, int Tq, int D,
                                                              float scale) {
  extern __shared__ __align__(16) float sc_smem[];
  const int DP = D + 1;
  float* Qs = sc_smem;               // [32][D]
  float* Ks = Qs + kScTile * D;      // [32][D+1], rotated landmark keys
  const int tid = threadIdx.x, lane = tid & 31, ty = tid >> 5;
  const int n0 = blockIdx.x * kScTile, t0 = blockIdx.y * kScTile;
  const int bh = blockIdx.z, b = bh / H, h = bh - b * H;
  const int N = desc.n_blocks, blk = desc.block;
  const T* qp = q + ((int64_t)bh * Tq) * D;
  for (int i = tid; i < kScTile * D; i += 128) {
    int r = i / D, d = i - r * D;
    Qs[i] = (t0 + r < Tq) ? to_f32(qp[(int64_t)(t0 + r) * D + d]) : 0.f;
  }
  for (int i = tid; i < kScTile * D; i += 128) {
    int r = i / D, d = i - r * D;
    int n = n0 + r;
    float val = 0.f;
    if (n < N) {
      const T* row = kc + b * desc.stride_b + h * desc.stride_h + (int64_t)n * desc.stride_block +
                     (int64_t)(blk - 1) * desc.stride_row;
      float x = to_f32(row[d]);
      if (rotary == LMK_ROTARY_NONE) {
        val = x;
      } else {
        int slot = slot_of(logical_age(n, desc.ring_start, N), N, desc.top_k);
        int pos = desc.pos_base + slot * blk + blk - 1;
        pos = max(0, min(pos, n_pos - 1));
        float c = to_f32(cos_t[(int64_t)pos * D + d]), s = to_f32(sin_t[(int64_t)pos * D + d]);
        float partner;
        if (rotary == LMK_ROTARY_HALF) partner = d < D / 2 ? -to_f32(row[d + D / 2]) : to_f32(row[d - D / 2]);
        else partner = (d & 1) ? to_f32(row[d - 1]) : -to_f32(row[d + 1]);
        val = rotary_elem<T>(x, partner, c, s);
      }
    }
    Ks[r * DP + d] = val;
  }
  __syncthreads();
  // thread: landmark n0+lane, tokens t0 + ty*8 .. +7
  float acc[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) acc[r] = 0.f;
  const float* krow = Ks + lane * DP;
  const float* qrows = Qs + ty * 8 * D;
  for (int d = 0; d < D; d += 4) {
    float k0 = krow[d], k1 = krow[d + 1], k2 = krow[d + 2], k3 = krow[d + 3];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      float4 qv = *reinterpret_cast<const float4*>(qrows + r * D + d);
      acc[r] = fmaf(qv.x, k0, acc[r]);
      acc[r] = fmaf(qv.y, k1, acc[r]);
      acc[r] = fmaf(qv.z, k2, acc[r]);
      acc[r] = fmaf(qv.w, k3, acc[r]);
    }
  }
  const int n = n0 + lane;
  if (n < N) {
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      int t = t0 + ty * 8 + r;
      if (t < Tq) {
        // 16-bit inputs: the reference's matmul output and the scaling are each rounded to the input dtype
        float v = to_f32(from_f32<T>(acc[r]));
        v = to_f32(from_f32<T>(v * scale));
        scores[((int64_t)bh * Tq + t) * N + n] = v;
      }
    }
  }
}

// in-place softmax over the last dim, one warp per row, result rounded to T
template <typename T>
__global__ void __launch_bounds__(128) row_softmax_kernel(float* __restrict__ s, int64_t rows, int n) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float* r = s + row * n;
  float mx = -INFINITY;
  for (int j = lane; j < n; j += 32) mx = fmaxf(mx, r[j]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < n; j += 32) sum += expf(r[j] - mx);
  sum = warp_sum(sum);
  for (int j = lane; j < n; j += 32) r[j] = to_f32(from_f32<T>(expf(r[j] - mx) / sum));
}

// ------------------------------------------------------------------------------------------- top-k
constexpr int kTopkMaxK = 32;

// k rounds of warp arg-max over vals[0..n) in shared memory (ties: lower index), then the picks are written in
// ascending order of logical age.  Called by one full warp.
__device__ __forceinline__ void select_topk_sorted(float* vals, int n, int k, int ring_start, bool vec4,
                                                   int32_t* __restrict__ out_row) {
  const int lane = threadIdx.x & 31;
  int mine = -1;   // lane i keeps the i-th pick
  for (int it = 0; it < k; ++it) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    auto consider = [&](float v, int j) {
      if (v > best || (v == best && j < bi)) {
        best = v;
        bi = j;
      }
    };
    if (vec4) {
      const float4* vals4 = reinterpret_cast<const float4*>(vals);
      for (int j = lane; j < n / 4; j += 32) {
        const float4 v = vals4[j];
        consider(v.x, 4 * j);
        consider(v.y, 4 * j + 1);
        consider(v.z, 4 * j + 2);
        consider(v.w, 4 * j + 3);
      }
    } else {
      for (int j = lane; j < n; j += 32) consider(vals[j], j);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == it) mine = bi;
    if (lane == 0) vals[bi] = __int_as_float(0x7fc00000);   // NaN marks a taken slot: it never compares true
    __syncwarp();
  }
  // ascending order by logical age: rank = number of picks with a smaller age
  int age = (lane < k) ? logical_age(mine, ring_start, n) : 0x7fffffff;
  int rank = 0;
  for (int u = 0; u < k; ++u) {
    int a = __shfl_sync(0xffffffffu, age, u);
    rank += (a < age) ? 1 : 0;
  }
  if (lane < k) out_row[rank] = mine;
}

__global__ void __launch_bounds__(128) topk_sorted_kernel(const float* __restrict__ scores, int32_t* __restrict__ idx,
                                                          int64_t rows, int64_t inner_count, int64_t outer_stride,
                                                          int64_t inner_stride, int reduce, int64_t reduce_stride,
                                                          int n, int k, int ring_start, int warps_per_cta) {
  extern __shared__ __align__(16) float tk_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * warps_per_cta + warp;
  if (warp >= warps_per_cta || row >= rows) return;
  float* vals = tk_smem + (size_t)warp * n;
  const int64_t outer = row / inner_count, inner = row - outer * inner_count;
  const float* src = scores + outer * outer_stride + inner * inner_stride;
  // rows of whole, 16-byte aligned float4 groups are moved and scanned four values at a time (several loads in flight
  // per lane; the scalar loop is latency-bound on a cold row)
  const bool vec4 = reduce == 1 && (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | (uintptr_t)(n * sizeof(float))) & 15) == 0;
  if (vec4) {
    const float4* src4 = reinterpret_cast<const float4*>(src);
    float4* vals4 = reinterpret_cast<float4*>(vals);
#pragma unroll 8
    for (int j = lane; j < n / 4; j += 32) {
      float4 v = src4[j];
      v.x = (v.x != v.x) ? -INFINITY : v.x;   // NaN scores rank lowest
      v.y = (v.y != v.y) ? -INFINITY : v.y;
      v.z = (v.z != v.z) ? -INFINITY : v.z;
      v.w = (v.w != v.w) ? -INFINITY : v.w;
      vals4[j] = v;
    }
  } else {
    for (int j = lane; j < n; j += 32) {
      float v = src[j];
      for (int r = 1; r < reduce; ++r) v = fmaxf(v, src[(int64_t)r * reduce_stride + j]);
      vals[j] = (v != v) ? -INFINITY : v;
    }
  }
  __syncwarp();
  select_topk_sorted(vals, n, k, ring_start, vec4, idx + row * k);
}

// Rows of at most 1024 scores (whole float4 groups, 16-byte aligned): the row stays in registers, 32 values per lane.
// A lower bound T of the k-th largest score comes from the lanes' maxima (the k largest lane maxima are k different
// scores, so the k-th of them cannot exceed the k-th largest score); every score >= T becomes a candidate in shared
// memory -- a handful -- and the k rounds of arg-max (value, then lower index: the same order as select_topk_sorted)
// run over the candidates only.  Rows with too many candidates (long runs of equal scores) take the general selection.
constexpr int kTopkRegCand = 64;

__global__ void __launch_bounds__(128, 8) topk_sorted_rows_kernel(const float* __restrict__ scores,
                                                               int32_t* __restrict__ idx, int64_t rows,
                                                               int64_t inner_count, int64_t outer_stride,
                                                               int64_t inner_stride, int n, int k, int ring_start) {
  extern __shared__ __align__(16) float tk_smem[];          // per warp: n floats (general selection) + candidates
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  float* vals = tk_smem + (size_t)warp * (n + 2 * kTopkRegCand);
  float* cand_v = vals + n;
  int* cand_i = reinterpret_cast<int*>(cand_v + kTopkRegCand);
  const int64_t outer = row / inner_count, inner = row - outer * inner_count;
  const float4* src4 = reinterpret_cast<const float4*>(scores + outer * outer_stride + inner * inner_stride);
  const int n4 = n >> 2;
  float v[32];
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int j = lane + 32 * m;
    float4 f = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    if (j < n4) f = src4[j];
    v[4 * m] = (f.x != f.x) ? -INFINITY : f.x;              // NaN scores rank lowest
    v[4 * m + 1] = (f.y != f.y) ? -INFINITY : f.y;
    v[4 * m + 2] = (f.z != f.z) ? -INFINITY : f.z;
    v[4 * m + 3] = (f.w != f.w) ? -INFINITY : f.w;
  }
  float cur = v[0];
#pragma unroll
  for (int e = 1; e < 32; ++e) cur = fmaxf(cur, v[e]);
  float T = -INFINITY;
  for (int it = 0; it < k; ++it) {                          // k-th largest of the 32 lane maxima
    T = warp_max(cur);
    const unsigned holders = __ballot_sync(0xffffffffu, cur == T);
    if (lane == __ffs(holders) - 1) cur = -INFINITY;
  }
  int cnt = 0;
#pragma unroll
  for (int e = 0; e < 32; ++e) cnt += (v[e] >= T && (lane + 32 * (e >> 2)) < n4) ? 1 : 0;
  int inc = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += u;
  }
  const int total = __shfl_sync(0xffffffffu, inc, 31);
  if (total > kTopkRegCand) {                               // uniform: the general selection on the staged row
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const int j = lane + 32 * m;
      if (j < n4) reinterpret_cast<float4*>(vals)[j] = make_float4(v[4 * m], v[4 * m + 1], v[4 * m + 2], v[4 * m + 3]);
    }
    __syncwarp();
    select_topk_sorted(vals, n, k, ring_start, true, idx + row * k);
    return;
  }
  int off = inc - cnt;
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    const int j = lane + 32 * (e >> 2);
    if (v[e] >= T && j < n4) {
      cand_v[off] = v[e];
      cand_i[off] = 4 * j + (e & 3);
      ++off;
    }
  }
  __syncwarp();
  // two candidates per lane at most; k rounds of arg-max, ties to the lower index
  float c0 = lane < total ? cand_v[lane] : -INFINITY, c1 = lane + 32 < total ? cand_v[lane + 32] : -INFINITY;
  int i0 = lane < total ? cand_i[lane] : 0x7fffffff, i1 = lane + 32 < total ? cand_i[lane + 32] : 0x7fffffff;
  int mine = -1;
  for (int it = 0; it < k; ++it) {
    float best = c0;
    int bi = i0;
    if (i1 != 0x7fffffff && (i0 == 0x7fffffff || c1 > best || (c1 == best && i1 < bi))) {
      best = c1;
      bi = i1;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == it) mine = bi;
    if (i0 == bi) i0 = 0x7fffffff;                          // taken
    if (i1 == bi) i1 = 0x7fffffff;
  }
  int age = (lane < k) ? logical_age(mine, ring_start, n) : 0x7fffffff;
  int rank = 0;
  for (int u = 0; u < k; ++u) {
    const int a = __shfl_sync(0xffffffffu, age, u);
    rank += (a < age) ? 1 : 0;
  }
  if (lane < k) idx[row * k + rank] = mine;
}

// The aggregated selection modes (maximum over `reduce` score rows first): one CTA of 1024 threads per output row.
// Few rows exist in these modes (batch * heads, or batch * tokens), so each CTA must pull its share of the scores at
// several hundred GB/s on its own: 16-byte loads, the reduce range split over `parts` thread groups with four
// independent chains each, partial maxima combined through shared memory, then the first warp selects.
__global__ void __launch_bounds__(1024) topk_reduce_sorted_kernel(const float* __restrict__ scores,
                                                                  int32_t* __restrict__ idx, int64_t inner_count,
                                                                  int64_t outer_stride, int64_t inner_stride,
                                                                  int reduce, int64_t reduce_stride, int n, int k,
                                                                  int ring_start, int vec4, int parts) {
  extern __shared__ __align__(16) float tk_smem[];      // [parts][n] partial maxima; row 0 becomes the result
  const int64_t row = blockIdx.x;
  const int64_t outer = row / inner_count, inner = row - outer * inner_count;
  const float* src = scores + outer * outer_stride + inner * inner_stride;
  const float ninf = -INFINITY;
  if (vec4) {
    const int cgs = n / 4;                               // column groups of four
    const int per = (int)blockDim.x / parts;             // threads per part
    const int part = threadIdx.x / per, t0 = threadIdx.x - part * per;
    if (part < parts) {
      for (int cg = t0; cg < cgs; cg += per) {
        float4 m[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) m[c] = make_float4(ninf, ninf, ninf, ninf);
        int r = part;
        for (; r + 3 * parts < reduce; r += 4 * parts) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)(r + c * parts) * reduce_stride + 4 * cg);
            m[c].x = fmaxf(m[c].x, v.x);
            m[c].y = fmaxf(m[c].y, v.y);
            m[c].z = fmaxf(m[c].z, v.z);
            m[c].w = fmaxf(m[c].w, v.w);
          }
        }
        for (; r < reduce; r += parts) {
          const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)r * reduce_stride + 4 * cg);
          m[0].x = fmaxf(m[0].x, v.x);
          m[0].y = fmaxf(m[0].y, v.y);
          m[0].z = fmaxf(m[0].z, v.z);
          m[0].w = fmaxf(m[0].w, v.w);
        }
        float4 o;                                        // fmaxf drops NaNs: a NaN score ranks lowest
        o.x = fmaxf(fmaxf(m[0].x, m[1].x), fmaxf(m[2].x, m[3].x));
        o.y = fmaxf(fmaxf(m[0].y, m[1].y), fmaxf(m[2].y, m[3].y));
        o.z = fmaxf(fmaxf(m[0].z, m[1].z), fmaxf(m[2].z, m[3].z));
        o.w = fmaxf(fmaxf(m[0].w, m[1].w), fmaxf(m[2].w, m[3].w));
        reinterpret_cast<float4*>(tk_smem + (size_t)part * n)[cg] = o;
      }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      float v = tk_smem[j];
      for (int p = 1; p < parts; ++p) v = fmaxf(v, tk_smem[(size_t)p * n + j]);
      tk_smem[j] = v;
    }
  } else {
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      float v = ninf;
      for (int r = 0; r < reduce; ++r) v = fmaxf(v, src[(int64_t)r * reduce_stride + j]);
      tk_smem[j] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) select_topk_sorted(tk_smem, n, k, ring_start, false, idx + row * k);
}

// ------------------------------------------------------------------------------------------- gather
// One CTA per (selected block i, token t, batch*head): copies block*D elements of K (rotated) and V with 16-byte
// vector accesses.
template <typename T>
__global__ void __launch_bounds__(128) gather_kv_kernel(const T* __restrict__ kc, const T* __restrict__ vc,
                                                        lmk_cache_desc kd, lmk_cache_desc vd,
                                                        const int32_t* __restrict__ idx, const T* __restrict__ cos_t,
                                                        const T* __restrict__ sin_t, int n_pos, int rotary,
                                                        T* __restrict__ k_out, T* __restrict__ v_out, int H, int Tq,
                                                        int D) {
  constexpr int VEC = 16 / sizeof(T);
  struct __align__(16) Vec { T v[VEC]; };
  const int i = blockIdx.x, t = blockIdx.y, bh = blockIdx.z;
  const int b = bh / H, h = bh - b * H;
  const int blk = kd.block, N = kd.n_blocks, top_k = kd.top_k;
  const int sel = idx[((int64_t)bh * Tq + t) * top_k + i];
  const bool recent = logical_age(sel, kd.ring_start, N) >= N - top_k;
  const int pos0 = kd.pos_base + (i + (recent ? 1 : 0)) * blk;
  const int vec_per_row = D / VEC;
  const int64_t out_base = (((int64_t)bh * Tq + t) * top_k + i) * blk * D;
  const T* ksrc = kc + b * kd.stride_b + h * kd.stride_h + (int64_t)sel * kd.stride_block;
  const T* vsrc = vc ? vc + b * vd.stride_b + h * vd.stride_h + (int64_t)sel * vd.stride_block : nullptr;
  for (int e = threadIdx.x; e < blk * vec_per_row; e += blockDim.x) {
    const int r = e / vec_per_row, d0 = (e - r * vec_per_row) * VEC;
    if (v_out != nullptr && vsrc != nullptr) {
      Vec vv = *reinterpret_cast<const Vec*>(vsrc + (int64_t)r * vd.stride_row + d0);
      *reinterpret_cast<Vec*>(v_out + out_base + (int64_t)r * D + d0) = vv;
    }
    if (k_out != nullptr) {
      const T* krow = ksrc + (int64_t)r * kd.stride_row;
      Vec x = *reinterpret_cast<const Vec*>(krow + d0);
      Vec o = x;
      if (rotary != LMK_ROTARY_NONE) {
        int pos = max(0, min(pos0 + r, n_pos - 1));
        Vec c = *reinterpret_cast<const Vec*>(cos_t + (int64_t)pos * D + d0);
        Vec s = *reinterpret_cast<const Vec*>(sin_t + (int64_t)pos * D + d0);
        if (rotary == LMK_ROTARY_HALF) {
          const bool lo = d0 < D / 2;
          Vec y = *reinterpret_cast<const Vec*>(krow + (lo ? d0 + D / 2 : d0 - D / 2));
#pragma unroll
          for (int u = 0; u < VEC; u += 2) {
            const float p0 = lo ? -to_f32(y.v[u]) : to_f32(y.v[u]);
            const float p1 = lo ? -to_f32(y.v[u + 1]) : to_f32(y.v[u + 1]);
            rotary_pair<T>(to_f32(x.v[u]), to_f32(x.v[u + 1]), p0, p1, to_f32(c.v[u]), to_f32(c.v[u + 1]),
                           to_f32(s.v[u]), to_f32(s.v[u + 1]), o.v[u], o.v[u + 1]);
          }
        } else {
#pragma unroll
          for (int u = 0; u < VEC; u += 2)
            rotary_pair<T>(to_f32(x.v[u]), to_f32(x.v[u + 1]), -to_f32(x.v[u + 1]), to_f32(x.v[u]), to_f32(c.v[u]),
                           to_f32(c.v[u + 1]), to_f32(s.v[u]), to_f32(s.v[u + 1]), o.v[u], o.v[u + 1]);
        }
      }
      *reinterpret_cast<Vec*>(k_out + out_base + (int64_t)r * D + d0) = o;
    }
  }
}

// ------------------------------------------------------------------------------------------- selected-block attention
// The two halves of attention over the selected blocks WITHOUT materialising the gather: logits of a query against
// the keys of its selected blocks (rotated at their slot positions, with the rounding steps of the gather kernel), and
// the probability-weighted sum of the selected value rows.  Blocks are read in place from the cache, so a block
// selected by many tokens of a head is served from L2 and nothing of size [B,H,T,top_k*block,D] is ever written.
//
// One CTA per (token t, batch*head); warp w takes selected blocks w, w+4, ...; every load instruction covers whole
// rows (coalesced) and the partial dot products of a row are combined with shuffles.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec_f32(const T* p, float (&o)[VEC]) {
  struct __align__(16) Vec { T v[VEC]; };
  const Vec x = *reinterpret_cast<const Vec*>(p);
#pragma unroll
  for (int u = 0; u < VEC; ++u) o[u] = to_f32(x.v[u]);
}

// 16-bit types: the rotation x * cos + p * sin runs on packed pairs with the rounding steps of the gather kernel
// (each product and the sum rounded to the 16-bit type, as the reference's tensor arithmetic does), which takes a
// third of the instructions of converting everything to fp32 first; the dot product accumulates in fp32.
// Tuning of the selected-block kernels, from sweeps on a B200 at the long-context retrieval shape: the logits kernel
// wants occupancy (8 CTAs per SM, i.e. <= 64 registers, even at the price of a small spill) rather than unrolling, and
// the value-sum kernel is insensitive to its unroll factor.
constexpr int kSelMinBlocks = 8;
constexpr int kSelUnroll = 1;
constexpr int kPvUnroll = 4;
template <typename T> struct Packed;      // arithmetic on two 16-bit values held in one 32-bit register
template <> struct Packed<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ void to_f32(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
};
template <> struct Packed<__half> {
  static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  static __device__ __forceinline__ void to_f32(uint32_t w, float& lo, float& hi) {
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(w));
  }
};
template <> struct Packed<float> {};
__device__ __forceinline__ void ld16(const void* p, uint32_t (&w)[4]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}

// This lane's share of q . rot(k_row): `krow` points at the lane's 16-byte vector of the low half of the row (its partner
// vector of the high half is HALF elements further), cr / sr at the same vectors of the cos / sin rows of the key's position.
// 16-bit types rotate on packed pairs with the rounding steps of the gather kernel; the dot product accumulates in fp32.
template <typename T, int VEC>
__device__ __forceinline__ float rotated_row_dot(const T* krow, const T* cr, const T* sr, int HALF, int rotary,
                                                 const float (&q0)[VEC], const float (&q1)[VEC]) {
  float acc0 = 0.f, acc1 = 0.f;
    if constexpr (sizeof(T) == 2) {
      uint32_t xl[4], xh[4];
      ld16(krow, xl);
      ld16(krow + HALF, xh);
      if (rotary != LMK_ROTARY_NONE) {
        uint32_t cl[4], ch[4], sl[4], sh[4], pl[4], ph[4];
        ld16(cr, cl);
        ld16(cr + HALF, ch);
        ld16(sr, sl);
        ld16(sr + HALF, sh);
        if (rotary == LMK_ROTARY_HALF) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {        // rotate_half: (-x[d + D/2], x[d])
            pl[u] = xh[u] ^ 0x80008000u;
            ph[u] = xl[u];
          }
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) {        // interleaved pairs: (x0, x1) -> (-x1, x0)
            pl[u] = __byte_perm(xl[u], xl[u], 0x1032) ^ 0x00008000u;
            ph[u] = __byte_perm(xh[u], xh[u], 0x1032) ^ 0x00008000u;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          xl[u] = Packed<T>::add(Packed<T>::mul(xl[u], cl[u]), Packed<T>::mul(pl[u], sl[u]));
          xh[u] = Packed<T>::add(Packed<T>::mul(xh[u], ch[u]), Packed<T>::mul(ph[u], sh[u]));
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f0, f1, g0, g1;
        Packed<T>::to_f32(xl[u], f0, f1);
        Packed<T>::to_f32(xh[u], g0, g1);
        acc0 = fmaf(q0[2 * u], f0, acc0);
        acc1 = fmaf(q0[2 * u + 1], f1, acc1);
        acc0 = fmaf(q1[2 * u], g0, acc0);
        acc1 = fmaf(q1[2 * u + 1], g1, acc1);
      }
    } else {
      float xl[VEC], xh[VEC];
      load_vec_f32<T, VEC>(krow, xl);
      load_vec_f32<T, VEC>(krow + HALF, xh);
      if (rotary != LMK_ROTARY_NONE) {
        float cl[VEC], ch[VEC], sl[VEC], sh[VEC], ol[VEC], oh[VEC];
        load_vec_f32<T, VEC>(cr, cl);
        load_vec_f32<T, VEC>(cr + HALF, ch);
        load_vec_f32<T, VEC>(sr, sl);
        load_vec_f32<T, VEC>(sr + HALF, sh);
        if (rotary == LMK_ROTARY_HALF) {
#pragma unroll
          for (int u = 0; u < VEC; ++u) {
            ol[u] = __fadd_rn(__fmul_rn(xl[u], cl[u]), __fmul_rn(-xh[u], sl[u]));
            oh[u] = __fadd_rn(__fmul_rn(xh[u], ch[u]), __fmul_rn(xl[u], sh[u]));
          }
        } else {
#pragma unroll
          for (int u = 0; u < VEC; u += 2) {
            ol[u] = __fadd_rn(__fmul_rn(xl[u], cl[u]), __fmul_rn(-xl[u + 1], sl[u]));
            ol[u + 1] = __fadd_rn(__fmul_rn(xl[u + 1], cl[u + 1]), __fmul_rn(xl[u], sl[u + 1]));
            oh[u] = __fadd_rn(__fmul_rn(xh[u], ch[u]), __fmul_rn(-xh[u + 1], sh[u]));
            oh[u + 1] = __fadd_rn(__fmul_rn(xh[u + 1], ch[u + 1]), __fmul_rn(xh[u], sh[u + 1]));
          }
        }
#pragma unroll
        for (int u = 0; u < VEC; ++u) {
          xl[u] = ol[u];
          xh[u] = oh[u];
        }
      }
#pragma unroll
      for (int u = 0; u < VEC; ++u) {
        acc0 = fmaf(q0[u], xl[u], acc0);
        acc1 = fmaf(q1[u], xh[u], acc1);
      }
    }
  return acc0 + acc1;
}

template <typename T, int LPR>
__global__ void __launch_bounds__(128, kSelMinBlocks) selected_logits_kernel(const T* __restrict__ q, const T* __restrict__ kc,
                                                              lmk_cache_desc kd, const int32_t* __restrict__ idx,
                                                              const T* __restrict__ cos_t, const T* __restrict__ sin_t,
                                                              int n_pos, int rotary, T* __restrict__ logits,
                                                              int64_t ld, int64_t col0, int H, int Tq, float scale) {
  // A row of LPR 16-byte vectors is spread over LP = LPR / 2 lanes: lane `sub` holds vector `sub` of the low half of
  // the features and the same vector of the high half, which are exactly the two operands of one rotate_half pair, so
  // no lane needs another lane's data; a warp handles 32 / LP rows per step.
  constexpr int VEC = 16 / sizeof(T);
  constexpr int D = LPR * VEC, HALF = D / 2, LP = LPR / 2, RPS = 32 / LP;
  const int t = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LP, rsub = lane / LP, d0 = sub * VEC;
  const int blk = kd.block, N = kd.n_blocks, top_k = kd.top_k;
  float q0[VEC], q1[VEC];
  load_vec_f32<T, VEC>(q + ((int64_t)bh * Tq + t) * D + d0, q0);
  load_vec_f32<T, VEC>(q + ((int64_t)bh * Tq + t) * D + HALF + d0, q1);
#pragma unroll
  for (int u = 0; u < VEC; ++u) {
    q0[u] *= scale;
    q1[u] *= scale;
  }
  const int32_t* idx_row = idx + ((int64_t)bh * Tq + t) * top_k;
  const T* kbase = kc + b * kd.stride_b + h * kd.stride_h;
  T* out_row = logits + ((int64_t)bh * Tq + t) * ld + col0;
  for (int i = warp; i < top_k; i += 4) {
    const int sel = idx_row[i];
    const bool recent = logical_age(sel, kd.ring_start, N) >= N - top_k;
    const int pos0 = kd.pos_base + (i + (recent ? 1 : 0)) * blk;
    const T* ksrc = kbase + (int64_t)sel * kd.stride_block + d0;
#pragma unroll kSelUnroll
    for (int r0 = 0; r0 < blk; r0 += RPS) {
      const int r = r0 + rsub;
      float acc = 0.f;
      if (r < blk) {
        const T* krow = ksrc + (int64_t)r * kd.stride_row;
        const int pos = max(0, min(pos0 + r, n_pos - 1));
        acc = rotated_row_dot<T, VEC>(krow, cos_t + (int64_t)pos * D + d0, sin_t + (int64_t)pos * D + d0, HALF, rotary,
                                      q0, q1);
      }
#pragma unroll
      for (int o = LP / 2; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && r < blk) out_row[(int64_t)i * blk + r] = from_f32<T>(acc);
    }
  }
}

// out[b,h,t,:] = sum over the selected rows j of probs[b,h,t,col0 + j] * V[row j].  One CTA per (t, batch*head):
// 16-byte column vectors across the threads of a row group, row groups strided over the rows, fp32 partial sums
// combined through shared memory.
template <typename T>
__global__ void __launch_bounds__(128) selected_pv_kernel(const T* __restrict__ probs, int64_t ld, int64_t col0,
                                                          const T* __restrict__ vc, lmk_cache_desc vd,
                                                          const int32_t* __restrict__ idx, T* __restrict__ out, int H,
                                                          int Tq, int D) {
  constexpr int VEC = 16 / sizeof(T);
  struct __align__(16) Vec { T v[VEC]; };
  extern __shared__ __align__(16) float sel_smem[];
  const int t = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H;
  const int blk = vd.block, top_k = vd.top_k, rows = top_k * blk;
  float* ps = sel_smem;                       // [rows]
  float* red = ps + ((rows + 3) & ~3);        // [row groups][D]
  const T* pp = probs + ((int64_t)bh * Tq + t) * ld + col0;
  for (int j = threadIdx.x; j < rows; j += blockDim.x) ps[j] = to_f32(pp[j]);
  __syncthreads();
  const int vec_per_row = D / VEC, groups = blockDim.x / vec_per_row;
  const int vcol = threadIdx.x % vec_per_row, rg = threadIdx.x / vec_per_row;
  float acc[VEC];
#pragma unroll
  for (int u = 0; u < VEC; ++u) acc[u] = 0.f;
  const T* vbase = vc + b * vd.stride_b + h * vd.stride_h;
  if (rg < groups) {
    for (int i = 0; i < top_k; ++i) {
      const int sel = idx[((int64_t)bh * Tq + t) * top_k + i];
      const T* vsrc = vbase + (int64_t)sel * vd.stride_block + vcol * VEC;
#pragma unroll kPvUnroll
      for (int r = rg; r < blk; r += groups) {
        const Vec v = *reinterpret_cast<const Vec*>(vsrc + (int64_t)r * vd.stride_row);
        const float p = ps[i * blk + r];
#pragma unroll
        for (int u = 0; u < VEC; ++u) acc[u] = fmaf(p, to_f32(v.v[u]), acc[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < VEC; ++u) red[rg * D + vcol * VEC + u] = acc[u];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = 0.f;
    for (int g = 0; g < groups; ++g) sum += red[g * D + d];
    out[((int64_t)bh * Tq + t) * D + d] = from_f32<T>(sum);
  }
}

// Attention over the selected blocks, fused with the merge into the attention over the local keys: nothing between
// the block reads and the final output goes through global memory (no logits, no probabilities).  One CTA per
// (token, batch*head); warp i takes selected block i (then i + 4, ...):
//   logits of the block's rows (keys rotated at their slot positions, read in place) -> softmax over the block's
//   non-landmark rows and the landmark logit x_i (log2 domain) -> o_i = sum_r s_r V[r]  (all in shared memory / registers)
// and then all threads combine, with R the log2 of the local keys' share of the outer softmax:
//   out = (2^(R - m) O_local + sum_i 2^(x_i - m) o_i) / (2^(R - m) + sum_i 2^(x_i - m)),  m = max(R, x_i).
// This is the grouped softmax of llama/llama_mem.py:222-243 over [selected blocks | local keys] written out for the
// prefix pattern of :415 (every selected block is a closed group whose last row is its landmark).
template <typename T, int LPR>
__global__ void __launch_bounds__(128, 8) selected_attend_kernel(const T* __restrict__ q, const T* __restrict__ kc,
                                                              lmk_cache_desc kd, const T* __restrict__ vc,
                                                              lmk_cache_desc vd, const int32_t* __restrict__ idx,
                                                              const T* __restrict__ cos_t, const T* __restrict__ sin_t,
                                                              int n_pos, int rotary, const T* __restrict__ o_local,
                                                              const float* __restrict__ R_local, int64_t local_rows,
                                                              T* __restrict__ out, int H, int Tq, float scale) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int D = LPR * VEC, HALF = D / 2, LP = LPR / 2, RPS = 32 / LP;
  constexpr int VGROUPS = 32 / LPR > 0 ? 32 / LPR : 1;      // value rows a warp reads per step
  struct __align__(16) Vec { T v[VEC]; };
  extern __shared__ __align__(16) float att_smem[];
  const int t = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LP, rsub = lane / LP, d0 = sub * VEC;
  const int blk = kd.block, N = kd.n_blocks, top_k = kd.top_k;
  const bool sym = rotary == LMK_ROTARY_HALF_SYM;      // equal table halves: the second ones are not read
  if (sym) rotary = LMK_ROTARY_HALF;
  float* lg = att_smem;                         // [top_k][blk] logits, then probabilities inside the block
  float* osel = lg + ((top_k * blk + 3) & ~3);  // [top_k][D]
  float* xsel = osel + top_k * D;               // [top_k] landmark logits, log2 domain
  float q0[VEC], q1[VEC];
  load_vec_f32<T, VEC>(q + ((int64_t)bh * Tq + t) * D + d0, q0);
  load_vec_f32<T, VEC>(q + ((int64_t)bh * Tq + t) * D + HALF + d0, q1);
#pragma unroll
  for (int u = 0; u < VEC; ++u) {
    q0[u] *= scale;
    q1[u] *= scale;
  }
  const int32_t* idx_row = idx + ((int64_t)bh * Tq + t) * top_k;
  const T* kbase = kc + b * kd.stride_b + h * kd.stride_h;
  const T* vbase = vc + b * vd.stride_b + h * vd.stride_h;
  constexpr float kL2e = 1.4426950408889634f;
  for (int i = warp; i < top_k; i += 4) {
    const int sel = idx_row[i];
    const bool recent = logical_age(sel, kd.ring_start, N) >= N - top_k;
    const int pos0 = kd.pos_base + (i + (recent ? 1 : 0)) * blk;
    const T* ksrc = kbase + (int64_t)sel * kd.stride_block + d0;
    float* lrow = lg + i * blk;
    if constexpr (sizeof(T) == 2 && LPR == 16) {
      // D = 128 in a 16-bit type: the logits of 16 rows at a time as mma.sync m16n8k16 tiles.  Thread (g, t) of the
      // warp loads the 16-byte vectors [32 c + 8 t, +8) of rows g and g + 8 (c = 0..3), rotates them on packed pairs
      // as above, and feeds their registers straight to the A fragments: a dot product does not depend on the order
      // of the features, so "k index 2t, 2t+1, 2t+8, 2t+9" may stand for any four features as long as the query's B
      // fragment (column 0 only) holds the same ones.  The sums over the features happen inside the instruction.
      const int g8 = lane >> 2, t4 = lane & 3;
      const T* qrow = q + ((int64_t)bh * Tq + t) * D;
      const T* kblk = kbase + (int64_t)sel * kd.stride_block;
      for (int m = 0; m < blk; m += 16) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int ra = m + g8, rb = ra + 8;
        const T* ka = kblk + (int64_t)min(ra, blk - 1) * kd.stride_row + 8 * t4;
        const T* kb2 = kblk + (int64_t)min(rb, blk - 1) * kd.stride_row + 8 * t4;
        const int pa = max(0, min(pos0 + min(ra, blk - 1), n_pos - 1)), pb = max(0, min(pos0 + min(rb, blk - 1), n_pos - 1));
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {           // chunk cc of the low half with its partner cc + 2 of the high half
          uint32_t xa[2][4], xb[2][4];             // [low / high][register]
          ld16(ka + 32 * cc, xa[0]);
          ld16(ka + 32 * cc + HALF, xa[1]);
          ld16(kb2 + 32 * cc, xb[0]);
          ld16(kb2 + 32 * cc + HALF, xb[1]);
          if (rotary != LMK_ROTARY_NONE) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
              uint32_t (&x)[2][4] = rr == 0 ? xa : xb;
              const int64_t po = (int64_t)(rr == 0 ? pa : pb) * D + 32 * cc + 8 * t4;
              uint32_t cl[4], ch[4], sl[4], sh[4];
              ld16(cos_t + po, cl);
              ld16(sin_t + po, sl);
              if (sym) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  ch[u] = cl[u];
                  sh[u] = sl[u];
                }
              } else {
                ld16(cos_t + po + HALF, ch);
                ld16(sin_t + po + HALF, sh);
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                uint32_t pl, ph;
                if (rotary == LMK_ROTARY_HALF) {
                  pl = x[1][u] ^ 0x80008000u;
                  ph = x[0][u];
                } else {
                  pl = __byte_perm(x[0][u], x[0][u], 0x1032) ^ 0x00008000u;
                  ph = __byte_perm(x[1][u], x[1][u], 0x1032) ^ 0x00008000u;
                }
                const uint32_t lo = Packed<T>::add(Packed<T>::mul(x[0][u], cl[u]), Packed<T>::mul(pl, sl[u]));
                const uint32_t hi = Packed<T>::add(Packed<T>::mul(x[1][u], ch[u]), Packed<T>::mul(ph, sh[u]));
                x[0][u] = lo;
                x[1][u] = hi;
              }
            }
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {          // low chunk cc, then high chunk cc + 2
            uint32_t qf[4] = {0u, 0u, 0u, 0u};      // the query's features of this chunk: column 0 of B only
            if (g8 == 0) ld16(qrow + 32 * cc + hh * HALF + 8 * t4, qf);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                             "{%0,%1,%2,%3};"
                             : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                             : "r"(xa[hh][2 * h2]), "r"(xb[hh][2 * h2]), "r"(xa[hh][2 * h2 + 1]), "r"(xb[hh][2 * h2 + 1]),
                               "r"(qf[2 * h2]), "r"(qf[2 * h2 + 1]));
              } else {
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                             "{%0,%1,%2,%3};"
                             : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                             : "r"(xa[hh][2 * h2]), "r"(xb[hh][2 * h2]), "r"(xa[hh][2 * h2 + 1]), "r"(xb[hh][2 * h2 + 1]),
                               "r"(qf[2 * h2]), "r"(qf[2 * h2 + 1]));
              }
            }
          }
        }
        if (t4 == 0) {                              // column 0 of the result: rows g and g + 8
          if (ra < blk) lrow[ra] = acc[0] * scale * kL2e;
          if (rb < blk) lrow[rb] = acc[2] * scale * kL2e;
        }
      }
    } else
    for (int r0 = 0; r0 < blk; r0 += RPS) {
      const int r = r0 + rsub;
      float acc = 0.f;
      if (r < blk) {
        const int pos = max(0, min(pos0 + r, n_pos - 1));
        acc = rotated_row_dot<T, VEC>(ksrc + (int64_t)r * kd.stride_row, cos_t + (int64_t)pos * D + d0,
                                      sin_t + (int64_t)pos * D + d0, HALF, rotary, q0, q1);
      }
#pragma unroll
      for (int o = LP / 2; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && r < blk) lrow[r] = acc * kL2e;
    }
    __syncwarp();
    // softmax inside the block over rows 0 .. blk-2; the last row is the landmark
    float mx = -INFINITY;
    for (int r = lane; r < blk - 1; r += 32) mx = fmaxf(mx, lrow[r]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int r = lane; r < blk - 1; r += 32) den += exp2f(lrow[r] - mx);
    den = warp_sum(den);
    const float x_lm = lrow[blk - 1];
    __syncwarp();
    const float rden = den > 0.f ? 1.f / den : 0.f;
    for (int r = lane; r < blk; r += 32) lrow[r] = r < blk - 1 ? exp2f(lrow[r] - mx) * rden : 0.f;
    if (lane == 0) xsel[i] = x_lm;
    __syncwarp();
    // o_i = sum_r p_r V[r]: LPR lanes cover one value row, VGROUPS rows per step
    const int vcol = lane % LPR, rg = lane / LPR;
    float acc[VEC];
#pragma unroll
    for (int u = 0; u < VEC; ++u) acc[u] = 0.f;
    const T* vsrc = vbase + (int64_t)sel * vd.stride_block + vcol * VEC;
    if (rg < VGROUPS) {
#pragma unroll 4
      for (int r = rg; r < blk; r += VGROUPS) {
        const Vec v = *reinterpret_cast<const Vec*>(vsrc + (int64_t)r * vd.stride_row);
        const float p = lrow[r];
#pragma unroll
        for (int u = 0; u < VEC; ++u) acc[u] = fmaf(p, to_f32(v.v[u]), acc[u]);
      }
    }
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1)
#pragma unroll
      for (int u = 0; u < VEC; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
    if (lane < LPR)
#pragma unroll
      for (int u = 0; u < VEC; ++u) osel[i * D + vcol * VEC + u] = acc[u];
  }
  __syncthreads();
  float Rl = R_local != nullptr ? R_local[(int64_t)bh * local_rows + t] : -INFINITY;
  if (Rl == INFINITY) Rl = -INFINITY;            // no local key is visible to this query
  float m = Rl;
  for (int i = 0; i < top_k; ++i) m = fmaxf(m, xsel[i]);
  const float w_loc = m == -INFINITY ? 0.f : exp2f(Rl - m);
  float Z = w_loc;
  for (int i = 0; i < top_k; ++i) Z += m == -INFINITY ? 0.f : exp2f(xsel[i] - m);
  const float rZ = Z > 0.f ? 1.f / Z : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = (R_local != nullptr && w_loc > 0.f) ? w_loc * to_f32(o_local[((int64_t)bh * local_rows + t) * D + d]) : 0.f;
    for (int i = 0; i < top_k; ++i) sum = fmaf(m == -INFINITY ? 0.f : exp2f(xsel[i] - m), osel[i * D + d], sum);
    out[((int64_t)bh * Tq + t) * D + d] = from_f32<T>(sum * rZ);
  }
}

int check_desc(const lmk_cache_desc* d, const char* what) {
  LMK_CHECK_ARG(d != nullptr, "%s: null cache descriptor", what);
  LMK_CHECK_ARG(d->block >= 1 && d->n_blocks >= 1, "%s: block %d / n_blocks %d must be positive", what, d->block,
                d->n_blocks);
  LMK_CHECK_ARG(d->top_k >= 0 && d->top_k <= d->n_blocks, "%s: top_k %d outside [0, n_blocks=%d]", what, d->top_k,
                d->n_blocks);
  LMK_CHECK_ARG(d->ring_start >= 0 && d->ring_start < d->n_blocks, "%s: ring_start %d outside [0, %d)", what,
                d->ring_start, d->n_blocks);
  return LMK_OK;
}

}  // namespace
}  // namespace lmk

using namespace lmk;

extern "C" int lmk_landmark_scores(const void* q, const void* k_cache, const lmk_cache_desc* desc,
                                   const void* cos_table, const void* sin_table, int n_pos, int rotary, float* scores,
                                   int B, int H, int T, int D, float sm_scale, int softmax, int dtype, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  int rc = check_desc(desc, "landmark_scores");
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(q && k_cache && scores, "landmark_scores: null pointer");
  LMK_CHECK_ARG(B >= 1 && H >= 1 && T >= 1, "landmark_scores: empty problem");
  LMK_CHECK_ARG(D >= 8 && D <= 256 && D % 8 == 0, "landmark_scores: head dim %d must be a multiple of 8 in [8,256]", D);
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "landmark_scores: bad dtype %d", dtype);
  LMK_CHECK_ARG(rotary >= LMK_ROTARY_NONE && rotary <= LMK_ROTARY_INTERLEAVED, "landmark_scores: bad rotary %d", rotary);
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || (cos_table && sin_table && n_pos >= 1),
                "landmark_scores: rotary tables missing");
  LMK_CHECK_ARG((int64_t)B * H <= 65535 && (T + kScTile - 1) / kScTile <= 65535, "landmark_scores: grid too large");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = (int64_t)B * H * T;
  if (workspace != nullptr && scores_sm100_supported(D, dtype, T, desc->n_blocks) &&
      workspace_bytes >= scores_sm100_workspace(B, H, desc->n_blocks) && ((uintptr_t)workspace % 256 == 0) &&
      (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)cos_table | (uintptr_t)sin_table) % 16 == 0) &&
      desc->stride_b % 8 == 0 && desc->stride_h % 8 == 0 && desc->stride_block % 8 == 0 && desc->stride_row % 8 == 0) {
    rc = scores_sm100(q, k_cache, *desc, cos_table, sin_table, n_pos, rotary, scores, B, H, T, sm_scale, dtype,
                      workspace, st);
    if (rc != LMK_OK) return rc;
    if (softmax) {
      if (dtype == LMK_F16) row_softmax_kernel<__half><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(scores, rows, desc->n_blocks);
      else row_softmax_kernel<__nv_bfloat16><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(scores, rows, desc->n_blocks);
      LMK_CUDA(cudaGetLastError());
    }
    return LMK_OK;
  }
  size_t smem = sizeof(float) * ((size_t)kScTile * D + (size_t)kScTile * (D + 1));
  dim3 grid((desc->n_blocks + kScTile - 1) / kScTile, (T + kScTile - 1) / kScTile, B * H);
#define LMK_SC_LAUNCH(TT)                                                                                          \
  do {                                                                                                             \
    LMK_CUDA(cudaFuncSetAttribute(landmark_scores_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                  (int)smem));                                                                     \
    landmark_scores_kernel<TT><<<grid, 128, smem, st>>>((const TT*)q, (const TT*)k_cache, *desc,                   \
                                                        (const TT*)cos_table, (const TT*)sin_table, n_pos, rotary, \
                                                        scores, H, T, D, sm_scale);                                \
    if (softmax)                                                                                                   \
      row_softmax_kernel<TT><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(scores, rows, desc->n_blocks);            \
  } while (0)
  if (dtype == LMK_F32) LMK_SC_LAUNCH(float);
  else if (dtype == LMK_F16) LMK_SC_LAUNCH(__half);
  else LMK_SC_LAUNCH(__nv_bfloat16);
#undef LMK_SC_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" size_t lmk_landmark_scores_workspace(int B, int H, int T, int D, int n_blocks, int dtype) {
  if (B < 1 || H < 1 || n_blocks < 1 || !scores_sm100_supported(D, dtype, T, n_blocks)) return 0;
  return scores_sm100_workspace(B, H, n_blocks);
}

extern "C" int lmk_topk_sorted(const float* scores, int32_t* idx_out, int64_t outer_count, int64_t inner_count,
                               int64_t outer_stride, int64_t inner_stride, int reduce, int64_t reduce_stride, int n,
                               int k, int ring_start, void* stream) {
  LMK_CHECK_ARG(scores && idx_out, "topk_sorted: null pointer");
  LMK_CHECK_ARG(outer_count >= 1 && inner_count >= 1 && reduce >= 1, "topk_sorted: empty problem");
  LMK_CHECK_ARG(n >= 1 && n <= 49152, "topk_sorted: n %d outside [1, 49152]", n);
  LMK_CHECK_ARG(k >= 1 && k <= kTopkMaxK && k <= n, "topk_sorted: k %d outside [1, min(n, %d)]", k, kTopkMaxK);
  LMK_CHECK_ARG(ring_start >= 0 && ring_start < n, "topk_sorted: ring_start %d outside [0, n)", ring_start);
  const int64_t rows = outer_count * inner_count;
  if (reduce > 1) {
    const bool vec4 = (n & 3) == 0 && (((uintptr_t)scores | (uintptr_t)(outer_stride * 4) | (uintptr_t)(inner_stride * 4) |
                                       (uintptr_t)(reduce_stride * 4)) & 15) == 0;
    int parts = 1;
    if (vec4) {
      parts = 1024 / (n / 4);                          // thread groups that split the reduce range
      parts = parts < 1 ? 1 : (parts > 8 ? 8 : parts);
      if (parts > reduce) parts = reduce;
      while ((size_t)parts * n * sizeof(float) > 200 * 1024) --parts;
    }
    const size_t rsmem = sizeof(float) * (size_t)n * parts;
    LMK_CUDA(cudaFuncSetAttribute(topk_reduce_sorted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rsmem));
    topk_reduce_sorted_kernel<<<(unsigned)rows, 1024, rsmem, (cudaStream_t)stream>>>(
        scores, idx_out, inner_count, outer_stride, inner_stride, reduce, reduce_stride, n, k, ring_start, vec4 ? 1 : 0,
        parts);
    LMK_CUDA(cudaGetLastError());
    return LMK_OK;
  }
  if (n <= 1024 && (n & 3) == 0 && k <= 32 &&
      (((uintptr_t)scores | (uintptr_t)(outer_stride * 4) | (uintptr_t)(inner_stride * 4)) & 15) == 0) {
    const size_t rsm = sizeof(float) * 4 * ((size_t)n + 2 * kTopkRegCand);
    topk_sorted_rows_kernel<<<(unsigned)((rows + 3) / 4), 128, rsm, (cudaStream_t)stream>>>(
        scores, idx_out, rows, inner_count, outer_stride, inner_stride, n, k, ring_start);
    LMK_CUDA(cudaGetLastError());
    return LMK_OK;
  }
  int wpc = n <= 2048 ? 4 : (n <= 8192 ? 2 : 1);
  size_t smem = sizeof(float) * (size_t)n * wpc;
  LMK_CUDA(cudaFuncSetAttribute(topk_sorted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_sorted_kernel<<<(unsigned)((rows + wpc - 1) / wpc), 128, smem, (cudaStream_t)stream>>>(
      scores, idx_out, rows, inner_count, outer_stride, inner_stride, reduce, reduce_stride, n, k, ring_start, wpc);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_gather_kv(const void* k_cache, const void* v_cache, const lmk_cache_desc* kdesc,
                             const lmk_cache_desc* vdesc, const int32_t* idx, const void* cos_table,
                             const void* sin_table, int n_pos, int rotary, void* k_out, void* v_out, int B, int H,
                             int T, int D, int dtype, void* stream) {
  int rc = check_desc(kdesc, "gather_kv");
  if (rc != LMK_OK) return rc;
  if (v_out != nullptr) {
    rc = check_desc(vdesc, "gather_kv(v)");
    if (rc != LMK_OK) return rc;
    LMK_CHECK_ARG(v_cache != nullptr, "gather_kv: v_out given without v_cache");
    LMK_CHECK_ARG(vdesc->block == kdesc->block && vdesc->n_blocks == kdesc->n_blocks && vdesc->top_k == kdesc->top_k,
                  "gather_kv: key and value cache descriptors disagree");
  }
  LMK_CHECK_ARG(idx != nullptr && (k_out != nullptr || v_out != nullptr), "gather_kv: null pointer");
  LMK_CHECK_ARG(k_out == nullptr || k_cache != nullptr, "gather_kv: k_out given without k_cache");
  LMK_CHECK_ARG(kdesc->top_k >= 1, "gather_kv: top_k must be >= 1");
  LMK_CHECK_ARG(B >= 1 && H >= 1 && T >= 1, "gather_kv: empty problem");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "gather_kv: bad dtype %d", dtype);
  const int vec = 16 / dtype_size(dtype);
  LMK_CHECK_ARG(D >= 2 * vec && D % (2 * vec) == 0, "gather_kv: head dim %d must be a multiple of %d", D, 2 * vec);
  LMK_CHECK_ARG(rotary >= LMK_ROTARY_NONE && rotary <= LMK_ROTARY_INTERLEAVED, "gather_kv: bad rotary %d", rotary);
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || k_out == nullptr || (cos_table && sin_table && n_pos >= 1),
                "gather_kv: rotary tables missing");
  const lmk_cache_desc* descs[2] = {kdesc, v_out ? vdesc : kdesc};
  for (const lmk_cache_desc* d : descs)
    LMK_CHECK_ARG(d->stride_b % vec == 0 && d->stride_h % vec == 0 && d->stride_block % vec == 0 &&
                      d->stride_row % vec == 0,
                  "gather_kv: cache strides must be multiples of %d elements (16 bytes)", vec);
  LMK_CHECK_ARG(((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)k_out | (uintptr_t)v_out |
                 (uintptr_t)cos_table | (uintptr_t)sin_table) % 16 == 0,
                "gather_kv: pointers must be 16-byte aligned");
  LMK_CHECK_ARG((int64_t)B * H <= 65535 && T <= 65535, "gather_kv: grid too large");
  dim3 grid(kdesc->top_k, T, B * H);
  cudaStream_t st = (cudaStream_t)stream;
  lmk_cache_desc vd = v_out ? *vdesc : *kdesc;
#define LMK_GA_LAUNCH(TT)                                                                                      \
  gather_kv_kernel<TT><<<grid, 128, 0, st>>>((const TT*)k_cache, (const TT*)v_cache, *kdesc, vd, idx,          \
                                             (const TT*)cos_table, (const TT*)sin_table, n_pos, rotary,        \
                                             (TT*)k_out, (TT*)v_out, H, T, D)
  if (dtype == LMK_F32) LMK_GA_LAUNCH(float);
  else if (dtype == LMK_F16) LMK_GA_LAUNCH(__half);
  else LMK_GA_LAUNCH(__nv_bfloat16);
#undef LMK_GA_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_selected_logits(const void* q, const void* k_cache, const lmk_cache_desc* kdesc, const int32_t* idx,
                                   const void* cos_table, const void* sin_table, int n_pos, int rotary, void* logits,
                                   int64_t ld, int64_t col0, int B, int H, int T, int D, float sm_scale, int dtype,
                                   void* stream) {
  int rc = check_desc(kdesc, "selected_logits");
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(q && k_cache && idx && logits, "selected_logits: null pointer");
  LMK_CHECK_ARG((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)cos_table | (uintptr_t)sin_table) & 15) == 0,
                "selected_logits: q, cache and rotary tables must be 16-byte aligned");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "selected_logits: unknown dtype %d", dtype);
  LMK_CHECK_ARG(B >= 0 && H >= 1 && T >= 0 && D >= 1, "selected_logits: bad shape");
  const int vec = dtype == LMK_F32 ? 4 : 8;
  const int lpr = D / vec;
  LMK_CHECK_ARG(D % vec == 0 && (lpr == 4 || lpr == 8 || lpr == 16 || lpr == 32),
                "selected_logits: D=%d must be 4, 8, 16 or 32 vectors of 16 bytes", D);
  LMK_CHECK_ARG(kdesc->stride_row % vec == 0 && kdesc->stride_block % vec == 0 && kdesc->stride_h % vec == 0 &&
                    kdesc->stride_b % vec == 0,
                "selected_logits: cache strides must be multiples of %d elements", vec);
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || (cos_table && sin_table && n_pos >= 1),
                "selected_logits: rotary needs cos/sin tables");
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || rotary == LMK_ROTARY_HALF || rotary == LMK_ROTARY_INTERLEAVED,
                "selected_logits: unknown rotary mode %d", rotary);
  LMK_CHECK_ARG(col0 >= 0 && ld >= col0 + (int64_t)kdesc->top_k * kdesc->block,
                "selected_logits: row stride %lld too small for %d x %d columns at offset %lld", (long long)ld,
                kdesc->top_k, kdesc->block, (long long)col0);
  if (B == 0 || T == 0 || kdesc->top_k == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "selected_logits: grid too large");
  dim3 grid(T, B * H);
  cudaStream_t st = (cudaStream_t)stream;
#define LMK_SL_LAUNCH(TT, LPR)                                                                                     \
  selected_logits_kernel<TT, LPR><<<grid, 128, 0, st>>>((const TT*)q, (const TT*)k_cache, *kdesc, idx,            \
                                                        (const TT*)cos_table, (const TT*)sin_table, n_pos, rotary, \
                                                        (TT*)logits, ld, col0, H, T, sm_scale)
#define LMK_SL_DISPATCH(TT)                     \
  switch (lpr) {                                \
    case 4: LMK_SL_LAUNCH(TT, 4); break;        \
    case 8: LMK_SL_LAUNCH(TT, 8); break;        \
    case 16: LMK_SL_LAUNCH(TT, 16); break;      \
    default: LMK_SL_LAUNCH(TT, 32); break;      \
  }
  if (dtype == LMK_F32) { LMK_SL_DISPATCH(float) }
  else if (dtype == LMK_F16) { LMK_SL_DISPATCH(__half) }
  else { LMK_SL_DISPATCH(__nv_bfloat16) }
#undef LMK_SL_DISPATCH
#undef LMK_SL_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_selected_pv(const void* probs, int64_t ld, int64_t col0, const void* v_cache,
                               const lmk_cache_desc* vdesc, const int32_t* idx, void* out, int B, int H, int T, int D,
                               int dtype, void* stream) {
  int rc = check_desc(vdesc, "selected_pv");
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(probs && v_cache && idx && out, "selected_pv: null pointer");
  LMK_CHECK_ARG(((uintptr_t)v_cache & 15) == 0, "selected_pv: the cache must be 16-byte aligned");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "selected_pv: unknown dtype %d", dtype);
  LMK_CHECK_ARG(B >= 0 && H >= 1 && T >= 0 && D >= 1, "selected_pv: bad shape");
  const int vec = dtype == LMK_F32 ? 4 : 8;
  LMK_CHECK_ARG(D % vec == 0 && D / vec <= 128 && 128 % (D / vec) == 0,
                "selected_pv: D=%d must give a power-of-two number (<= 128) of 16-byte vectors per row", D);
  LMK_CHECK_ARG(vdesc->stride_row % vec == 0 && vdesc->stride_block % vec == 0 && vdesc->stride_h % vec == 0 &&
                    vdesc->stride_b % vec == 0,
                "selected_pv: cache strides must be multiples of %d elements", vec);
  const int64_t rows = (int64_t)vdesc->top_k * vdesc->block;
  LMK_CHECK_ARG(col0 >= 0 && ld >= col0 + rows, "selected_pv: row stride %lld too small", (long long)ld);
  if (B == 0 || T == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "selected_pv: grid too large");
  const size_t smem = (size_t)(((rows + 3) & ~3) + (int64_t)(128 / (D / vec)) * D) * sizeof(float);
  LMK_CHECK_ARG(smem <= 48 * 1024, "selected_pv: top_k * block = %lld rows do not fit in shared memory",
                (long long)rows);
  dim3 grid(T, B * H);
  cudaStream_t st = (cudaStream_t)stream;
#define LMK_SP_LAUNCH(TT)                                                                                       \
  selected_pv_kernel<TT><<<grid, 128, smem, st>>>((const TT*)probs, ld, col0, (const TT*)v_cache, *vdesc, idx,  \
                                                  (TT*)out, H, T, D)
  if (dtype == LMK_F32) LMK_SP_LAUNCH(float);
  else if (dtype == LMK_F16) LMK_SP_LAUNCH(__half);
  else LMK_SP_LAUNCH(__nv_bfloat16);
#undef LMK_SP_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_selected_attend(const void* q, const void* k_cache, const lmk_cache_desc* kdesc, const void* v_cache,
                                   const lmk_cache_desc* vdesc, const int32_t* idx, const void* cos_table,
                                   const void* sin_table, int n_pos, int rotary, const void* o_local,
                                   const float* R_local, int64_t local_rows, void* out, int B, int H, int T, int D,
                                   float sm_scale, int dtype, void* stream) {
  int rc = check_desc(kdesc, "selected_attend");
  if (rc != LMK_OK) return rc;
  if ((rc = check_desc(vdesc, "selected_attend")) != LMK_OK) return rc;
  LMK_CHECK_ARG(q && k_cache && v_cache && idx && out, "selected_attend: null pointer");
  LMK_CHECK_ARG((R_local == nullptr) == (o_local == nullptr), "selected_attend: o_local and R_local go together");
  LMK_CHECK_ARG(R_local == nullptr || local_rows >= T, "selected_attend: local_rows %lld < T %d", (long long)local_rows, T);
  LMK_CHECK_ARG((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_table | (uintptr_t)sin_table) &
                 15) == 0, "selected_attend: q, caches and rotary tables must be 16-byte aligned");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "selected_attend: unknown dtype %d", dtype);
  LMK_CHECK_ARG(B >= 0 && H >= 1 && T >= 0 && D >= 1, "selected_attend: bad shape");
  LMK_CHECK_ARG(kdesc->block == vdesc->block && kdesc->top_k == vdesc->top_k && kdesc->n_blocks == vdesc->n_blocks &&
                    kdesc->ring_start == vdesc->ring_start, "selected_attend: key and value descriptors disagree");
  LMK_CHECK_ARG(kdesc->block >= 2, "selected_attend: a block needs at least one key before its landmark");
  const int vec = dtype == LMK_F32 ? 4 : 8;
  const int lpr = D / vec;
  LMK_CHECK_ARG(D % vec == 0 && (lpr == 4 || lpr == 8 || lpr == 16 || lpr == 32),
                "selected_attend: D=%d must be 4, 8, 16 or 32 vectors of 16 bytes", D);
  for (const lmk_cache_desc* d : {kdesc, vdesc})
    LMK_CHECK_ARG(d->stride_row % vec == 0 && d->stride_block % vec == 0 && d->stride_h % vec == 0 &&
                      d->stride_b % vec == 0, "selected_attend: cache strides must be multiples of %d elements", vec);
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || (cos_table && sin_table && n_pos >= 1),
                "selected_attend: rotary needs cos/sin tables");
  LMK_CHECK_ARG(rotary == LMK_ROTARY_NONE || rotary == LMK_ROTARY_HALF || rotary == LMK_ROTARY_INTERLEAVED ||
                    rotary == LMK_ROTARY_HALF_SYM,
                "selected_attend: unknown rotary mode %d", rotary);
  LMK_CHECK_ARG(kdesc->top_k >= 1, "selected_attend: top_k must be at least 1");
  if (B == 0 || T == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "selected_attend: grid too large");
  const size_t smem = (size_t)(((kdesc->top_k * kdesc->block + 3) & ~3) + kdesc->top_k * D + kdesc->top_k) * sizeof(float);
  LMK_CHECK_ARG(smem <= 48 * 1024, "selected_attend: top_k * (block + D) = %d x (%d + %d) floats do not fit in shared memory",
                kdesc->top_k, kdesc->block, D);
  dim3 grid(T, B * H);
  cudaStream_t st = (cudaStream_t)stream;
#define LMK_SA_LAUNCH(TT, LPR)                                                                                        \
  selected_attend_kernel<TT, LPR><<<grid, 128, smem, st>>>((const TT*)q, (const TT*)k_cache, *kdesc,                 \
                                                           (const TT*)v_cache, *vdesc, idx, (const TT*)cos_table,    \
                                                           (const TT*)sin_table, n_pos, rotary, (const TT*)o_local,  \
                                                           R_local, local_rows, (TT*)out, H, T, sm_scale)
#define LMK_SA_DISPATCH(TT)                     \
  switch (lpr) {                                \
    case 4: LMK_SA_LAUNCH(TT, 4); break;        \
    case 8: LMK_SA_LAUNCH(TT, 8); break;        \
    case 16: LMK_SA_LAUNCH(TT, 16); break;      \
    default: LMK_SA_LAUNCH(TT, 32); break;      \
  }
  if (dtype == LMK_F32) { LMK_SA_DISPATCH(float) }
  else if (dtype == LMK_F16) { LMK_SA_DISPATCH(__half) }
  else { LMK_SA_DISPATCH(__nv_bfloat16) }
#undef LMK_SA_DISPATCH
#undef LMK_SA_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}
