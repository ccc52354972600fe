// Stand-alone landmark grouped softmax (forward and backward) on materialised score rows.
//
// One warp owns one row [Lk].  Keys that are neither landmark, last-section nor hidden belong to the group whose
// id is the running count of landmarks (an inclusive prefix count, so ids never decrease along the row and each
// group is a contiguous run once bucket members are given the identity element).  The bucket = {landmarks,
// last-section keys, hidden keys} has its own softmax.  Group reductions are segmented warp scans keyed on the
// prefix count; the last lane of each segment is the only writer of that group's slot, and chunks are visited
// in order, so results are bit-reproducible (no floating-point atomics).
//
// Reference semantics: llama/llama_mem.py:168-243 (guards = 0) and lm_benchmark/models/landmark.py:37-119
// (guards = 1: an all -inf group yields 0 instead of NaN, :48,:54).
#include "common.cuh"
#include "attn_params.h"

namespace lmk {
namespace {

constexpr int kGsWarps = 4;

struct GsParams {
  const void* x;
  int64_t xs[3];
  const uint8_t* is_mem; int64_t ms[4];
  const uint8_t* last; int64_t ls[4];
  const uint8_t* hidden; int64_t hs[4];
  float* probs;
  float* group_prob; int max_mem_cnt;
  const float* gprobs;
  float* gx;
  int B, H, Lq, Lk, guards, max_groups;
  // causal mode of the rows kernel: the three masks are derived from one flag per (batch row, key) and the rule
  // "query i sees keys 0 .. i + Lk - Lq" (mask block of lm_benchmark/models/landmark.py:210-224); hidden scores count
  // as -inf whatever x holds there
  const uint8_t* row_flags; int64_t row_flags_stride; int causal;
  int* status;          // device status word: set to kErrSoftmaxGroups when a row holds max_groups or more landmarks
};

enum { kErrSoftmaxGroups = 501 };

struct Elem {
  float x;
  bool mem, last, hid, bucket, in;
  int c;   // inclusive landmark count
};

template <typename T>
struct RowReader {
  const T* x;
  const uint8_t *m, *l, *h;
  int64_t mcs, lcs, hcs;
  int Lk, lane;
  int base;   // landmarks seen before the current chunk
  __device__ __forceinline__ void restart() { base = 0; }
  __device__ __forceinline__ Elem load(int j0) {
    Elem e;
    int j = j0 + lane;
    e.in = j < Lk;
    e.x = e.in ? to_f32(x[j]) : -INFINITY;
    e.mem = e.in && m[j * mcs] != 0;
    e.last = e.in && l[j * lcs] != 0;
    e.hid = e.in && h != nullptr && h[j * hcs] != 0;
    unsigned bal = __ballot_sync(0xffffffffu, e.mem);
    e.c = base + __popc(bal & (0xffffffffu >> (31 - lane)));
    base += __popc(bal);
    e.bucket = e.mem || e.last || e.hid || !e.in;
    return e;
  }
};

// inclusive segmented scans over lanes; segments = runs of equal key
__device__ __forceinline__ float seg_scan_max(float v, int key, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float u = __shfl_up_sync(0xffffffffu, v, o);
    int k = __shfl_up_sync(0xffffffffu, key, o);
    if (lane >= o && k == key) v = fmaxf(v, u);
  }
  return v;
}
__device__ __forceinline__ float seg_scan_sum(float v, int key, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    float u = __shfl_up_sync(0xffffffffu, v, o);
    int k = __shfl_up_sync(0xffffffffu, key, o);
    if (lane >= o && k == key) v += u;
  }
  return v;
}
__device__ __forceinline__ bool seg_tail(int key, int lane) {
  int nk = __shfl_down_sync(0xffffffffu, key, 1);
  return lane == 31 || nk != key;
}

template <typename T, bool kBackward>
__global__ void __launch_bounds__(kGsWarps * 32) grouped_softmax_kernel(GsParams p) {
  extern __shared__ float gs_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = p.max_groups;
  float* gmax = gs_smem + (size_t)warp * G * 4;
  float* gsum = gmax + G;
  float* gw = gsum + G;     // exp(landmark score - bucket max) of the landmark closing each group
  float* gc = gw + G;       // backward: sum over the group of inner prob * grad
  const int64_t row = (int64_t)blockIdx.x * kGsWarps + warp;
  const int64_t rows = (int64_t)p.B * p.H * p.Lq;
  if (row >= rows) return;
  const int b = (int)(row / ((int64_t)p.H * p.Lq));
  const int h = (int)((row / p.Lq) % p.H);
  const int i = (int)(row % p.Lq);

  RowReader<T> rd;
  rd.x = reinterpret_cast<const T*>(p.x) + b * p.xs[0] + h * p.xs[1] + i * p.xs[2];
  rd.m = p.is_mem + b * p.ms[0] + h * p.ms[1] + i * p.ms[2];
  rd.l = p.last + b * p.ls[0] + h * p.ls[1] + i * p.ls[2];
  rd.h = p.hidden ? p.hidden + b * p.hs[0] + h * p.hs[1] + i * p.hs[2] : nullptr;
  rd.mcs = p.ms[3]; rd.lcs = p.ls[3]; rd.hcs = p.hs[3];
  rd.Lk = p.Lk; rd.lane = lane;
  const bool guards = p.guards != 0;

  for (int g = lane; g < G; g += 32) {
    gmax[g] = -INFINITY;
    gsum[g] = 0.f;
    gw[g] = 0.f;
    gc[g] = 0.f;
  }
  __syncwarp();

  // pass 1: maxima
  float bmax = -INFINITY;
  rd.restart();
  for (int j0 = 0; j0 < p.Lk; j0 += 32) {
    Elem e = rd.load(j0);
    bmax = fmaxf(bmax, (e.bucket && e.in) ? e.x : -INFINITY);
    float v = seg_scan_max(e.bucket ? -INFINITY : e.x, e.c, lane);
    if (seg_tail(e.c, lane) && e.c < G) gmax[e.c] = fmaxf(gmax[e.c], v);
    __syncwarp();
  }
  if (lane == 0 && rd.base >= G && p.status != nullptr) atomicCAS(p.status, 0, kErrSoftmaxGroups);
  bmax = warp_max(bmax);
  if (guards && isinf(bmax)) bmax = 0.f;

  // pass 2: sums; remember exp(landmark - bmax) per closed group
  float bsum = 0.f;
  rd.restart();
  for (int j0 = 0; j0 < p.Lk; j0 += 32) {
    Elem e = rd.load(j0);
    float ex = 0.f;
    if (e.in) {
      if (e.bucket) {
        ex = expf(e.x - bmax);
        bsum += ex;
        if (e.mem && e.c - 1 < G) gw[e.c - 1] = ex;
      } else if (e.c < G) {
        float mx = gmax[e.c];
        if (guards && isinf(mx)) mx = 0.f;
        ex = expf(e.x - mx);
      }
    }
    float v = seg_scan_sum(e.bucket ? 0.f : ex, e.c, lane);
    if (seg_tail(e.c, lane) && e.c < G) gsum[e.c] += v;
    __syncwarp();
  }
  bsum = warp_sum(bsum);
  const float binv = (guards && bsum < 0.5f) ? 0.f : 1.f / bsum;

  if (!kBackward) {
    float* out = p.probs + row * p.Lk;
    float last_total = 0.f;
    rd.restart();
    for (int j0 = 0; j0 < p.Lk; j0 += 32) {
      Elem e = rd.load(j0);
      float pr = 0.f;
      if (e.in) {
        if (e.bucket) {
          pr = e.last ? expf(e.x - bmax) * binv : 0.f;
          if (!guards && !e.last) pr = expf(e.x - bmax) * binv * 0.f;   // keeps NaN propagation of the llama flavour
          last_total += e.last ? pr : 0.f;
        } else if (e.c < G) {
          float mx = gmax[e.c];
          if (guards && isinf(mx)) mx = 0.f;
          float den = gsum[e.c];
          float inner = (guards && den < 0.5f) ? 0.f : expf(e.x - mx) / den;
          pr = inner * (gw[e.c] * binv);
        }
        out[j0 + lane] = pr;
      }
    }
    if (p.group_prob != nullptr) {
      last_total = warp_sum(last_total);
      float* gp = p.group_prob + row * p.max_mem_cnt;
      for (int g = lane; g < p.max_mem_cnt - 1; g += 32) gp[g] = g < G ? gw[g] * binv : 0.f;
      if (lane == 0) gp[p.max_mem_cnt - 1] = last_total;
    }
  } else {
    // pass 3: c_g = sum_j inner_j * grad_j per group, T = sum_j P_j * grad_j over the row
    const float* gr = p.gprobs + row * p.Lk;
    float total = 0.f;
    rd.restart();
    for (int j0 = 0; j0 < p.Lk; j0 += 32) {
      Elem e = rd.load(j0);
      float contrib = 0.f;
      if (e.in) {
        float gj = gr[j0 + lane];
        if (e.bucket) {
          if (e.last) total += expf(e.x - bmax) * binv * gj;
        } else if (e.c < G) {
          float mx = gmax[e.c];
          if (guards && isinf(mx)) mx = 0.f;
          float den = gsum[e.c];
          float inner = (guards && den < 0.5f) ? 0.f : expf(e.x - mx) / den;
          contrib = inner * gj;
          total += contrib * gw[e.c] * binv;
        }
      }
      float v = seg_scan_sum(contrib, e.c, lane);
      if (seg_tail(e.c, lane) && e.c < G) gc[e.c] += v;
      __syncwarp();
    }
    total = warp_sum(total);
    // pass 4: gradients
    float* out = p.gx + row * p.Lk;
    rd.restart();
    for (int j0 = 0; j0 < p.Lk; j0 += 32) {
      Elem e = rd.load(j0);
      if (!e.in) continue;
      float gj = gr[j0 + lane];
      float dx = 0.f;
      if (e.bucket) {
        float bj = expf(e.x - bmax) * binv;
        float hj = (e.last ? gj : 0.f) + ((e.mem && e.c - 1 < G) ? gc[e.c - 1] : 0.f);
        dx = (e.hid && !e.last && !e.mem) ? 0.f : bj * (hj - total);
      } else if (e.c < G) {
        float mx = gmax[e.c];
        if (guards && isinf(mx)) mx = 0.f;
        float den = gsum[e.c];
        float inner = (guards && den < 0.5f) ? 0.f : expf(e.x - mx) / den;
        dx = inner * gw[e.c] * binv * (gj - gc[e.c]);
      }
      out[j0 + lane] = dx;
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Rows of up to kFastMaxLk keys: the row is copied from global memory to shared memory once (cp.async, the whole row
// in flight at a time), eight contiguous keys per lane, and kept there (raw scores, then exponentials) together with
// the decoded mask bits and the landmark count in front of every lane's keys.  A lane walks its eight keys
// sequentially; only the partial result of the group that is open at the lane's last key (and, for lanes holding a
// landmark, the part in front of its first landmark) crosses lanes, through one segmented scan per 256 keys instead
// of one per 32.  Chunks of 256 keys that are hidden and -inf throughout (the upper triangle of a causal score
// matrix) are recognised in the first pass and skipped by the others.  All sums are taken in a fixed order, so
// results are bit-reproducible.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kFastMaxLk = 4096;
constexpr int kFastChunk = 256;
constexpr size_t kFastMaxSmem = 96 * 1024;
constexpr float kLog2e = 1.4426950408889634f;

// exp(a - b) as 2^((a - b) * log2 e): the difference is formed first, so that the argument's rounding error stays
// proportional to the (small) distance from the maximum.
__device__ __forceinline__ float exp_diff(float a, float b) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"((a - b) * kLog2e));
  return y;
}

// Raw flags of a lane's eight keys, one byte per key: lo = keys 0-3, hi = keys 4-7;
// bit 0 landmark, bit 1 last section, bit 2 hidden, bit 3 inside the row.  Keys beyond the row's end read 0x04.
struct RawFlags { uint32_t lo, hi; };

// Byte-wise forms of the row accesses for rows whose pieces are unaligned, strided or cut by the row's end; kept out
// of line so that the common path stays small in the instruction cache.
__device__ __noinline__ uint2 mask_bytes_slow(const uint8_t* p, int64_t cs, int j, int n_in) {
  uint2 w = make_uint2(0u, 0u);
  for (int v = 0; v < n_in; ++v)
    if (p[(int64_t)(j + v) * cs] & 1u) (v < 4 ? w.x : w.y) |= 1u << (8 * (v & 3));
  return w;
}
__device__ __noinline__ float4 load4f_slow(const float* g, int n) {
  float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
  if (n > 0) r.x = g[0];
  if (n > 1) r.y = g[1];
  if (n > 2) r.z = g[2];
  if (n > 3) r.w = g[3];
  return r;
}
__device__ __noinline__ void store4f_slow(float* g, int n, float4 r) {
  if (n > 0) g[0] = r.x;
  if (n > 1) g[1] = r.y;
  if (n > 2) g[2] = r.z;
  if (n > 3) g[3] = r.w;
}

struct MaskRow {
  const uint8_t* p;
  int64_t cs;
  bool vec;
  __device__ __forceinline__ void init(const uint8_t* ptr, int64_t stride) {
    p = ptr; cs = stride;
    vec = ptr != nullptr && stride == 1 && (reinterpret_cast<uintptr_t>(ptr) & 7) == 0;
  }
  // eight mask bytes (bit 0 of each is the truth value) of keys j .. j + 7; n_in of them lie inside the row
  __device__ __forceinline__ uint2 load8(int j, int n_in) const {
    if (p == nullptr) return make_uint2(0u, 0u);
    if (vec && n_in == 8) {
      const uint2 w = *reinterpret_cast<const uint2*>(p + j);
      return make_uint2(w.x & 0x01010101u, w.y & 0x01010101u);
    }
    return mask_bytes_slow(p, cs, j, n_in);
  }
};

// Flags of a lane's eight keys after the first pass, one nibble per key: key v sits in byte v & 3, nibble v >> 2;
// bit 0 landmark, bit 1 last section, bit 2 bucket (landmark, last section, hidden or outside the row),
// bit 3 hidden without being landmark or last section.
__device__ __forceinline__ uint32_t nibble_flags(uint32_t t) {
  const uint32_t bucket = (t | (t >> 1) | (t >> 2) | ~(t >> 3)) & 0x01010101u;
  const uint32_t off = (t >> 2) & ~(t >> 1) & ~t & 0x01010101u;
  return (t & 0x03030303u) | (bucket << 2) | (off << 3);
}
#define LMK_KEY_FLAG(F, v, bit) ((((F) >> (8 * ((v) & 3) + 4 * ((v) >> 2) + (bit))) & 1u) != 0)

// Per (chunk, lane) record kept in shared memory.
//   flags: see nibble_flags
//   info:  c0 (13 bits) | landmarks in the lane << 13 (4 bits) | scan flags << 17 (6 bits) | dead << 23
struct Meta {
  uint32_t flags, info;
  __device__ __forceinline__ int c0() const { return (int)(info & 0x1fffu); }
  __device__ __forceinline__ int nlm() const { return (int)((info >> 13) & 15u); }
  __device__ __forceinline__ bool dead() const { return (info >> 23) & 1u; }
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Eight floats of one lane in the row buffer: two 16-byte accesses, conflict-free across the warp.
__device__ __forceinline__ void row_put(float* buf, int lane, const float (&x)[8]) {
  *reinterpret_cast<float4*>(buf + lane * 4) = make_float4(x[0], x[1], x[2], x[3]);
  *reinterpret_cast<float4*>(buf + 128 + lane * 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void row_get(const float* buf, int lane, float (&x)[8]) {
  float4 a = *reinterpret_cast<const float4*>(buf + lane * 4), b = *reinterpret_cast<const float4*>(buf + 128 + lane * 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void load8f(const float* g, bool vec, int n_in, float (&x)[8]) {
  float4 a, b;
  if (vec && n_in == 8) {
    a = *reinterpret_cast<const float4*>(g);
    b = *reinterpret_cast<const float4*>(g + 4);
  } else {
    a = load4f_slow(g, n_in);
    b = load4f_slow(g + 4, n_in - 4);
  }
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8f(float* g, bool vec, int n_in, const float (&x)[8]) {
  const float4 a = make_float4(x[0], x[1], x[2], x[3]), b = make_float4(x[4], x[5], x[6], x[7]);
  if (vec && n_in == 8) {
    *reinterpret_cast<float4*>(g) = a;
    *reinterpret_cast<float4*>(g + 4) = b;
  } else {
    store4f_slow(g, n_in, a);
    store4f_slow(g + 4, n_in - 4, b);
  }
}

// Copies the lane's keys of every chunk into the row buffer: asynchronously where the 16-byte pieces are aligned
// and wholly inside the row, with plain loads elsewhere (-inf beyond the row's end).  16-bit scores are parked in
// the upper half of the chunk's slot and widened by stage_get.
template <typename T>
__device__ __forceinline__ void stage_row(const T* x, int Lk, int n_chunks, int lane, float* xbuf) {
  const bool xvec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  // chunks in which this lane's eight keys lie wholly inside the row
  const int n_full = xvec ? max(Lk - lane * 8 - 8 + kFastChunk, 0) / kFastChunk : 0;
  {
    const T* src = x + lane * 8;
    uint32_t dst = (uint32_t)__cvta_generic_to_shared(xbuf + lane * 4);
    for (int k = 0; k < n_full; ++k) {
      if constexpr (sizeof(T) == 4) {
        cp_async16(dst, src);
        cp_async16(dst + 512, src + 4);
      } else {
        cp_async16(dst + 512, src);
      }
      src += kFastChunk;
      dst += kFastChunk * 4;
    }
  }
  for (int k = n_full; k < n_chunks; ++k) {
    const int j = k * kFastChunk + lane * 8;
    float* buf = xbuf + k * kFastChunk;
    float t[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) t[v] = j + v < Lk ? to_f32(x[j + v]) : -INFINITY;
    if constexpr (sizeof(T) == 4) {
      row_put(buf, lane, t);
    } else {                                  // park as 16-bit values, like the asynchronous copies
      T* e = reinterpret_cast<T*>(buf + 128 + lane * 4);
#pragma unroll
      for (int v = 0; v < 8; ++v) e[v] = from_f32<T>(t[v]);
    }
  }
}
template <typename T>
__device__ __forceinline__ void stage_get(float* buf, int lane, float (&x)[8]) {
  if constexpr (sizeof(T) == 4) {
    row_get(buf, lane, x);
  } else {
    uint4 w = *reinterpret_cast<const uint4*>(buf + 128 + lane * 4);
    const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
    for (int v = 0; v < 8; ++v) x[v] = to_f32(e[v]);
    row_put(buf, lane, x);                      // only this lane's own parked bytes are overwritten
  }
}

// Folds the per-lane partial results of one chunk into the per-group accumulators.  `head` covers the lane's keys in
// front of its first landmark (all of them if it has none) and belongs to group c0; `tail` covers the keys behind its
// last landmark and belongs to group c0 + nlm.  Groups that begin and end inside one lane were written by that lane.
// flags: bit s (s < 5) = step s of the segmented scan combines with the lane 2^s below, bit 5 = the lane ends a run
// of lanes whose last key lies in the same group.
template <bool kMax>
__device__ __forceinline__ void fold_chunk(float head, float tail, int nlm, int c0, uint32_t flags, float* acc, int G,
                                           int lane) {
  const int key = c0 + nlm;
  float v = nlm ? tail : head;
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    float u = __shfl_up_sync(0xffffffffu, v, 1 << s);
    if ((flags >> s) & 1u) v = kMax ? fmaxf(v, u) : v + u;
  }
  const float hn = __shfl_down_sync(0xffffffffu, head, 1);
  if (flags & 32u) {
    if (lane < 31) v = kMax ? fmaxf(v, hn) : v + hn;
    if (key < G) acc[key] = kMax ? fmaxf(acc[key], v) : acc[key] + v;
  }
  if (lane == 0 && nlm > 0 && c0 < G) acc[c0] = kMax ? fmaxf(acc[c0], head) : acc[c0] + head;
  __syncwarp();
}

template <typename T, bool kBackward, bool kCausal>
__global__ void __launch_bounds__(kGsWarps * 32) grouped_softmax_rows_kernel(GsParams p, int n_chunks) {
  extern __shared__ __align__(16) float gs_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = p.max_groups;
  const size_t per_warp = (size_t)n_chunks * (kFastChunk + 64) + 4 * (size_t)G;
  float* xbuf = gs_smem + warp * per_warp;
  Meta* meta = reinterpret_cast<Meta*>(xbuf + (size_t)n_chunks * kFastChunk) + lane;   // [chunk][lane]
  float* gmax = xbuf + (size_t)n_chunks * (kFastChunk + 64);
  float* gsum = gmax + G;
  float* gw = gsum + G;     // exp(landmark score - bucket max) of the landmark closing each group
  float* gc = gw + G;       // backward: sum over the group of inner prob * grad
  const int64_t row = (int64_t)blockIdx.x * kGsWarps + warp;
  const int64_t rows = (int64_t)p.B * p.H * p.Lq;
  if (row >= rows) return;
  uint32_t bh;                                      // B * H fits 32 bits
  int i;
  if (rows <= 0xffffffffLL) {
    bh = (uint32_t)row / (uint32_t)p.Lq;
    i = (int)((uint32_t)row - bh * (uint32_t)p.Lq);
  } else {
    bh = (uint32_t)(row / p.Lq);
    i = (int)(row - (int64_t)bh * p.Lq);
  }
  const int b = (int)(bh / (uint32_t)p.H);
  const int h = (int)(bh - (uint32_t)b * (uint32_t)p.H);
  const bool guards = p.guards != 0;

  const T* xrow = reinterpret_cast<const T*>(p.x) + b * p.xs[0] + h * p.xs[1] + i * p.xs[2];
  constexpr bool causal = kCausal;
  const int pi = i + p.Lk - p.Lq;                   // causal mode: the last key this query sees
  const int n_live = causal ? min(n_chunks, pi / kFastChunk + 1) : n_chunks;   // chunks with a visible key
  stage_row<T>(xrow, p.Lk, n_live, lane, xbuf);            // asynchronous copies, awaited below
  MaskRow mm, ml, mh;
  int p_last = -1;                                  // causal mode: the last landmark in front of key pi
  if (causal) {
    mm.init(p.row_flags + b * p.row_flags_stride, 1);
    ml.init(nullptr, 0);
    mh.init(nullptr, 0);
    for (int j0 = (max(pi - 1, 0) / kFastChunk) * kFastChunk; j0 >= 0 && p_last < 0; j0 -= kFastChunk) {
      const int j = j0 + lane * 8;
      const uint2 m = mm.load8(j, min(max(min(p.Lk, pi) - j, 0), 8));      // keys in front of pi only
      const uint64_t w = ((uint64_t)m.y << 32) | m.x;
      int best = w ? j + (63 - __clzll((long long)w)) / 8 : -1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
      p_last = best;
    }
  } else {
    mm.init(p.is_mem + b * p.ms[0] + h * p.ms[1] + i * p.ms[2], p.ms[3]);
    ml.init(p.last + b * p.ls[0] + h * p.ls[1] + i * p.ls[2], p.ls[3]);
    mh.init(p.hidden ? p.hidden + b * p.hs[0] + h * p.hs[1] + i * p.hs[2] : nullptr, p.hs[3]);
  }
  auto low_bytes = [](int n) -> uint64_t { return n >= 8 ? ~0ull : ((1ull << (8 * n)) - 1ull); };
  auto load_flags = [&](int k) -> RawFlags {
    const int j = k * kFastChunk + lane * 8;
    const int n_in = min(max(p.Lk - j, 0), 8);
    RawFlags f;
    if (causal) {
      constexpr uint64_t kOnes = 0x0101010101010101ull;
      const uint2 m = mm.load8(j, n_in);
      const uint64_t m64 = ((uint64_t)m.y << 32) | m.x;
      const uint64_t inside = kOnes & low_bytes(n_in);
      const uint64_t vis = inside & low_bytes(min(max(pi - j + 1, 0), 8));       // keys 0 .. pi
      const uint64_t front = kOnes & low_bytes(min(max(pi - j, 0), 8));           // keys in front of pi
      const uint64_t open = kOnes & ~low_bytes(min(max(p_last + 1 - j, 0), 8));   // keys behind the last landmark
      const uint64_t mem = m64 & vis & front;        // a landmark at pi itself is masked like a hidden key
      const uint64_t last = vis & ~m64 & open;
      const uint64_t hid = kOnes & ~(mem | last | (vis & ~m64));
      const uint64_t w = mem | (last << 1) | (hid << 2) | (inside << 3);
      f.lo = (uint32_t)w;
      f.hi = (uint32_t)(w >> 32);
      return f;
    }
    const uint2 m = mm.load8(j, n_in), l = ml.load8(j, n_in), hd = mh.load8(j, n_in);
    f.lo = m.x | (l.x << 1) | (hd.x << 2);
    f.hi = m.y | (l.y << 1) | (hd.y << 2);
    if (n_in == 8) {
      f.lo |= 0x08080808u;
      f.hi |= 0x08080808u;
    } else {                                    // keys beyond the row's end: hidden, outside
      const uint64_t inside = n_in ? (0x0808080808080808ull >> (8 * (8 - n_in))) : 0ull;
      const uint64_t w = (((uint64_t)f.hi << 32) | f.lo) | inside | (0x0404040404040404ull & ~(inside >> 1));
      f.lo = (uint32_t)w;
      f.hi = (uint32_t)(w >> 32);
    }
    return f;
  };

  const RawFlags raw0 = load_flags(0);              // under way while the row arrives
  for (int g = lane; g < G; g += 32) {
    gmax[g] = -INFINITY;
    gsum[g] = 0.f;
    gw[g] = 0.f;
    gc[g] = 0.f;
  }
  cp_async_wait_all();
  __syncwarp();

  // pass 1: decode the masks, count the landmarks, group and bucket maxima
  float bmax = -INFINITY;
  {
    int base = 0;
    RawFlags raw = raw0;
    for (int k = 0; k < n_chunks; ++k) {
      if (k >= n_live) {                            // causal mode: nothing visible from here on, nothing was read
        meta[k * 32] = Meta{0u, (uint32_t)base | (1u << 23)};
        continue;
      }
      RawFlags nraw = raw;
      if (k + 1 < n_live) nraw = load_flags(k + 1);
      float x[8];
      stage_get<T>(xbuf + k * kFastChunk, lane, x);
      if (causal && k == n_live - 1) {              // hidden scores count as -inf whatever the tensor holds
#pragma unroll
        for (int v = 0; v < 8; ++v)
          if (((v < 4 ? raw.lo : raw.hi) >> (8 * (v & 3) + 2)) & 1u) x[v] = -INFINITY;
        row_put(xbuf + k * kFastChunk, lane, x);
      }
      // all keys of the lane hidden, none a landmark or in the last section
      const bool shut = (raw.lo & raw.hi & 0x04040404u) == 0x04040404u && ((raw.lo | raw.hi) & 0x03030303u) == 0u;
      if (__all_sync(0xffffffffu, shut)) {
        bool inert = true;
#pragma unroll
        for (int v = 0; v < 8; ++v) inert = inert && x[v] == -INFINITY;
        if (__all_sync(0xffffffffu, inert)) {     // nothing finite either: the other passes skip the chunk
          meta[k * 32] = Meta{0u, (uint32_t)base | (1u << 23)};
          raw = nraw;
          continue;
        }
      }
      const uint32_t F = nibble_flags(raw.lo) | (nibble_flags(raw.hi) << 4);
      const int nlm = __popc(F & 0x11111111u);
      // landmarks in front of this lane's keys within the chunk
      const unsigned starts = __ballot_sync(0xffffffffu, nlm != 0);
      int c0;
      if (__ballot_sync(0xffffffffu, nlm > 1) == 0) {
        c0 = base + __popc(starts & ((1u << lane) - 1u));
        base += __popc(starts);
      } else {
        int inc = nlm;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int t = __shfl_up_sync(0xffffffffu, inc, o);
          if (lane >= o) inc += t;
        }
        c0 = base + inc - nlm;
        base += __shfl_sync(0xffffffffu, inc, 31);
      }
      // a lane holding a landmark begins a run of lanes whose last key lies in the same group
      const unsigned below = starts & ((2u << lane) - 1u);
      const int dist = lane - (below ? 31 - __clz(below) : 0);
      uint32_t flags = (1u << (32 - __clz(dist))) - 1u;
      if (lane == 31 || ((starts >> 1) >> lane) & 1u) flags |= 32u;

      float run = -INFINITY, head = -INFINITY;
      int c = c0;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        if (LMK_KEY_FLAG(F, v, 0)) {
          if (c == c0) head = run;
          else if (c < G) gmax[c] = fmaxf(gmax[c], run);
          run = -INFINITY;
          ++c;
        }
        const bool bk = LMK_KEY_FLAG(F, v, 2);           // keys outside the row hold -inf
        run = fmaxf(run, bk ? -INFINITY : x[v]);
        bmax = fmaxf(bmax, bk ? x[v] : -INFINITY);
      }
      meta[k * 32] = Meta{F, (uint32_t)c0 | ((uint32_t)nlm << 13) | (flags << 17)};
      fold_chunk<true>(nlm ? head : run, run, nlm, c0, flags, gmax, G, lane);
      raw = nraw;
    }
    if (lane == 0 && base >= G && p.status != nullptr) atomicCAS(p.status, 0, kErrSoftmaxGroups);
  }
  bmax = warp_max(bmax);
  if (guards && isinf(bmax)) bmax = 0.f;

  // stabiliser of group c; +inf beyond the last slot makes every exponential of such a group 0
  auto group_max = [&](int c) -> float {
    if (c >= G) return INFINITY;
    const float mx = gmax[c];
    return (guards && isinf(mx)) ? 0.f : mx;
  };

  // pass 2: exponentials (kept in the row buffer), group and bucket sums, landmark weights
  float bsum = 0.f;
  for (int k = 0; k < n_chunks; ++k) {
    const Meta mt = meta[k * 32];
    if (mt.dead()) continue;
    float x[8];
    row_get(xbuf + k * kFastChunk, lane, x);
    const uint32_t F = mt.flags;
    const int c0 = mt.c0();
    int c = c0;
    float mx = group_max(c);
    float run = 0.f, head = 0.f;
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const bool bk = LMK_KEY_FLAG(F, v, 2);
      const float ex = exp_diff(x[v], bk ? bmax : mx);     // keys beyond the row's end hold -inf
      x[v] = ex;
      bsum += bk ? ex : 0.f;
      run += bk ? 0.f : ex;
      if (LMK_KEY_FLAG(F, v, 0)) {
        if (c < G) gw[c] = ex;
        if (c == c0) head = run;
        else if (c < G) gsum[c] += run;
        run = 0.f;
        ++c;
        mx = group_max(c);
      }
    }
    row_put(xbuf + k * kFastChunk, lane, x);
    fold_chunk<false>(mt.nlm() ? head : run, run, mt.nlm(), c0, mt.info >> 17, gsum, G, lane);
  }
  bsum = warp_sum(bsum);
  const float binv = (guards && bsum < 0.5f) ? 0.f : 1.f / bsum;

  // scale of a non-bucket key of group c: its outer weight over its group's sum
  auto inv_den = [&](int c) -> float {
    if (c >= G) return 0.f;
    const float den = gsum[c];                      // 0 only for a group without keys: nothing is scaled by it
    return ((guards && den < 0.5f) || den == 0.f) ? 0.f : 1.f / den;
  };
  auto weight = [&](int c) -> float { return c < G ? gw[c] * binv : 0.f; };

  if (!kBackward) {
    float* out = p.probs + row * p.Lk;
    const bool ovec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    const float off = guards ? 0.f : binv * 0.f;    // bucket keys outside the last section (NaN if binv is not finite)
    const bool want_gp = p.group_prob != nullptr;
    float last_total = 0.f;
    for (int k = 0; k < n_chunks; ++k) {
      const Meta mt = meta[k * 32];
      const int j = k * kFastChunk + lane * 8;
      const int n_in = min(max(p.Lk - j, 0), 8);
      float x[8];
      if (mt.dead()) {
#pragma unroll
        for (int v = 0; v < 8; ++v) x[v] = 0.f * off;
        store8f(out + j, ovec, n_in, x);
        continue;
      }
      row_get(xbuf + k * kFastChunk, lane, x);
      const uint32_t F = mt.flags;
      int c = mt.c0();
      float sc = inv_den(c) * weight(c);
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const float s = LMK_KEY_FLAG(F, v, 1) ? binv : (LMK_KEY_FLAG(F, v, 2) ? off : sc);
        x[v] *= s;
        if (LMK_KEY_FLAG(F, v, 0)) {
          ++c;
          sc = inv_den(c) * weight(c);
        }
      }
      if (want_gp) {
#pragma unroll
        for (int v = 0; v < 8; ++v) last_total += LMK_KEY_FLAG(F, v, 1) ? x[v] : 0.f;
      }
      store8f(out + j, ovec, n_in, x);
    }
    if (want_gp) {
      last_total = warp_sum(last_total);
      float* gp = p.group_prob + row * p.max_mem_cnt;
      for (int g = lane; g < p.max_mem_cnt - 1; g += 32) gp[g] = g < G ? gw[g] * binv : 0.f;
      if (lane == 0) gp[p.max_mem_cnt - 1] = last_total;
    }
  } else {
    const float* gr = p.gprobs + row * p.Lk;
    float* out = p.gx + row * p.Lk;
    const bool gvec = (reinterpret_cast<uintptr_t>(gr) & 15) == 0;
    const bool ovec = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    // pass 3: c_g = sum_j inner_j * grad_j per group, total = sum_j P_j * grad_j over the row
    float total = 0.f;
    // the gradients of the next live chunk are requested before the current one is worked on
    auto load_grad = [&](int k, float (&g)[8]) {
      const int j = k * kFastChunk + lane * 8;
      load8f(gr + j, gvec, min(max(p.Lk - j, 0), 8), g);
    };
    Meta mnext = meta[0];
    float gn[8];
    if (!mnext.dead()) load_grad(0, gn);
    for (int k = 0; k < n_chunks; ++k) {
      const Meta mt = mnext;
      float x[8], g[8];
#pragma unroll
      for (int v = 0; v < 8; ++v) g[v] = gn[v];
      if (k + 1 < n_chunks) {
        mnext = meta[(k + 1) * 32];
        if (!mnext.dead()) load_grad(k + 1, gn);
      }
      if (mt.dead()) continue;
      row_get(xbuf + k * kFastChunk, lane, x);
      const uint32_t F = mt.flags;
      const int c0 = mt.c0();
      int c = c0;
      float id = inv_den(c), wt = weight(c);
      float run = 0.f, head = 0.f, lsum = 0.f;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const float xg = x[v] * g[v];
        lsum += LMK_KEY_FLAG(F, v, 1) ? xg : 0.f;
        run += LMK_KEY_FLAG(F, v, 2) ? 0.f : xg;
        if (LMK_KEY_FLAG(F, v, 0)) {
          run *= id;
          total += run * wt;
          if (c == c0) head = run;
          else if (c < G) gc[c] += run;
          run = 0.f;
          ++c;
          id = inv_den(c);
          wt = weight(c);
        }
      }
      run *= id;
      total += run * wt + lsum * binv;
      fold_chunk<false>(mt.nlm() ? head : run, run, mt.nlm(), c0, mt.info >> 17, gc, G, lane);
    }
    total = warp_sum(total);
    // pass 4: gradients
    mnext = meta[0];
    if (!mnext.dead()) load_grad(0, gn);
    for (int k = 0; k < n_chunks; ++k) {
      const Meta mt = mnext;
      const int j = k * kFastChunk + lane * 8;
      const int n_in = min(max(p.Lk - j, 0), 8);
      float x[8], g[8];
#pragma unroll
      for (int v = 0; v < 8; ++v) g[v] = gn[v];
      if (k + 1 < n_chunks) {
        mnext = meta[(k + 1) * 32];
        if (!mnext.dead()) load_grad(k + 1, gn);
      }
      if (mt.dead()) {
#pragma unroll
        for (int v = 0; v < 8; ++v) x[v] = 0.f;
        store8f(out + j, ovec, n_in, x);
        continue;
      }
      row_get(xbuf + k * kFastChunk, lane, x);
      const uint32_t F = mt.flags;
      int c = mt.c0();
      float sc = inv_den(c) * weight(c), cg = c < G ? gc[c] : 0.f;
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const bool bk = LMK_KEY_FLAG(F, v, 2), is_last = LMK_KEY_FLAG(F, v, 1);
        // bucket: P_j * ((g_j if last section) - total); group member: P_j * (g_j - c_g)
        const float s = bk ? (LMK_KEY_FLAG(F, v, 3) ? 0.f : binv) : sc;
        const float a = (bk && !is_last) ? 0.f : g[v];
        float dx = x[v] * s * (a - (bk ? total : cg));
        if (LMK_KEY_FLAG(F, v, 0)) {                 // a landmark also receives its group's c_g
          dx = x[v] * binv * ((is_last ? g[v] : 0.f) + cg - total);
          ++c;
          sc = inv_den(c) * weight(c);
          cg = c < G ? gc[c] : 0.f;
        }
        x[v] = dx;
      }
      store8f(out + j, ovec, n_in, x);
    }
  }
}
#undef LMK_KEY_FLAG

static size_t fast_smem_bytes(int Lk, int max_groups) {
  const size_t n_chunks = (size_t)(Lk + kFastChunk - 1) / kFastChunk;
  return sizeof(float) * kGsWarps * (n_chunks * (kFastChunk + 64) + 4 * (size_t)max_groups);
}

template <bool kBackward>
int launch(const GsParams& p, int dtype, cudaStream_t st) {
  const int64_t rows = (int64_t)p.B * p.H * p.Lq;
  if (rows == 0 || p.Lk == 0) return LMK_OK;
  GsParams& pw = const_cast<GsParams&>(p);
  pw.status = device_status_word();
  unsigned grid = (unsigned)((rows + kGsWarps - 1) / kGsWarps);
  const bool fast = p.Lk <= kFastMaxLk && fast_smem_bytes(p.Lk, p.max_groups) <= kFastMaxSmem;
  if (p.causal && !fast)
    return fail(LMK_ERR_UNSUPPORTED, "grouped_softmax_causal: rows of %d keys with %d groups do not fit the row kernel "
                                     "(at most %d keys); build the masks and use lmk_grouped_softmax_fwd", p.Lk,
                p.max_groups, kFastMaxLk);
  const int n_chunks = (p.Lk + kFastChunk - 1) / kFastChunk;
  size_t smem = fast ? fast_smem_bytes(p.Lk, p.max_groups) : sizeof(float) * 4 * (size_t)p.max_groups * kGsWarps;
#define LMK_GS_LAUNCH(T)                                                                                     \
  do {                                                                                                       \
    if (fast && p.causal) {                                                                                  \
      LMK_CUDA(cudaFuncSetAttribute(grouped_softmax_rows_kernel<T, kBackward, true>,                         \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
      grouped_softmax_rows_kernel<T, kBackward, true><<<grid, kGsWarps * 32, smem, st>>>(p, n_chunks);       \
    } else if (fast) {                                                                                       \
      LMK_CUDA(cudaFuncSetAttribute(grouped_softmax_rows_kernel<T, kBackward, false>,                        \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
      grouped_softmax_rows_kernel<T, kBackward, false><<<grid, kGsWarps * 32, smem, st>>>(p, n_chunks);      \
    } else {                                                                                                 \
      LMK_CUDA(cudaFuncSetAttribute(grouped_softmax_kernel<T, kBackward>,                                    \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                \
      grouped_softmax_kernel<T, kBackward><<<grid, kGsWarps * 32, smem, st>>>(p);                            \
    }                                                                                                        \
  } while (0)
  if (dtype == LMK_F32) LMK_GS_LAUNCH(float);
  else if (dtype == LMK_F16) LMK_GS_LAUNCH(__half);
  else LMK_GS_LAUNCH(__nv_bfloat16);
#undef LMK_GS_LAUNCH
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

int fill(GsParams& p, const void* x, const int64_t* xs, const uint8_t* is_mem, const int64_t* ms,
         const uint8_t* last, const int64_t* ls, const uint8_t* hidden, const int64_t* hs, int B, int H, int Lq,
         int Lk, int dtype, int guards, int max_groups) {
  LMK_CHECK_ARG(x && is_mem && last && xs && ms && ls, "grouped_softmax: null pointer");
  LMK_CHECK_ARG(!hidden || hs, "grouped_softmax: hidden mask without strides");
  LMK_CHECK_ARG(B >= 0 && H >= 0 && Lq >= 0 && Lk >= 0, "grouped_softmax: negative dimension");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "grouped_softmax: bad dtype %d", dtype);
  LMK_CHECK_ARG(max_groups >= 1 && max_groups <= 2048, "grouped_softmax: max_groups %d outside [1, 2048]", max_groups);
  p.x = x;
  p.is_mem = is_mem; p.last = last; p.hidden = hidden;
  for (int i = 0; i < 3; ++i) p.xs[i] = xs[i];
  for (int i = 0; i < 4; ++i) {
    p.ms[i] = ms[i];
    p.ls[i] = ls[i];
    p.hs[i] = hidden ? hs[i] : 0;
  }
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.guards = guards; p.max_groups = max_groups;
  return LMK_OK;
}

}  // namespace
}  // namespace lmk

extern "C" int lmk_grouped_softmax_fwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem,
                                       const int64_t is_mem_strides[4], const uint8_t* last_section,
                                       const int64_t last_strides[4], const uint8_t* hidden,
                                       const int64_t hidden_strides[4], float* probs, float* group_prob,
                                       int max_mem_cnt, int B, int H, int Lq, int Lk, int dtype, int guards,
                                       int max_groups, void* stream) {
  lmk::GsParams p{};
  int rc = lmk::fill(p, x, x_strides, is_mem, is_mem_strides, last_section, last_strides, hidden, hidden_strides,
                     B, H, Lq, Lk, dtype, guards, max_groups);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(probs != nullptr, "grouped_softmax_fwd: probs is null");
  LMK_CHECK_ARG(group_prob == nullptr || max_mem_cnt >= 2, "grouped_softmax_fwd: max_mem_cnt must be >= 2");
  p.probs = probs;
  p.group_prob = group_prob;
  p.max_mem_cnt = max_mem_cnt;
  return lmk::launch<false>(p, dtype, (cudaStream_t)stream);
}

extern "C" int lmk_grouped_softmax_bwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem,
                                       const int64_t is_mem_strides[4], const uint8_t* last_section,
                                       const int64_t last_strides[4], const uint8_t* hidden,
                                       const int64_t hidden_strides[4], const float* grad_probs, float* grad_x,
                                       int B, int H, int Lq, int Lk, int dtype, int guards, int max_groups,
                                       void* stream) {
  lmk::GsParams p{};
  int rc = lmk::fill(p, x, x_strides, is_mem, is_mem_strides, last_section, last_strides, hidden, hidden_strides,
                     B, H, Lq, Lk, dtype, guards, max_groups);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(grad_probs && grad_x, "grouped_softmax_bwd: null gradient pointer");
  p.gprobs = grad_probs;
  p.gx = grad_x;
  return lmk::launch<true>(p, dtype, (cudaStream_t)stream);
}

// Mask block + grouped softmax of the lm_benchmark call site (lm_benchmark/models/landmark.py:210-232) from one flag
// per (batch row, key): query i sees keys 0 .. i + Lk - Lq; hidden scores count as -inf.
static int fill_causal(lmk::GsParams& p, const void* x, const int64_t* xs, const uint8_t* is_mem_row, int64_t row_stride,
                       int B, int H, int Lq, int Lk, int dtype, int max_groups) {
  LMK_CHECK_ARG(x && xs && is_mem_row, "grouped_softmax_causal: null pointer");
  LMK_CHECK_ARG(B >= 0 && H >= 0 && Lq >= 0 && Lk >= Lq, "grouped_softmax_causal: need Lk >= Lq >= 0");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "grouped_softmax_causal: bad dtype %d", dtype);
  LMK_CHECK_ARG(max_groups >= 1 && max_groups <= 2048, "grouped_softmax_causal: max_groups %d outside [1, 2048]", max_groups);
  p.x = x;
  for (int i = 0; i < 3; ++i) p.xs[i] = xs[i];
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.guards = 1; p.max_groups = max_groups;
  p.row_flags = is_mem_row; p.row_flags_stride = row_stride; p.causal = 1;
  return LMK_OK;
}

extern "C" int lmk_grouped_softmax_causal_fwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem_row,
                                              int64_t is_mem_stride, float* probs, int B, int H, int Lq, int Lk,
                                              int dtype, int max_groups, void* stream) {
  lmk::GsParams p{};
  int rc = fill_causal(p, x, x_strides, is_mem_row, is_mem_stride, B, H, Lq, Lk, dtype, max_groups);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(probs != nullptr, "grouped_softmax_causal_fwd: probs is null");
  p.probs = probs;
  return lmk::launch<false>(p, dtype, (cudaStream_t)stream);
}

extern "C" int lmk_grouped_softmax_causal_bwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem_row,
                                              int64_t is_mem_stride, const float* grad_probs, float* grad_x, int B,
                                              int H, int Lq, int Lk, int dtype, int max_groups, void* stream) {
  lmk::GsParams p{};
  int rc = fill_causal(p, x, x_strides, is_mem_row, is_mem_stride, B, H, Lq, Lk, dtype, max_groups);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(grad_probs && grad_x, "grouped_softmax_causal_bwd: null gradient pointer");
  p.gprobs = grad_probs;
  p.gx = grad_x;
  return lmk::launch<true>(p, dtype, (cudaStream_t)stream);
}
