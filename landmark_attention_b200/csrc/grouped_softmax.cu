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
};

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

template <bool kBackward>
int launch(const GsParams& p, int dtype, cudaStream_t st) {
  const int64_t rows = (int64_t)p.B * p.H * p.Lq;
  if (rows == 0 || p.Lk == 0) return LMK_OK;
  size_t smem = sizeof(float) * 4 * (size_t)p.max_groups * kGsWarps;
  unsigned grid = (unsigned)((rows + kGsWarps - 1) / kGsWarps);
#define LMK_GS_LAUNCH(T)                                                                                     \
  do {                                                                                                       \
    LMK_CUDA(cudaFuncSetAttribute(grouped_softmax_kernel<T, kBackward>,                                      \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                  \
    grouped_softmax_kernel<T, kBackward><<<grid, kGsWarps * 32, smem, st>>>(p);                              \
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
