// Write side of the landmark block cache: append whole blocks of un-rotated keys / values to a (ring) block cache of
// any layout and, in the same pass, copy every block's landmark key (its last row) into a dense [B, H, capacity, D]
// array, so that scoring reads 1/block of the key bytes contiguously instead of one strided row per block.
//
// Reference: MemLMCacheStorage.store_in_cache (lm_benchmark/models/caches/mem_cache.py:111-158), which writes the
// ring buffer [B, capacity, block, H, D] with tensor copies and keeps no separate landmark array.
//
// lmk_chunk_prepare is the read-side counterpart for one chunk of a LLaMA layer: rotary position embedding of the
// chunk's queries and keys (llama/llama_mem.py:127-149: x * cos + rotate_half(x) * sin in the tensors' 16-bit type),
// zero-padded copies in whole 128-row tiles for the tensor-core attention, the landmark flags of the padded rows, and
// the append of the un-rotated keys / values to a preallocated cache (:424-425) -- one launch instead of the
// index / multiply / concatenate / copy kernels of the tensor-library formulation.
#include "common.cuh"

namespace lmk {
namespace {

template <typename T> struct Pair16;      // arithmetic on two 16-bit values held in one 32-bit register
template <> struct Pair16<__nv_bfloat16> {
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
};
template <> struct Pair16<__half> {
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
};

// x * cos + rotate_half(x) * sin on one 16-byte vector of the low half (lo) and its partner of the high half (hi),
// with the three roundings of the tensor formulation (two products, one sum).
template <typename T>
__device__ __forceinline__ void rotate_half_pair(uint4& lo, uint4& hi, const uint4& cl, const uint4& ch, const uint4& sl,
                                                 const uint4& sh) {
  const uint32_t* l = reinterpret_cast<const uint32_t*>(&lo);
  const uint32_t* h = reinterpret_cast<const uint32_t*>(&hi);
  const uint32_t *c0 = reinterpret_cast<const uint32_t*>(&cl), *c1 = reinterpret_cast<const uint32_t*>(&ch);
  const uint32_t *s0 = reinterpret_cast<const uint32_t*>(&sl), *s1 = reinterpret_cast<const uint32_t*>(&sh);
  uint32_t ol[4], oh[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {        // rotate_half(x) = (-x[d + D/2], x[d])
    ol[u] = Pair16<T>::add(Pair16<T>::mul(l[u], c0[u]), Pair16<T>::mul(h[u] ^ 0x80008000u, s0[u]));
    oh[u] = Pair16<T>::add(Pair16<T>::mul(h[u], c1[u]), Pair16<T>::mul(l[u], s1[u]));
  }
  lo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
  hi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
}

struct PrepParams {
  const void *q, *k, *v;
  int64_t qs[3], ks[3], vs[3];          // element strides {batch, head, row}
  const void *cos_t, *sin_t;
  int n_pos;
  int64_t pos0;
  const uint8_t* chunk_flags;
  int block;
  void *q_rot, *q_pad, *k_pad, *v_pad;
  uint8_t* flags_pad;
  void *cache_k, *cache_v;
  int64_t cs[3];                        // cache element strides {batch, head, row}
  int64_t cache_pos;
  int H, T, t_pad, D;
};

// 16-bit types; D / 16 threads per row, each owning one vector of the low half and its partner of the high half.
template <typename T>
__global__ void __launch_bounds__(128) chunk_prepare_kernel(PrepParams p) {
  const int lp = p.D / 16;                         // threads per row
  const int rows_per_cta = 128 / lp;
  const int t = blockIdx.x * rows_per_cta + threadIdx.x / lp;
  const int sub = threadIdx.x % lp, d0 = sub * 8, half = p.D / 2;
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  if (threadIdx.x >= rows_per_cta * lp || t >= p.t_pad) return;
  auto vec = [](const void* base, int64_t off) { return *reinterpret_cast<const uint4*>(static_cast<const T*>(base) + off); };
  auto put = [](void* base, int64_t off, const uint4& w) { *reinterpret_cast<uint4*>(static_cast<T*>(base) + off) = w; };
  const int64_t pad_off = ((int64_t)bh * p.t_pad + t) * p.D + d0;
  if (t >= p.T) {                                  // padding rows of the tiles
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    put(p.q_pad, pad_off, z); put(p.q_pad, pad_off + half, z);
    put(p.k_pad, pad_off, z); put(p.k_pad, pad_off + half, z);
    put(p.v_pad, pad_off, z); put(p.v_pad, pad_off + half, z);
    if (h == 0 && sub == 0) p.flags_pad[(int64_t)b * p.t_pad + t] = 0;
    return;
  }
  const int64_t pos = min(p.pos0 + t, (int64_t)p.n_pos - 1);
  const int64_t qo = b * p.qs[0] + h * p.qs[1] + t * p.qs[2] + d0;
  const int64_t ko = b * p.ks[0] + h * p.ks[1] + t * p.ks[2] + d0;
  const int64_t vo = b * p.vs[0] + h * p.vs[1] + t * p.vs[2] + d0;
  uint4 ql = vec(p.q, qo), qh = vec(p.q, qo + half);
  uint4 kl = vec(p.k, ko), kh = vec(p.k, ko + half);
  const uint4 vl = vec(p.v, vo), vh = vec(p.v, vo + half);
  const uint4 cl = vec(p.cos_t, pos * p.D + d0), ch = vec(p.cos_t, pos * p.D + d0 + half);
  const uint4 sl = vec(p.sin_t, pos * p.D + d0), sh = vec(p.sin_t, pos * p.D + d0 + half);
  if (p.cache_k != nullptr) {                      // the cache keeps un-rotated keys
    const int64_t co = b * p.cs[0] + h * p.cs[1] + (p.cache_pos + t) * p.cs[2] + d0;
    put(p.cache_k, co, kl); put(p.cache_k, co + half, kh);
    put(p.cache_v, co, vl); put(p.cache_v, co + half, vh);
  }
  rotate_half_pair<T>(ql, qh, cl, ch, sl, sh);
  rotate_half_pair<T>(kl, kh, cl, ch, sl, sh);
  const int64_t rot_off = ((int64_t)bh * p.T + t) * p.D + d0;
  put(p.q_rot, rot_off, ql); put(p.q_rot, rot_off + half, qh);
  put(p.q_pad, pad_off, ql); put(p.q_pad, pad_off + half, qh);
  put(p.k_pad, pad_off, kl); put(p.k_pad, pad_off + half, kh);
  put(p.v_pad, pad_off, vl); put(p.v_pad, pad_off + half, vh);
  if (h == 0 && sub == 0)
    p.flags_pad[(int64_t)b * p.t_pad + t] =
        p.chunk_flags != nullptr ? (p.chunk_flags[t] != 0) : ((p.pos0 + t) % p.block == p.block - 1);
}

// One CTA per (block to store, batch*head); 16-byte vectors, rows spread over the threads.
__global__ void __launch_bounds__(128) cache_store_kernel(const uint4* __restrict__ k_src, const uint4* __restrict__ v_src,
                                                          int64_t src_b, int64_t src_h, int64_t src_row,
                                                          uint4* __restrict__ k_dst, uint4* __restrict__ v_dst,
                                                          lmk_cache_desc kd, lmk_cache_desc vd,
                                                          uint4* __restrict__ lm_dst, int64_t lm_b, int64_t lm_h,
                                                          int64_t lm_block, int H, int first_slot, int capacity,
                                                          int vec_per_row) {
  const int i = blockIdx.x, bh = blockIdx.y;
  const int b = bh / H, h = bh - b * H;
  const int blk = kd.block;
  int slot = first_slot + i;
  if (slot >= capacity) slot -= capacity;
  const int64_t s0 = b * src_b + h * src_h + (int64_t)i * blk * src_row;
  const int64_t kd0 = b * kd.stride_b + h * kd.stride_h + (int64_t)slot * kd.stride_block;
  const int64_t vd0 = b * vd.stride_b + h * vd.stride_h + (int64_t)slot * vd.stride_block;
  const int total = blk * vec_per_row;
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    const int r = e / vec_per_row, c = e - r * vec_per_row;
    const uint4 kv = k_src[s0 + (int64_t)r * src_row + c];
    const uint4 vv = v_src[s0 + (int64_t)r * src_row + c];
    k_dst[kd0 + (int64_t)r * kd.stride_row + c] = kv;
    v_dst[vd0 + (int64_t)r * vd.stride_row + c] = vv;
    if (lm_dst != nullptr && r == blk - 1) lm_dst[b * lm_b + h * lm_h + (int64_t)slot * lm_block + c] = kv;
  }
}


// Rotary position embedding of a [B,H,T,D] tensor pair (queries and keys of one layer) in one launch, both rotary
// flavours, forward or inverse (the inverse rotation is the gradient of the forward one).  16-bit types use packed
// arithmetic with the three roundings of the tensor formulation x * cos + rotate(x) * sin.
struct RotParams {
  const void* in[2];
  void* out[2];
  int64_t st[2][3];                     // element strides {batch, head, row} of the inputs; outputs are dense
  const void *cos_t, *sin_t;
  int n_pos;
  int64_t pos0;
  int mode, inverse, n_tensors;
  int H, T, D;
};

template <typename T>
__global__ void __launch_bounds__(256) rotary_pair_kernel(RotParams p) {
  constexpr int VEC = 16 / sizeof(T);
  const int vpr = p.D / VEC;                                 // vectors per row
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (int64_t)p.T * vpr) return;
  const int t = (int)(e / vpr), c = (int)(e - (int64_t)t * vpr);
  const int bh = blockIdx.y, b = bh / p.H, h = bh - b * p.H;
  const int64_t pos = min(p.pos0 + t, (int64_t)p.n_pos - 1);
  const int half = p.D / 2;
  // the partner elements: interleaved pairs live in the same vector; rotate-half pairs d with d +- D/2
  const bool lower = c * VEC < half;
  const int pc = p.mode == LMK_ROTARY_HALF ? (lower ? c + vpr / 2 : c - vpr / 2) : c;
  const uint4 cs = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.cos_t) + pos * p.D + c * VEC);
  uint4 sn = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.sin_t) + pos * p.D + c * VEC);
  for (int i = 0; i < p.n_tensors; ++i) {
    const T* src = static_cast<const T*>(p.in[i]) + b * p.st[i][0] + h * p.st[i][1] + t * p.st[i][2];
    const uint4 x = *reinterpret_cast<const uint4*>(src + c * VEC);
    const uint4 y = *reinterpret_cast<const uint4*>(src + pc * VEC);
    uint4 o;
    if constexpr (sizeof(T) == 2) {
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&x);
      const uint32_t* yw = reinterpret_cast<const uint32_t*>(&y);
      const uint32_t *cw = reinterpret_cast<const uint32_t*>(&cs), *sw = reinterpret_cast<const uint32_t*>(&sn);
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t rot;                   // rotate(x) at this position
        if (p.mode == LMK_ROTARY_HALF) rot = lower ? (yw[u] ^ 0x80008000u) : yw[u];
        else rot = __byte_perm(xw[u], xw[u], 0x1032) ^ 0x00008000u;       // (x0, x1) -> (-x1, x0)
        const uint32_t s = p.inverse ? (sw[u] ^ 0x80008000u) : sw[u];
        ow[u] = Pair16<T>::add(Pair16<T>::mul(xw[u], cw[u]), Pair16<T>::mul(rot, s));
      }
    } else {
      const float* xf = reinterpret_cast<const float*>(&x);
      const float* yf = reinterpret_cast<const float*>(&y);
      const float *cf = reinterpret_cast<const float*>(&cs), *sf = reinterpret_cast<const float*>(&sn);
      float* of = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float rot;
        if (p.mode == LMK_ROTARY_HALF) rot = lower ? -yf[u] : yf[u];
        else rot = (u & 1) ? xf[u - 1] : -xf[u + 1];
        const float s = p.inverse ? -sf[u] : sf[u];
        of[u] = xf[u] * cf[u] + rot * s;
      }
    }
    *reinterpret_cast<uint4*>(static_cast<T*>(p.out[i]) + (((int64_t)bh * p.T + t) * p.D) + c * VEC) = o;
  }
}

}  // namespace
}  // namespace lmk

extern "C" int lmk_cache_store(const void* k_src, const void* v_src, const int64_t src_strides[3], void* k_cache,
                               void* v_cache, const lmk_cache_desc* kdesc, const lmk_cache_desc* vdesc,
                               void* landmark_keys, const int64_t landmark_strides[3], int B, int H, int n_store,
                               int first_slot, int capacity, int D, int dtype, void* stream) {
  using namespace lmk;
  LMK_CHECK_ARG(k_src && v_src && k_cache && v_cache && kdesc && vdesc && src_strides, "cache_store: null pointer");
  LMK_CHECK_ARG(landmark_keys == nullptr || landmark_strides != nullptr, "cache_store: landmark array without strides");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "cache_store: unknown dtype %d", dtype);
  LMK_CHECK_ARG(B >= 0 && H >= 1 && D >= 1 && n_store >= 0, "cache_store: bad shape");
  LMK_CHECK_ARG(kdesc->block >= 1 && kdesc->block == vdesc->block, "cache_store: block sizes must agree and be positive");
  LMK_CHECK_ARG(capacity >= 1 && first_slot >= 0 && first_slot < capacity && n_store <= capacity,
                "cache_store: slots %d..+%d do not fit a ring of %d blocks", first_slot, n_store, capacity);
  const int vec = dtype == LMK_F32 ? 4 : 8;
  LMK_CHECK_ARG(D % vec == 0, "cache_store: D=%d must be a multiple of %d elements (16 bytes)", D, vec);
  const int64_t* ss = src_strides;
  auto aligned = [&](int64_t s) { return s % vec == 0; };
  LMK_CHECK_ARG(aligned(ss[0]) && aligned(ss[1]) && aligned(ss[2]), "cache_store: source strides must be multiples of %d", vec);
  for (const lmk_cache_desc* d : {kdesc, vdesc})
    LMK_CHECK_ARG(aligned(d->stride_b) && aligned(d->stride_h) && aligned(d->stride_block) && aligned(d->stride_row),
                  "cache_store: cache strides must be multiples of %d elements", vec);
  LMK_CHECK_ARG((((uintptr_t)k_src | (uintptr_t)v_src | (uintptr_t)k_cache | (uintptr_t)v_cache |
                  (uintptr_t)landmark_keys) & 15) == 0, "cache_store: pointers must be 16-byte aligned");
  if (landmark_keys)
    LMK_CHECK_ARG(aligned(landmark_strides[0]) && aligned(landmark_strides[1]) && aligned(landmark_strides[2]),
                  "cache_store: landmark array strides must be multiples of %d", vec);
  if (B == 0 || n_store == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "cache_store: grid too large");
  // strides in units of 16-byte vectors
  lmk_cache_desc kd = *kdesc, vd = *vdesc;
  for (lmk_cache_desc* d : {&kd, &vd}) {
    d->stride_b /= vec; d->stride_h /= vec; d->stride_block /= vec; d->stride_row /= vec;
  }
  dim3 grid(n_store, B * H);
  cache_store_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      (const uint4*)k_src, (const uint4*)v_src, ss[0] / vec, ss[1] / vec, ss[2] / vec, (uint4*)k_cache, (uint4*)v_cache,
      kd, vd, (uint4*)landmark_keys, landmark_keys ? landmark_strides[0] / vec : 0,
      landmark_keys ? landmark_strides[1] / vec : 0, landmark_keys ? landmark_strides[2] / vec : 0, H, first_slot,
      capacity, D / vec);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_chunk_prepare(const void* q, const void* k, const void* v, const int64_t q_strides[3],
                                 const int64_t k_strides[3], const int64_t v_strides[3], const void* cos_table,
                                 const void* sin_table, int n_pos, int64_t pos0, const uint8_t* chunk_flags, int block,
                                 void* q_rot, void* q_pad, void* k_pad, void* v_pad, uint8_t* flags_pad, void* cache_k,
                                 void* cache_v, const int64_t cache_strides[3], int64_t cache_pos, int B, int H, int T,
                                 int t_pad, int D, int dtype, void* stream) {
  using namespace lmk;
  LMK_CHECK_ARG(q && k && v && q_strides && k_strides && v_strides && cos_table && sin_table && q_rot && q_pad &&
                    k_pad && v_pad && flags_pad, "chunk_prepare: null pointer");
  LMK_CHECK_ARG(dtype == LMK_F16 || dtype == LMK_BF16, "chunk_prepare: 16-bit types only (dtype %d)", dtype);
  LMK_CHECK_ARG(B >= 0 && H >= 1 && T >= 1 && t_pad >= T, "chunk_prepare: bad shape");
  LMK_CHECK_ARG(D >= 16 && D <= 2048 && D % 16 == 0 && 128 % (D / 16) == 0,
                "chunk_prepare: head dim %d must be 16, 32, 64, 128, ... with D / 16 dividing 128", D);
  LMK_CHECK_ARG(n_pos >= 1 && pos0 >= 0 && block >= 1, "chunk_prepare: bad positions");
  LMK_CHECK_ARG((cache_k == nullptr) == (cache_v == nullptr), "chunk_prepare: cache_k and cache_v go together");
  LMK_CHECK_ARG(cache_k == nullptr || (cache_strides != nullptr && cache_pos >= 0), "chunk_prepare: cache strides missing");
  uintptr_t align = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)cos_table | (uintptr_t)sin_table |
                    (uintptr_t)q_rot | (uintptr_t)q_pad | (uintptr_t)k_pad | (uintptr_t)v_pad | (uintptr_t)cache_k |
                    (uintptr_t)cache_v;
  LMK_CHECK_ARG((align & 15) == 0, "chunk_prepare: pointers must be 16-byte aligned");
  for (int i = 0; i < 3; ++i) {
    LMK_CHECK_ARG(q_strides[i] % 8 == 0 && k_strides[i] % 8 == 0 && v_strides[i] % 8 == 0,
                  "chunk_prepare: strides must be multiples of 8 elements");
    LMK_CHECK_ARG(cache_k == nullptr || cache_strides[i] % 8 == 0, "chunk_prepare: cache strides must be multiples of 8");
  }
  if (B == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "chunk_prepare: grid too large");
  PrepParams p{};
  p.q = q; p.k = k; p.v = v;
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = q_strides[i]; p.ks[i] = k_strides[i]; p.vs[i] = v_strides[i];
    p.cs[i] = cache_k ? cache_strides[i] : 0;
  }
  p.cos_t = cos_table; p.sin_t = sin_table; p.n_pos = n_pos; p.pos0 = pos0;
  p.chunk_flags = chunk_flags; p.block = block;
  p.q_rot = q_rot; p.q_pad = q_pad; p.k_pad = k_pad; p.v_pad = v_pad; p.flags_pad = flags_pad;
  p.cache_k = cache_k; p.cache_v = cache_v; p.cache_pos = cache_pos;
  p.H = H; p.T = T; p.t_pad = t_pad; p.D = D;
  const int rows_per_cta = 128 / (D / 16);
  dim3 grid((t_pad + rows_per_cta - 1) / rows_per_cta, B * H);
  if (dtype == LMK_BF16) chunk_prepare_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  else chunk_prepare_kernel<__half><<<grid, 128, 0, (cudaStream_t)stream>>>(p);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

extern "C" int lmk_rotary_apply(const void* q, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
                                const void* cos_table, const void* sin_table, int n_pos, int64_t pos0, int rotary,
                                int inverse, void* q_out, void* k_out, int B, int H, int T, int D, int dtype,
                                void* stream) {
  using namespace lmk;
  LMK_CHECK_ARG(q && q_strides && q_out && cos_table && sin_table, "rotary_apply: null pointer");
  LMK_CHECK_ARG((k == nullptr) == (k_out == nullptr) && (k == nullptr || k_strides != nullptr),
                "rotary_apply: k, k_strides and k_out go together");
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "rotary_apply: bad dtype %d", dtype);
  LMK_CHECK_ARG(rotary == LMK_ROTARY_HALF || rotary == LMK_ROTARY_INTERLEAVED, "rotary_apply: bad rotary mode %d", rotary);
  const int vec = dtype == LMK_F32 ? 4 : 8;
  LMK_CHECK_ARG(B >= 0 && H >= 1 && T >= 0 && D >= 2 * vec && D % (2 * vec) == 0,
                "rotary_apply: head dim %d must be a multiple of %d", D, 2 * vec);
  LMK_CHECK_ARG(n_pos >= 1 && pos0 >= 0, "rotary_apply: bad positions");
  uintptr_t align = (uintptr_t)q | (uintptr_t)k | (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)cos_table |
                    (uintptr_t)sin_table;
  LMK_CHECK_ARG((align & 15) == 0, "rotary_apply: pointers must be 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    LMK_CHECK_ARG(q_strides[i] % vec == 0 && (k == nullptr || k_strides[i] % vec == 0),
                  "rotary_apply: strides must be multiples of %d elements", vec);
  if (B == 0 || T == 0) return LMK_OK;
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "rotary_apply: grid too large");
  RotParams p{};
  p.in[0] = q; p.in[1] = k; p.out[0] = q_out; p.out[1] = k_out;
  for (int i = 0; i < 3; ++i) {
    p.st[0][i] = q_strides[i];
    p.st[1][i] = k ? k_strides[i] : 0;
  }
  p.cos_t = cos_table; p.sin_t = sin_table; p.n_pos = n_pos; p.pos0 = pos0;
  p.mode = rotary; p.inverse = inverse != 0; p.n_tensors = k ? 2 : 1;
  p.H = H; p.T = T; p.D = D;
  const int64_t vecs = (int64_t)T * (D / vec);
  dim3 grid((unsigned)((vecs + 255) / 256), B * H);
  if (dtype == LMK_BF16) rotary_pair_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else if (dtype == LMK_F16) rotary_pair_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  else rotary_pair_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}
