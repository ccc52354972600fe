// Write side of the landmark block cache: append whole blocks of un-rotated keys / values to a (ring) block cache of
// any layout and, in the same pass, copy every block's landmark key (its last row) into a dense [B, H, capacity, D]
// array, so that scoring reads 1/block of the key bytes contiguously instead of one strided row per block.
//
// Reference: MemLMCacheStorage.store_in_cache (lm_benchmark/models/caches/mem_cache.py:111-158), which writes the
// ring buffer [B, capacity, block, H, D] with tensor copies and keeps no separate landmark array.
#include "common.cuh"

namespace lmk {
namespace {

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
