// Landmark scoring on the tensor cores (bf16/fp16, head dim 128):
//   1. rotate_landmarks_kernel gathers the landmark key of every cached block and rotates it at its slot position
//      (same rounding sequence as torch's x*cos + rotate_half(x)*sin in the input dtype) into a dense [B*H, N, 128]
//      scratch matrix;
//   2. scores_gemm_kernel computes one [128 tokens x 128 landmarks] tile of Q . K_lm^T per CTA: TMA loads, eight
//      tcgen05 MMAs (M128 N128 K16) into TMEM, and an epilogue that applies the softmax scale with the reference's two
//      roundings to the input dtype and writes fp32 scores.
// Reference: llama/llama_mem.py:357-367, lm_benchmark/models/caches/mem_cache.py:51-61.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "scores_sm100.h"
#include "attn_params.h"

namespace lmk {

namespace {

using namespace ptx;

__host__ __device__ __forceinline__ int logical_age2(int phys, int ring_start, int n) {
  int l = phys - ring_start;
  return l < 0 ? l + n : l;
}

constexpr int kRotPerCta = 16;

template <typename T> struct Pk16;      // two 16-bit values in one register, rounded like the tensor formulation
template <> struct Pk16<__nv_bfloat16> {
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
template <> struct Pk16<__half> {
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

// Sixteen landmark rows per CTA, eight threads per row: each thread takes one 16-byte vector of the low half of the
// row and its partner of the high half, so every load of the CTA is in flight at once.
template <typename T>
__global__ void __launch_bounds__(128) rotate_landmarks_kernel(const T* __restrict__ kc, lmk_cache_desc desc,
                                                               const T* __restrict__ cos_t, const T* __restrict__ sin_t,
                                                               int n_pos, int rotary, T* __restrict__ out, int H) {
  constexpr int D = 128, HALF = 64;
  const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
  const int N = desc.n_blocks, blk = desc.block;
  const int n = blockIdx.x * kRotPerCta + (threadIdx.x >> 3), d0 = (threadIdx.x & 7) * 8;
  if (n >= N) return;
  const T* row = kc + b * desc.stride_b + h * desc.stride_h + (int64_t)n * desc.stride_block +
                 (int64_t)(blk - 1) * desc.stride_row;
  uint4 lo = *reinterpret_cast<const uint4*>(row + d0), hi = *reinterpret_cast<const uint4*>(row + HALF + d0);
  if (rotary != LMK_ROTARY_NONE) {
    const int logical = logical_age2(n, desc.ring_start, N);
    const int first_recent = N - desc.top_k;
    const int slot = logical >= first_recent ? logical - first_recent + 1 : 0;
    int pos = desc.pos_base + slot * blk + blk - 1;
    pos = max(0, min(pos, n_pos - 1));
    const uint4 cl = *reinterpret_cast<const uint4*>(cos_t + (int64_t)pos * D + d0);
    const uint4 ch = *reinterpret_cast<const uint4*>(cos_t + (int64_t)pos * D + HALF + d0);
    const uint4 sl = *reinterpret_cast<const uint4*>(sin_t + (int64_t)pos * D + d0);
    const uint4 sh = *reinterpret_cast<const uint4*>(sin_t + (int64_t)pos * D + HALF + d0);
    const uint32_t *l = reinterpret_cast<const uint32_t*>(&lo), *hh = reinterpret_cast<const uint32_t*>(&hi);
    const uint32_t *c0 = reinterpret_cast<const uint32_t*>(&cl), *c1 = reinterpret_cast<const uint32_t*>(&ch);
    const uint32_t *s0 = reinterpret_cast<const uint32_t*>(&sl), *s1 = reinterpret_cast<const uint32_t*>(&sh);
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t pl, ph;                 // rotate(x) for the low and the high vector
      if (rotary == LMK_ROTARY_HALF) {
        pl = hh[u] ^ 0x80008000u;      // (-x[d + D/2], x[d])
        ph = l[u];
      } else {
        pl = __byte_perm(l[u], l[u], 0x1032) ^ 0x00008000u;      // pairs (x0, x1) -> (-x1, x0)
        ph = __byte_perm(hh[u], hh[u], 0x1032) ^ 0x00008000u;
      }
      ol[u] = Pk16<T>::add(Pk16<T>::mul(l[u], c0[u]), Pk16<T>::mul(pl, s0[u]));
      oh[u] = Pk16<T>::add(Pk16<T>::mul(hh[u], c1[u]), Pk16<T>::mul(ph, s1[u]));
    }
    lo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    hi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
  T* dst = out + ((int64_t)bh * N + n) * D;
  *reinterpret_cast<uint4*>(dst + d0) = lo;
  *reinterpret_cast<uint4*>(dst + HALF + d0) = hi;
}

struct ScoreSmem {
  uint64_t full;
  uint64_t done;
  uint32_t tmem_base;
};

template <typename T>
__global__ void __launch_bounds__(128) scores_gemm_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                          const __grid_constant__ CUtensorMap tm_k,
                                                          float* __restrict__ scores, int Tq, int N, float scale,
                                                          int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t a_tile = base, b_tile = base + 32768u;
  ScoreSmem* sm = reinterpret_cast<ScoreSmem*>(smem_raw + (base - raw) + 128u * 132u * 4u);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n0 = blockIdx.x * 128, t0 = blockIdx.y * 128, bh = blockIdx.z;
  if (tid == 0) {
    mbar_init(smem_u32(&sm->full), 1);
    mbar_init(smem_u32(&sm->done), 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(smem_u32(&sm->tmem_base), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  if (tid == 0) {
    const uint32_t fb = smem_u32(&sm->full);
    mbar_arrive_expect_tx(fb, 65536u);
    tma_load_3d(a_tile, &tm_q, fb, 0, t0, bh);
    tma_load_3d(a_tile + 16384u, &tm_q, fb, 64, t0, bh);
    tma_load_3d(b_tile, &tm_k, fb, 0, n0, bh);
    tma_load_3d(b_tile + 16384u, &tm_k, fb, 64, n0, bh);
    mbar_wait(fb, 0, status, 401);
    tc_fence_after();
    constexpr uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t idesc = instr_desc_f16(fmt, 128, 128, 0, 0);
    const uint64_t da = smem_desc_sw128(a_tile, 16, 1024), db = smem_desc_sw128(b_tile, 16, 1024);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_f16_ss(tmem, desc_advance(da, kmajor_step(kk, 16384u)), desc_advance(db, kmajor_step(kk, 16384u)), idesc,
                 kk > 0);
    mma_commit(smem_u32(&sm->done));
  }
  __syncwarp();
  mbar_wait(smem_u32(&sm->done), 0, status, 402);
  tc_fence_after();
  // Epilogue: TMEM -> registers (thread = token row) -> shared memory (rows padded to 132 floats so that 16-byte
  // stores of 32 different rows spread over all banks) -> global memory one full 512-byte row per warp instruction.
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  float* stage = reinterpret_cast<float*>(smem_raw + (base - raw));     // reuses the operand tiles
  constexpr int kPad = 132;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(tmem + c * 32 + lane_base, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float4 v;
      // the reference's matmul output and the scaling are each rounded to the input dtype
      v.x = to_f32(from_f32<T>(to_f32(from_f32<T>(__uint_as_float(r[j]))) * scale));
      v.y = to_f32(from_f32<T>(to_f32(from_f32<T>(__uint_as_float(r[j + 1]))) * scale));
      v.z = to_f32(from_f32<T>(to_f32(from_f32<T>(__uint_as_float(r[j + 2]))) * scale));
      v.w = to_f32(from_f32<T>(to_f32(from_f32<T>(__uint_as_float(r[j + 3]))) * scale));
      *reinterpret_cast<float4*>(stage + tid * kPad + c * 32 + j) = v;
    }
  }
  __syncwarp();     // each warp reads back only the 32 rows it wrote
  const int lane = tid & 31;
  const bool vec_ok = (N % 4 == 0);
  for (int rr = 0; rr < 32; ++rr) {
    const int t = t0 + warp * 32 + rr;
    if (t >= Tq) break;
    const float4 v = *reinterpret_cast<const float4*>(stage + (warp * 32 + rr) * kPad + lane * 4);
    float* orow = scores + ((int64_t)bh * Tq + t) * N + n0 + lane * 4;
    const int n = n0 + lane * 4;
    if (vec_ok && n + 3 < N) {
      *reinterpret_cast<float4*>(orow) = v;
    } else {
      if (n < N) orow[0] = v.x;
      if (n + 1 < N) orow[1] = v.y;
      if (n + 2 < N) orow[2] = v.z;
      if (n + 3 < N) orow[3] = v.w;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_map_3d(CUtensorMap* m, const void* ptr, int dtype, int64_t rows, int64_t batches) {
  static EncodeTiledFn enc = nullptr;
  if (enc == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<EncodeTiledFn>(p);
  }
  if (!enc) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)batches};
  cuuint64_t strides[2] = {256, (cuuint64_t)rows * 256};
  cuuint32_t box[3] = {64, (cuuint32_t)(rows < 128 ? rows : 128), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, dtype == LMK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LMK_ERR_CUDA, "cuTensorMapEncodeTiled (scores) failed with %d", (int)r);
  return LMK_OK;
}

template <typename T>
int run(const void* q, const void* k_cache, const lmk_cache_desc& desc, const void* cos_t, const void* sin_t, int n_pos,
        int rotary, float* scores, int B, int H, int Tq, float scale, int dtype, void* workspace, cudaStream_t st) {
  const int N = desc.n_blocks;
  dim3 g1((N + kRotPerCta - 1) / kRotPerCta, B * H);
  rotate_landmarks_kernel<T><<<g1, 128, 0, st>>>((const T*)k_cache, desc, (const T*)cos_t, (const T*)sin_t, n_pos,
                                                 rotary, (T*)workspace, H);
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaSetDevice(dev);   // bind the context for the driver call
  CUtensorMap tq, tk;
  int rc;
  if ((rc = make_map_3d(&tq, q, dtype, Tq, (int64_t)B * H)) != LMK_OK) return rc;
  if ((rc = make_map_3d(&tk, workspace, dtype, N, (int64_t)B * H)) != LMK_OK) return rc;
  const size_t smem = 1024 + 128 * 132 * 4 + sizeof(ScoreSmem);   // operand tiles (64 KB), reused as the padded output stage
  LMK_CUDA(cudaFuncSetAttribute(scores_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 g2((N + 127) / 128, (Tq + 127) / 128, B * H);
  int* status = device_status_word();
  if (status == nullptr) return fail(LMK_ERR_CUDA, "device status word is not addressable");
  scores_gemm_kernel<T><<<g2, 128, smem, st>>>(tq, tk, scores, Tq, N, scale, status);
  LMK_CUDA(cudaGetLastError());
  return LMK_OK;
}

}  // namespace

bool scores_sm100_supported(int D, int dtype, int Tq, int N) {
  // boxes of fewer than 128 rows leave part of the operand tiles unwritten; keep those small cases on the CUDA cores
  return D == 128 && (dtype == LMK_BF16 || dtype == LMK_F16) && Tq >= 128 && N >= 128;
}

size_t scores_sm100_workspace(int B, int H, int N) { return (size_t)B * H * N * 128 * 2; }

int scores_sm100(const void* q, const void* k_cache, const lmk_cache_desc& desc, const void* cos_t, const void* sin_t,
                 int n_pos, int rotary, float* scores, int B, int H, int Tq, float scale, int dtype, void* workspace,
                 cudaStream_t st) {
  if (dtype == LMK_BF16)
    return run<__nv_bfloat16>(q, k_cache, desc, cos_t, sin_t, n_pos, rotary, scores, B, H, Tq, scale, dtype, workspace, st);
  return run<__half>(q, k_cache, desc, cos_t, sin_t, n_pos, rotary, scores, B, H, Tq, scale, dtype, workspace, st);
}

}  // namespace lmk
