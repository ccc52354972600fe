// extern "C" entry points of libb200lmk.so for the fused attention kernels, plus error reporting.
// Argument checks mirror the assertions of the reference wrapper (llama/ltriton/flash_landmark_attention.py:319-324,
// 359-360, 396-397) and are done on the host before anything is launched.
#include "common.cuh"
#include "attn_params.h"

#include <mutex>

// Scratch for lmk_attn_bwd_static: one float per (batch, head, query row).  Lives in every GPU that loads the library
// until the process exits.  In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
#define LMK_STATIC_SCRATCH_FLOATS (1 << 20)
static __device__ __align__(256) float g_static_bwd_scratch[LMK_STATIC_SCRATCH_FLOATS];

namespace lmk {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

namespace {

int check_common(const void* q, const void* k, const void* v, int B, int H, int Lq, int Lk, int D,
                 const int64_t* qs, const int64_t* ks, const int64_t* vs, int block, int dtype, int path) {
  LMK_CHECK_ARG(q && k && v, "attention: q, k or v is null");
  LMK_CHECK_ARG(qs && ks && vs, "attention: stride arrays are required");
  LMK_CHECK_ARG(B >= 1 && H >= 1 && Lq >= 1 && Lk >= 1, "attention: empty problem (B=%d H=%d Lq=%d Lk=%d)", B, H, Lq, Lk);
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "attention: B*H = %lld exceeds 65535", (long long)B * H);
  LMK_CHECK_ARG(D <= 128, "FlashAttention only support head dimensions up to 128 (got %d)", D);
  LMK_CHECK_ARG(D >= 8 && D % 8 == 0, "attention: head dim %d must be a multiple of 8", D);
  LMK_CHECK_ARG(dtype == LMK_F32 || dtype == LMK_F16 || dtype == LMK_BF16, "attention: bad dtype %d", dtype);
  LMK_CHECK_ARG(block >= 2, "attention: block size %d must be >= 2", block);
  LMK_CHECK_ARG(Lk >= Lq && (Lk - Lq) % block == 0,
                "attention: key history Lk-Lq = %d must be a non-negative multiple of block %d", Lk - Lq, block);
  LMK_CHECK_ARG(path >= LMK_PATH_AUTO && path <= LMK_PATH_TCGEN05, "attention: bad path %d", path);
  return LMK_OK;
}

void fill(AttnParams& p, const void* q, const void* k, const void* v, int B, int H, int Lq, int Lk, int D,
          const int64_t* qs, const int64_t* ks, const int64_t* vs, int block, float scale) {
  p.q = q; p.k = k; p.v = v;
  p.B = B; p.H = H; p.Lq = Lq; p.Lk = Lk; p.D = D; p.block = block; p.scale = scale;
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = qs[i];
    p.ks[i] = ks[i];
    p.vs[i] = vs[i];
  }
}

// 1 = general, 2 = tcgen05, <0 = error.  LMK_PATH_AUTO takes the tcgen05 kernels only when the shape AND the operands
// (alignment, strides) qualify, and the general kernels otherwise; an explicit LMK_PATH_TCGEN05 request that cannot be
// met is an error.
int pick_path(int path, const AttnParams& p, int dtype, bool backward) {
  // the tcgen05 kernels take maxima on raw dot products, which needs a positive softmax scale
  const bool shape_ok = attn_sm100_supported(p.B, p.H, p.Lq, p.Lk, p.D, p.block, dtype) && p.scale > 0.f;
  const bool fast = shape_ok && attn_sm100_operands_ok(p, backward);
  if (path == LMK_PATH_TCGEN05) {
    if (!shape_ok)
      return fail(LMK_ERR_UNSUPPORTED,
                  "tcgen05 path needs bf16/fp16, D=128, block=64, Lq a multiple of 128 and a positive scale (got "
                  "dtype=%d D=%d block=%d Lq=%d Lk=%d scale=%g)", dtype, p.D, p.block, p.Lq, p.Lk, (double)p.scale);
    if (!fast)
      return fail(LMK_ERR_UNSUPPORTED,
                  "tcgen05 path needs 16-byte aligned tensors with positive batch/head strides and strides that are "
                  "multiples of 8 elements");
    return LMK_PATH_TCGEN05;
  }
  if (path == LMK_PATH_AUTO && fast) return LMK_PATH_TCGEN05;
  const int block = p.block;
  if (block > 128) return fail(LMK_ERR_UNSUPPORTED, "general path supports block sizes up to 128 (got %d)", block);
  return LMK_PATH_GENERAL;
}

}  // namespace
}  // namespace lmk

using namespace lmk;

extern "C" int lmk_version(void) { return LMK_VERSION; }

extern "C" const char* lmk_last_error(void) { return error_buffer(); }

extern "C" int lmk_device_status(int* status, int clear) {
  int v = 0;
  const int rc = device_status(&v, clear);
  if (status) *status = v;
  if (rc != LMK_OK) return rc;
  if (v != 0) return fail(LMK_ERR_DEVICE, "a bounded wait expired inside a kernel (site %d)", v);
  return LMK_OK;
}

extern "C" void lmk_debug_set_max_ctas(int n) { attn_sm100_set_max_ctas(n); }

extern "C" int lmk_attn_tcgen05_supported(int B, int H, int Lq, int Lk, int D, int block, int dtype) {
  return attn_sm100_supported(B, H, Lq, Lk, D, block, dtype) ? 1 : 0;
}

extern "C" int lmk_attn_fwd(const void* q, const void* k, const void* v, void* o, float* L, float* M, int B, int H,
                            int Lq, int Lk, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                            const int64_t v_strides[3], int block, float sm_scale, int dtype, int path,
                            void* stream) {
  int rc = check_common(q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, block, dtype, path);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(o && L && M, "attn_fwd: o, L or M is null");
  AttnParams p{};
  fill(p, q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, block, sm_scale);
  p.o = o; p.L = L; p.M = M;
  int which = pick_path(path, p, dtype, false);
  if (which < 0) return which;
  if (which == LMK_PATH_TCGEN05) return attn_sm100_fwd(p, dtype, (cudaStream_t)stream);
  return attn_general_fwd(p, dtype, (cudaStream_t)stream);
}

extern "C" size_t lmk_attn_bwd_workspace(int B, int H, int Lq, int Lk, int D, int block, int dtype, int path) {
  if (B < 1 || H < 1 || Lq < 1 || Lk < 1) return 0;
  // with LMK_PATH_AUTO the kernel family also depends on the operands' alignment, which is not known here: both
  // families need one float per (batch, head, query row), the larger figure is returned
  const size_t a = attn_sm100_bwd_workspace(B, H, Lq, Lk, D), b = attn_general_bwd_workspace(B, H, Lq);
  if (path == LMK_PATH_TCGEN05) return a;
  if (path == LMK_PATH_GENERAL) return b;
  return a > b ? a : b;
}

extern "C" int lmk_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO,
                            const float* L, const float* M, void* dQ, void* dK, void* dV, void* workspace,
                            size_t workspace_bytes, int B, int H, int Lq, int Lk, int D,
                            const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                            int block, float sm_scale, int dtype, int path, void* stream) {
  int rc = check_common(q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, block, dtype, path);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(o && dO && L && M && dQ && dK && dV, "attn_bwd: null tensor pointer");
  LMK_CHECK_ARG(Lq % block == 0 && Lk % block == 0, "Backward supported only for full blocks (Lq=%d Lk=%d block=%d)",
                Lq, Lk, block);
  AttnParams p{};
  fill(p, q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, block, sm_scale);
  p.o = const_cast<void*>(o); p.dO = dO;
  int which = pick_path(path, p, dtype, true);
  if (which < 0) return which;
  const size_t need = lmk_attn_bwd_workspace(B, H, Lq, Lk, D, block, dtype, which);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need))
    return fail(LMK_ERR_WORKSPACE, "attn_bwd: workspace of %zu bytes required, %zu given", need, workspace_bytes);
  LMK_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "attn_bwd: workspace must be 256-byte aligned");
  p.L = const_cast<float*>(L); p.M = const_cast<float*>(M);
  p.dq = dQ; p.dk = dK; p.dv = dV;
  p.workspace = workspace; p.workspace_bytes = workspace_bytes;
  if (which == LMK_PATH_TCGEN05) return attn_sm100_bwd(p, dtype, (cudaStream_t)stream);
  p.delta = reinterpret_cast<float*>(workspace);
  return attn_general_bwd(p, dtype, (cudaStream_t)stream);
}

// Device address of g_static_bwd_scratch on the current device, resolved once per device.
static int static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* addr[kMaxDevices] = {nullptr};
  int dev = 0;
  LMK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(LMK_ERR_UNSUPPORTED, "attn_bwd_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_bwd_scratch);   // current device = dev
    if (e != cudaSuccess || p == nullptr)
      return fail(LMK_ERR_CUDA, "attn_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    addr[dev] = p;
  }
  *out = addr[dev];
  return LMK_OK;
}

extern "C" size_t lmk_attn_bwd_static_max_rows(void) { return (size_t)LMK_STATIC_SCRATCH_FLOATS; }

extern "C" int lmk_attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const void* dO,
                                   const float* L, const float* M, void* dQ, void* dK, void* dV, int B, int H, int Lq,
                                   int Lk, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                                   const int64_t v_strides[3], int block, float sm_scale, int dtype, int path,
                                   void* stream) {
  if (B >= 1 && H >= 1 && Lq >= 1) {
    const size_t need = lmk_attn_bwd_workspace(B, H, Lq, Lk, D, block, dtype, path);
    if (need > sizeof(float) * (size_t)LMK_STATIC_SCRATCH_FLOATS)
      return fail(LMK_ERR_WORKSPACE,
                  "attn_bwd_static: B*H*Lq = %lld rows exceed the built-in scratch of %d rows; use lmk_attn_bwd with a "
                  "caller-provided workspace", (long long)B * H * Lq, LMK_STATIC_SCRATCH_FLOATS);
  }
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != LMK_OK) return rc;
  return lmk_attn_bwd(q, k, v, o, dO, L, M, dQ, dK, dV, scratch, sizeof(float) * (size_t)LMK_STATIC_SCRATCH_FLOATS, B,
                      H, Lq, Lk, D, q_strides, k_strides, v_strides, block, sm_scale, dtype, path, stream);
}

// ------------------------------------------------------------------------------------------------ arbitrary landmarks
namespace {
int check_mask_common(const void* q, const void* k, const void* v, const uint8_t* is_mem, int B, int H, int Lq, int Lk,
                      int D, const int64_t* qs, const int64_t* ks, const int64_t* vs, int max_groups, int dtype) {
  LMK_CHECK_ARG(q && k && v && is_mem, "masked attention: q, k, v or is_mem is null");
  LMK_CHECK_ARG(qs && ks && vs, "masked attention: stride arrays are required");
  LMK_CHECK_ARG(B >= 1 && H >= 1 && Lq >= 1 && Lk >= Lq, "masked attention: bad sizes (B=%d H=%d Lq=%d Lk=%d)", B, H, Lq, Lk);
  LMK_CHECK_ARG((int64_t)B * H <= 65535, "masked attention: B*H = %lld exceeds 65535", (long long)B * H);
  LMK_CHECK_ARG(max_groups >= 1, "masked attention: max_groups must be positive");
  if (!attn_mask_sm100_supported(B, H, Lq, Lk, D, dtype))
    return fail(LMK_ERR_UNSUPPORTED,
                "masked attention needs bf16/fp16, D=128, Lq a multiple of 128, Lk and Lk-Lq multiples of 64, Lk <= 32768 "
                "(got dtype=%d D=%d Lq=%d Lk=%d)", dtype, D, Lq, Lk);
  if (max_groups > attn_mask_sm100_max_groups())
    return fail(LMK_ERR_UNSUPPORTED, "masked attention keeps statistics for at most %d landmark groups per row (got %d)",
                attn_mask_sm100_max_groups(), max_groups);
  return LMK_OK;
}
}  // namespace

extern "C" int lmk_attn_mask_supported(int B, int H, int Lq, int Lk, int D, int dtype) {
  return attn_mask_sm100_supported(B, H, Lq, Lk, D, dtype) ? attn_mask_sm100_max_groups() : 0;
}

extern "C" int lmk_attn_mask_fwd(const void* q, const void* k, const void* v, const uint8_t* is_mem,
                                 int64_t is_mem_stride, void* o, float* R, float* A, int B, int H, int Lq, int Lk, int D,
                                 const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                                 int max_groups, float sm_scale, int dtype, void* stream) {
  int rc = check_mask_common(q, k, v, is_mem, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, max_groups, dtype);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(o && R && A, "attn_mask_fwd: o, R or A is null");
  AttnParams p{};
  fill(p, q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, 0, sm_scale);
  p.o = o;
  return attn_mask_sm100_fwd(p, is_mem, is_mem_stride, R, A, max_groups, dtype, (cudaStream_t)stream);
}

extern "C" size_t lmk_attn_mask_bwd_workspace(int B, int H, int Lq, int max_groups) {
  if (B < 1 || H < 1 || Lq < 1 || max_groups < 1) return 0;
  return attn_mask_sm100_bwd_workspace(B, H, Lq, max_groups);
}

extern "C" int lmk_attn_mask_bwd(const void* q, const void* k, const void* v, const uint8_t* is_mem,
                                 int64_t is_mem_stride, const void* o, const void* dO, const float* R, const float* A,
                                 void* dQ, void* dK, void* dV, void* workspace, size_t workspace_bytes, int B, int H,
                                 int Lq, int Lk, int D, const int64_t q_strides[3], const int64_t k_strides[3],
                                 const int64_t v_strides[3], int max_groups, float sm_scale, int dtype, void* stream) {
  int rc = check_mask_common(q, k, v, is_mem, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, max_groups, dtype);
  if (rc != LMK_OK) return rc;
  LMK_CHECK_ARG(o && dO && R && A && dQ && dK && dV, "attn_mask_bwd: null tensor pointer");
  const size_t need = attn_mask_sm100_bwd_workspace(B, H, Lq, max_groups);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(LMK_ERR_WORKSPACE, "attn_mask_bwd: workspace of %zu bytes required, %zu given", need, workspace_bytes);
  LMK_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "attn_mask_bwd: workspace must be 256-byte aligned");
  AttnParams p{};
  fill(p, q, k, v, B, H, Lq, Lk, D, q_strides, k_strides, v_strides, 0, sm_scale);
  p.o = const_cast<void*>(o); p.dO = dO;
  p.dq = dQ; p.dk = dK; p.dv = dV;
  p.workspace = workspace; p.workspace_bytes = workspace_bytes;
  return attn_mask_sm100_bwd(p, is_mem, is_mem_stride, R, A, max_groups, dtype, (cudaStream_t)stream);
}
