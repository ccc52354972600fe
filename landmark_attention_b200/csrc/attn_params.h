// Argument block shared by the fused-attention kernel families.
#pragma once
#include <stdint.h>
#include <stddef.h>
#include <cuda.h>
#include <cuda_runtime.h>

namespace lmk {

struct AttnParams {
  const void* q; const void* k; const void* v;
  void* o;                 // forward output / backward input
  const void* dO;
  float* L; float* M;      // [B*H, Lq]
  void* dq; void* dk; void* dv;
  float* delta;            // [B*H, Lq] scratch (backward)
  void* workspace; size_t workspace_bytes;
  int B, H, Lq, Lk, D, block;
  int64_t qs[3], ks[3], vs[3];   // element strides {batch, head, row}
  float scale;
};

int attn_general_fwd(const AttnParams& p, int dtype, cudaStream_t st);
int attn_general_bwd(const AttnParams& p, int dtype, cudaStream_t st);
size_t attn_general_bwd_workspace(int B, int H, int Lq);

bool attn_sm100_supported(int B, int H, int Lq, int Lk, int D, int block, int dtype);
// pointers and strides of q, k, v (and o, dO for the backward pass) are addressable by TMA
bool attn_sm100_operands_ok(const AttnParams& p, bool backward);
void attn_sm100_set_max_ctas(int n);
int attn_sm100_fwd(const AttnParams& p, int dtype, cudaStream_t st);
int attn_sm100_bwd(const AttnParams& p, int dtype, cudaStream_t st);
size_t attn_sm100_bwd_workspace(int B, int H, int Lq, int Lk, int D);
int device_status(int* out, int clear);
int* device_status_word();

// TMA descriptor of a [B, H, L, 128] 16-bit tensor with element strides {batch, head, row}: box = 64 features x
// `box_rows` rows, 128-byte swizzle (cached by pointer, shape and strides).  Binds the device's primary context first.
int tensor_map_4d(CUtensorMap* m, const void* ptr, int dtype, int B, int H, int L, const int64_t st[3], int box_rows);
bool tensor_map_operand_ok(const void* p, const int64_t st[3]);

// Fused attention with arbitrary landmark positions (attn_mask_sm100.cu).  R [B*H, Lq], A [B*H, G, Lq] fp32.
bool attn_mask_sm100_supported(int B, int H, int Lq, int Lk, int D, int dtype);
int attn_mask_sm100_fwd(const AttnParams& p, const uint8_t* is_mem, int64_t is_mem_stride, float* R, float* A, int G,
                        int dtype, cudaStream_t st);
int attn_mask_sm100_bwd(const AttnParams& p, const uint8_t* is_mem, int64_t is_mem_stride, const float* R,
                        const float* A, int G, int dtype, cudaStream_t st);
size_t attn_mask_sm100_bwd_workspace(int B, int H, int Lq, int G);
int attn_mask_sm100_max_groups();

}  // namespace lmk
