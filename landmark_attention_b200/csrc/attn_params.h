// Argument block shared by the fused-attention kernel families.
#pragma once
#include <stdint.h>
#include <stddef.h>
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

}  // namespace lmk
