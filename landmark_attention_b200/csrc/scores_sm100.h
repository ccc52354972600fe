// Tensor-core landmark scoring (see scores_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "../../include/b200lmk.h"

namespace lmk {
bool scores_sm100_supported(int D, int dtype, int Tq, int N);
size_t scores_sm100_workspace(int B, int H, int N);
int scores_sm100(const void* q, const void* k_cache, const lmk_cache_desc& desc, const void* cos_t, const void* sin_t,
                 int n_pos, int rotary, float* scores, int B, int H, int Tq, float scale, int dtype, void* workspace,
                 cudaStream_t st);
}  // namespace lmk
