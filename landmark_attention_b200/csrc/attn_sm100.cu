// placeholder
#include "common.cuh"
#include "attn_params.h"
namespace lmk {
bool attn_sm100_supported(int, int, int, int, int, int, int) { return false; }
int attn_sm100_fwd(const AttnParams&, int, cudaStream_t) { return fail(LMK_ERR_UNSUPPORTED, "tcgen05 path not built"); }
int attn_sm100_bwd(const AttnParams&, int, cudaStream_t) { return fail(LMK_ERR_UNSUPPORTED, "tcgen05 path not built"); }
size_t attn_sm100_bwd_workspace(int, int, int, int, int) { return 0; }
}
