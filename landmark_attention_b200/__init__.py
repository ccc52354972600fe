"""B200-native kernels for the landmark-attention hot path (fused fwd/bwd, grouped softmax, block retrieval).

The package is a thin PyTorch host layer over libb200lmk.so (C ABI in include/b200lmk.h).  It has no CPU or
eager fallback: calls fail loudly when the library is missing or a tensor is not on a CUDA device.
"""
from ._lib import PATH_AUTO, PATH_GENERAL, PATH_TCGEN05, ROTARY_HALF, ROTARY_INTERLEAVED, ROTARY_NONE, lib  # noqa: F401
from .fused import (FusedLandmarkAttention, attn_forward_with_stats, fused_landmark_attention,  # noqa: F401
                    landmark_sdpa)
from .host_pipeline import HostAttentionPipeline  # noqa: F401
from .grouped_softmax import (landmark_grouped_softmax, landmark_grouped_softmax_causal,  # noqa: F401
                              landmark_grouped_softmax_lm,
                              lm_landmark_attention, prepare_landmark_masks)
from .masked import landmark_attention_masked, masked_attention_supported  # noqa: F401
from .mem_cache import MemLMCache, MemLMCacheStorage  # noqa: F401
from .retrieval import (LandmarkKVCache, OffloadedLandmarkCache, chunk_prepare, gather_kv, landmark_scores, llama_retrieval_attention, make_desc,  # noqa: F401
                        rotary_apply, rotary_tables_half, rotary_tables_interleaved, selected_attend, selected_logits, selected_pv,
                        topk_sorted)
