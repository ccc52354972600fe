/*
 * b200lmk.h — C ABI of libb200lmk.so: landmark attention kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless stated otherwise; the library
 *     never allocates or frees device memory.  What it keeps between calls: a per-thread error string,
 *     a per-device status word (lmk_device_status), a host-side table of encoded TMA descriptors keyed
 *     by (pointer, shape, strides), and the fixed scratch array of lmk_attn_bwd_static.
 *   - Calls are asynchronous: they return once the kernels are queued on `stream`.
 *   - Tensors are row-major with a contiguous last dimension.  q/k/v take explicit element strides
 *     {batch, head, row}; all other tensors are dense in the documented shape.
 *   - dtype: LMK_F32, LMK_F16 or LMK_BF16 (all of q, k, v, o, dO, dQ, dK, dV share it).
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - Return value: LMK_OK (0) or a negative LMK_ERR_* code.  Nothing is launched when an argument
 *     check fails.  lmk_last_error() returns a description of the calling thread's last failure.
 *
 * Each entry point names the interface of epfml/landmark-attention it replaces (file:line relative to
 * that project's root).
 */
#ifndef B200LMK_H
#define B200LMK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LMK_VERSION 100

enum { LMK_F32 = 0, LMK_F16 = 1, LMK_BF16 = 2 };

enum {
  LMK_OK = 0,
  LMK_ERR_INVALID = -1,     /* bad shape / pointer / flag (the reference raises AssertionError / ValueError) */
  LMK_ERR_UNSUPPORTED = -2, /* valid request that no kernel in this build covers */
  LMK_ERR_CUDA = -3,        /* a CUDA runtime or driver call failed */
  LMK_ERR_WORKSPACE = -4,   /* workspace missing or too small */
  LMK_ERR_DEVICE = -5       /* returned by lmk_device_status only: a bounded wait expired inside an earlier kernel */
};

/* Kernel family selection for the fused attention entry points. */
enum {
  LMK_PATH_AUTO = 0,    /* tcgen05 path when shape, alignment and strides qualify, otherwise the general path */
  LMK_PATH_GENERAL = 1, /* CUDA-core fp32-accumulate kernels: any dtype, D <= 128, block <= 128 */
  LMK_PATH_TCGEN05 = 2  /* TMA + tcgen05/TMEM kernels: bf16/fp16, D == 128, block == 64, full 128-row tiles */
};

int lmk_version(void);
const char* lmk_last_error(void);

/*
 * Device-side status word of the current device.  Every wait inside the tcgen05 kernels is bounded; a wait that
 * expires records a site code (> 0) here instead of hanging, and the kernel runs to its end with undefined results.
 * The compute entry points cannot see this (they return before their kernels run), so a caller that wants to know
 * polls this function after the work: it synchronises the device, writes the code (0 = healthy) to *status (nullable),
 * clears it when `clear` != 0, and returns LMK_ERR_DEVICE when the code is non-zero.  No counterpart in the reference.
 */
int lmk_device_status(int* status, int clear);

/*
 * Test hook: upper bound on the CTAs of the persistent backward kernels (0 = one per SM, the default), so that small
 * test problems still make every CTA walk through several work units.  No counterpart in the reference.
 */
void lmk_debug_set_max_ctas(int n);

/* 1 if the (shape, dtype) is handled by the tcgen05 kernels, else 0. */
int lmk_attn_tcgen05_supported(int B, int H, int Lq, int Lk, int D, int block, int dtype);

/*
 * Fused landmark attention, forward.
 * Replaces FusedLandmarkAttention.forward + _fwd_kernel
 *   (llama/ltriton/flash_landmark_attention.py:6-122, 311-353).
 *   q [B,H,Lq,D], k,v [B,H,Lk,D] (strided), o [B,H,Lq,D] dense, L and M [B*H, Lq] fp32
 *   (sum of exponentials and maximum of the outer softmax, as the reference stores them).
 *   Landmark = last key of each `block`; (Lk-Lq) must be a multiple of block (:396-397); D <= 128 (:321).
 */
int lmk_attn_fwd(const void* q, const void* k, const void* v, void* o, float* L, float* M,
                 int B, int H, int Lq, int Lk, int D,
                 const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                 int block, float sm_scale, int dtype, int path, void* stream);

/*
 * Bytes of scratch lmk_attn_bwd needs for this problem (0 is possible).
 * Stands for the temporaries FusedLandmarkAttention.backward allocates
 *   (fp32 dq, do_scaled, delta: flash_landmark_attention.py:363-367).
 */
size_t lmk_attn_bwd_workspace(int B, int H, int Lq, int Lk, int D, int block, int dtype, int path);

/*
 * Fused landmark attention, backward (recompute based).
 * Replaces FusedLandmarkAttention.backward + _bwd_preprocess + _bwd_kernel
 *   (llama/ltriton/flash_landmark_attention.py:125-305, 356-389).
 *   o, dO, dQ [B,H,Lq,D] dense; dK, dV [B,H,Lk,D] dense; L, M from the forward call.
 *   Lq and Lk must be multiples of block (:359-360).  workspace: >= lmk_attn_bwd_workspace(...) bytes,
 *   256-byte aligned, contents irrelevant on entry.
 */
int lmk_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO,
                 const float* L, const float* M, void* dQ, void* dK, void* dV,
                 void* workspace, size_t workspace_bytes,
                 int B, int H, int Lq, int Lk, int D,
                 const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                 int block, float sm_scale, int dtype, int path, void* stream);

/*
 * Backward pass for callers that cannot allocate device memory.  (No counterpart in the reference.)
 *
 * Some hosts of this library may not call cudaMalloc at the point where they run the backward pass: a plugin that is
 * handed finished buffers by its runtime and owns no allocator, code running inside a region where allocation is
 * forbidden (for example while another component holds the allocator lock or a memory pool is frozen), or a
 * real-time loop that must not touch the allocator.  lmk_attn_bwd needs lmk_attn_bwd_workspace() bytes of scratch
 * (one float per batch*head*query row) from such a caller; this variant brings its own: a fixed array compiled into
 * the library image, resident on every GPU that loads the library until the process exits.
 *
 *   - Same arguments and results as lmk_attn_bwd, without workspace / workspace_bytes.
 *   - Limit: B*H*Lq <= lmk_attn_bwd_static_max_rows() (1,048,576 rows = 4 MiB of scratch per GPU).  Larger problems are
 *     rejected with LMK_ERR_WORKSPACE and nothing is launched; use lmk_attn_bwd for them.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on each device looks up the
 *     array's device address (a one-time host-side query with that device current); make that first call before
 *     starting any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to start at zero (every element that is read was
 *     written earlier in the same call), so it is never cleared; it keeps the previous call's contents.  Two calls
 *     whose kernels can overlap on the GPU (different streams, no ordering between them) race on it: serialise them.
 */
size_t lmk_attn_bwd_static_max_rows(void);
int lmk_attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const void* dO,
                        const float* L, const float* M, void* dQ, void* dK, void* dV,
                        int B, int H, int Lq, int Lk, int D,
                        const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                        int block, float sm_scale, int dtype, int path, void* stream);

/*
 * Fused landmark attention with landmarks at ARBITRARY key positions, forward.
 * Replaces the attention of CausalSelfAttention.forward without cache -- scores, causal fill, the mask block, the
 * grouped softmax and att @ v (lm_benchmark/models/landmark.py:196-236 with :210-224 and :37-119) -- in one kernel
 * family on the tensor cores; no [B,H,Lq,Lk] tensor (scores, boolean masks, probabilities) is ever materialised.
 *   q [B,H,Lq,D], k,v [B,H,Lk,D] (strided, already rotated), o [B,H,Lq,D] dense.
 *   is_mem: one byte per (batch row, key), non-zero = landmark; row b starts at is_mem + b * is_mem_stride
 *     (landmark.py:368 builds it per batch row; windows are cut at random offsets, optim/utils.py:21-26).
 *   Causal with the query rows aligned to the end of the keys (query i sits at key position Lk - Lq + i).
 *   R [B*H, Lq] and A [B*H, max_groups, Lq] fp32 are written for the backward pass (log2-domain normalisers of the
 *     outer softmax and of every closed landmark group).
 *   max_groups: upper bound on the number of landmarks before any query (the reference's max_mem_cnt - 1,
 *     landmark.py:88-119); lmk_attn_mask_supported returns the largest value this build accepts (0: shape not
 *     supported).  A row with more landmarks sets the device status word (lmk_device_status) and gets undefined output.
 *   Shape contract: bf16/fp16, D = 128, Lq a multiple of 128, Lk and Lk - Lq multiples of 64, Lk <= 32768.
 */
int lmk_attn_mask_supported(int B, int H, int Lq, int Lk, int D, int dtype);
int lmk_attn_mask_fwd(const void* q, const void* k, const void* v, const uint8_t* is_mem, int64_t is_mem_stride,
                      void* o, float* R, float* A, int B, int H, int Lq, int Lk, int D,
                      const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                      int max_groups, float sm_scale, int dtype, void* stream);

/*
 * Backward of lmk_attn_mask_fwd (what autograd derives for lm_benchmark/models/landmark.py:196-236 through
 * LandmarkGroupedSoftmaxFunction.backward, :66-86).  o, dO, dQ dense [B,H,Lq,D]; dK, dV dense [B,H,Lk,D]; R, A from
 * the forward call; workspace >= lmk_attn_mask_bwd_workspace(...) bytes, 256-byte aligned, contents irrelevant.
 */
size_t lmk_attn_mask_bwd_workspace(int B, int H, int Lq, int max_groups);
int lmk_attn_mask_bwd(const void* q, const void* k, const void* v, const uint8_t* is_mem, int64_t is_mem_stride,
                      const void* o, const void* dO, const float* R, const float* A,
                      void* dQ, void* dK, void* dV, void* workspace, size_t workspace_bytes,
                      int B, int H, int Lq, int Lk, int D,
                      const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                      int max_groups, float sm_scale, int dtype, void* stream);

/*
 * Stand-alone landmark grouped softmax over the last dimension of x [B,H,Lq,Lk].
 * Replaces LandmarkGroupedSoftmaxFunction.forward + landmark_grouped_softmax
 *   (llama/llama_mem.py:168-243; lm_benchmark/models/landmark.py:37-119).
 *   x: dtype `dtype`, element strides x_strides {b,h,row}, last dim contiguous.
 *   is_mem, last_section, hidden (nullable): bool bytes (0 or 1), broadcastable, element strides {b,h,row,col}
 *     (0 = broadcast).  `hidden` is the lm_benchmark attn_mask argument.
 *   probs: fp32 dense [B,H,Lq,Lk].  group_prob (nullable): fp32 dense [B,H,Lq,max_mem_cnt]
 *     (slot g = probability of the landmark closing group g, last slot = total last-section probability).
 *   guards != 0 selects the lm_benchmark flavour (all -inf group -> 0 instead of NaN).
 *   max_groups: upper bound on 1 + number of landmarks in any row (<= 2048); a row with max_groups or more
 *     landmarks records 501 in the device status word (lmk_device_status) and its surplus groups get probability 0.
 */
int lmk_grouped_softmax_fwd(const void* x, const int64_t x_strides[3],
                            const uint8_t* is_mem, const int64_t is_mem_strides[4],
                            const uint8_t* last_section, const int64_t last_strides[4],
                            const uint8_t* hidden, const int64_t hidden_strides[4],
                            float* probs, float* group_prob, int max_mem_cnt,
                            int B, int H, int Lq, int Lk, int dtype, int guards, int max_groups, void* stream);

/*
 * Backward of the grouped softmax: grad_x (fp32 dense [B,H,Lq,Lk]) from grad_probs (fp32 dense), recomputing
 * the probabilities from x.  Replaces LandmarkGroupedSoftmaxFunction.backward and the autograd chain through
 * the group-probability multiply (llama/llama_mem.py:198-220, 238-240).
 */
int lmk_grouped_softmax_bwd(const void* x, const int64_t x_strides[3],
                            const uint8_t* is_mem, const int64_t is_mem_strides[4],
                            const uint8_t* last_section, const int64_t last_strides[4],
                            const uint8_t* hidden, const int64_t hidden_strides[4],
                            const float* grad_probs, float* grad_x,
                            int B, int H, int Lq, int Lk, int dtype, int guards, int max_groups, void* stream);

/*
 * The same softmax for the lm_benchmark call site without any [Lq,Lk] mask: the mask block of
 * lm_benchmark/models/landmark.py:210-224 (causal rule "query i sees keys 0 .. i + Lk - Lq", last section, the masked
 * landmark of the query's own block) is derived inside the kernel from one flag per (batch row, key), hidden scores
 * count as -inf whatever x holds there (the masked_fill of :224), and rows are only read up to their last visible key.
 * lm_benchmark flavour (guards).  Rows of at most 4096 keys; longer ones return LMK_ERR_UNSUPPORTED (build the masks and
 * call lmk_grouped_softmax_fwd).
 *   x [B,H,Lq,Lk] as above; is_mem_row: bool bytes, row b at is_mem_row + b * is_mem_stride; probs / grad_probs /
 *   grad_x: fp32 dense [B,H,Lq,Lk].
 */
int lmk_grouped_softmax_causal_fwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem_row,
                                   int64_t is_mem_stride, float* probs, int B, int H, int Lq, int Lk, int dtype,
                                   int max_groups, void* stream);
int lmk_grouped_softmax_causal_bwd(const void* x, const int64_t x_strides[3], const uint8_t* is_mem_row,
                                   int64_t is_mem_stride, const float* grad_probs, float* grad_x, int B, int H, int Lq,
                                   int Lk, int dtype, int max_groups, void* stream);

/* Rotary conventions for the retrieval kernels. */
enum {
  LMK_ROTARY_NONE = 0,
  LMK_ROTARY_HALF = 1,       /* pairs (d, d+D/2): llama/llama_mem.py:127-149 */
  LMK_ROTARY_INTERLEAVED = 2, /* pairs (2d, 2d+1): lm_benchmark/models/positional_encoders/rotary_utils.py:17-31 */
  LMK_ROTARY_HALF_SYM = 3     /* LMK_ROTARY_HALF with the caller's promise that cos[p][d] == cos[p][d + D/2] and the same
                                 for sin (tables built as cat(freqs, freqs), llama/llama_mem.py:104-108): the second
                                 halves are not read.  Accepted by lmk_selected_attend only. */
};

/*
 * Description of a block cache of un-rotated keys/values split in landmark blocks of `block` tokens.
 *   strides (elements): batch, head, block, row; last dim contiguous.
 *   n_blocks: blocks currently held; ring_start: physical index of the OLDEST block (0 unless the cache is a
 *   ring buffer, lm_benchmark/models/caches/mem_cache.py:53-56); top_k: number of blocks to retrieve;
 *   pos_base: position of the first key of slot 0 (llama: prefix_len, llama_mem.py:361; lm_benchmark: 0).
 * Slot rule shared by both call sites (llama_mem.py:362-365, mem_cache.py:58-59): a block whose logical age
 * index is among the newest top_k is scored at slot 1 + (its rank among them), every other block at slot 0;
 * its landmark key is rotated at position pos_base + slot*block + block-1.
 */
typedef struct {
  int64_t stride_b, stride_h, stride_block, stride_row;
  int n_blocks, ring_start, block, top_k;
  int pos_base;
} lmk_cache_desc;

/*
 * Append whole blocks to a block cache and keep a dense array of their landmark keys.
 * Replaces the ring-buffer writes of MemLMCacheStorage.store_in_cache (lm_benchmark/models/caches/mem_cache.py:140-158)
 * and adds what that code does not keep: landmark_keys, where block slot s of (b, h) holds the un-rotated key of the
 * block's last row, so that lmk_landmark_scores can read the landmark keys contiguously (pass it a descriptor
 * with stride_block = the array's slot stride and stride_row = 0).
 *   k_src, v_src [B,H,n_store*block,D] with element strides {batch, head, row} (the chunk's whole blocks, oldest first);
 *   block i is written to physical slot (first_slot + i) mod capacity of k_cache / v_cache, addressed through the
 *   descriptors' strides (any layout: the reference's [B,capacity,block,H,D] or a head-major [B,H,capacity,block,D]);
 *   landmark_keys (nullable) with element strides {batch, head, slot}.  16-byte aligned pointers, D * sizeof(dtype) and
 *   all strides multiples of 16 bytes.  The descriptors' n_blocks / ring_start / top_k / pos_base are not used.
 */
int lmk_cache_store(const void* k_src, const void* v_src, const int64_t src_strides[3], void* k_cache, void* v_cache,
                    const lmk_cache_desc* kdesc, const lmk_cache_desc* vdesc, void* landmark_keys,
                    const int64_t landmark_strides[3], int B, int H, int n_store, int first_slot, int capacity, int D,
                    int dtype, void* stream);

/*
 * Everything a LLaMA layer does to one chunk's projections before its landmark attention, in one launch
 * (replaces apply_rotary_pos_emb on the chunk, llama/llama_mem.py:127-149 and :335, and the cache concatenation of
 * :424-425; the padded copies and flags feed lmk_attn_mask_fwd).  16-bit types, rotate-half rotary.
 *   q, k, v [B,H,T,D] un-rotated, element strides {batch, head, row}, last dim contiguous.
 *   cos_table, sin_table [n_pos, D] of the same dtype; row t is rotated at position min(pos0 + t, n_pos - 1) with the
 *     roundings of the tensor formulation (x * cos and rotate_half(x) * sin rounded, then their sum).
 *   q_rot [B,H,T,D] dense: rotated queries.  q_pad, k_pad, v_pad [B,H,t_pad,D] dense: rotated queries, rotated keys and
 *     values with rows T .. t_pad-1 zero.  flags_pad [B,t_pad]: landmark flags of the rows, chunk_flags[t] (T bytes,
 *     nullable) or (pos0 + t) % block == block - 1; 0 for padding rows.
 *   cache_k, cache_v (nullable, both or none): un-rotated k, v are also written to rows cache_pos .. cache_pos + T - 1
 *     of a cache addressed with element strides cache_strides {batch, head, row}.
 * All pointers 16-byte aligned, strides multiples of 8 elements, D a power of two times 16 up to 2048.
 */
int lmk_chunk_prepare(const void* q, const void* k, const void* v, const int64_t q_strides[3],
                      const int64_t k_strides[3], const int64_t v_strides[3], const void* cos_table,
                      const void* sin_table, int n_pos, int64_t pos0, const uint8_t* chunk_flags, int block,
                      void* q_rot, void* q_pad, void* k_pad, void* v_pad, uint8_t* flags_pad, void* cache_k,
                      void* cache_v, const int64_t cache_strides[3], int64_t cache_pos, int B, int H, int T, int t_pad,
                      int D, int dtype, void* stream);

/*
 * Rotary position embedding of the queries and keys of one layer in one launch: out = x * cos + rotate(x) * sin at
 * positions pos0 + t, t = 0 .. T-1 (clamped to n_pos - 1).  rotary = LMK_ROTARY_HALF: rotate(x) = (-x[d + D/2], x[d])
 * (llama/llama_mem.py:127-149); LMK_ROTARY_INTERLEAVED: pairs (x0, x1) -> (-x1, x0)
 * (lm_benchmark/models/positional_encoders/rotary_utils.py:17-31, adapt_queries / adapt_keys of rotary.py).
 * inverse != 0 rotates by the negative angle, which is the gradient of the forward call.  16-bit types round the two
 * products and the sum as the tensor formulation does.
 *   q, k (k nullable together with k_out) [B,H,T,D], element strides {batch, head, row}, last dim contiguous;
 *   cos_table, sin_table [n_pos, D] of the same dtype; q_out, k_out dense [B,H,T,D].
 */
int lmk_rotary_apply(const void* q, const void* k, const int64_t q_strides[3], const int64_t k_strides[3],
                     const void* cos_table, const void* sin_table, int n_pos, int64_t pos0, int rotary, int inverse,
                     void* q_out, void* k_out, int B, int H, int T, int D, int dtype, void* stream);

/*
 * Landmark scores: scores[b,h,t,n] = sm_scale * q[b,h,t,:] . rot(K[b,h,n,block-1,:], slot position of n).
 * Replaces llama/llama_mem.py:357-367 and lm_benchmark/models/caches/mem_cache.py:51-61.
 *   q [B,H,T,D] dense (already rotated), k_cache per desc, cos/sin tables [n_pos, D] in `dtype` (NULL with
 *   LMK_ROTARY_NONE), scores fp32 dense [B,H,T,n_blocks]; softmax != 0 applies a softmax over n in fp32
 *   (mem_cache.py:62; llama_mem.py:376 mode B) and, when dtype is 16-bit, rounds it to dtype as the reference does.
 *   workspace (nullable): lmk_landmark_scores_workspace(...) bytes, 256-byte aligned.  When given and the shape
 *   qualifies (bf16/fp16, D = 128, T >= 128, n_blocks >= 128) the product runs on the tensor cores (rotated landmark
 *   keys are staged in the workspace); otherwise a CUDA-core kernel is used.
 */
size_t lmk_landmark_scores_workspace(int B, int H, int T, int D, int n_blocks, int dtype);
int lmk_landmark_scores(const void* q, const void* k_cache, const lmk_cache_desc* desc,
                        const void* cos_table, const void* sin_table, int n_pos, int rotary,
                        float* scores, int B, int H, int T, int D, float sm_scale, int softmax,
                        int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Per-row top-k with ascending index output.  Replaces `topk(...)[1].sort(...)[0]`
 *   (llama/llama_mem.py:384; mem_cache.py:72-83).
 *   scores: fp32, logical shape [rows, reduce, n] addressed as scores[row*row_stride + r*reduce_stride + j];
 *   each row's value at j is the maximum over r (reduce = 1: plain rows; reduce > 1 implements the
 *   max_over_tokens / max_over_heads aggregation, mem_cache.py:63-70).  rows are decomposed as
 *   row = outer*inner_count + inner with offset outer*outer_stride + inner*inner_stride.
 *   idx_out int32 [rows, k]: indices of the k largest values (ties: lower index first), sorted ascending.
 *   With ring_start != 0 the ascending order is by logical age (physical - ring_start mod n), as
 *   mem_cache.py:73-83 does, but physical indices are returned.
 */
int lmk_topk_sorted(const float* scores, int32_t* idx_out, int64_t outer_count, int64_t inner_count,
                    int64_t outer_stride, int64_t inner_stride, int reduce, int64_t reduce_stride,
                    int n, int k, int ring_start, void* stream);

/*
 * Gather the selected blocks and rotate the gathered keys at their slot positions.
 * Replaces llama/llama_mem.py:386-398,408-410 and mem_cache.py:85-98.
 *   idx int32 dense [B,H,T,top_k] (physical block indices, ascending logical age);
 *   k_out, v_out dense [B,H,T,top_k*block,D] in `dtype` (either may be NULL to skip it);
 *   key position of row r of the i-th selected block: pos_base + (i + recent)*block + r, recent = 1 when the
 *   block is among the newest top_k (llama_mem.py:386-388, mem_cache.py:92-94).
 */
int lmk_gather_kv(const void* k_cache, const void* v_cache, const lmk_cache_desc* kdesc,
                  const lmk_cache_desc* vdesc, const int32_t* idx,
                  const void* cos_table, const void* sin_table, int n_pos, int rotary,
                  void* k_out, void* v_out, int B, int H, int T, int D, int dtype, void* stream);

/*
 * Attention over the selected blocks without materialising the gather (the two matmuls of
 * llama/llama_mem.py:399-404 and :468-474 fused with the gather + rotary of :386-398): the blocks are read in place.
 *   lmk_selected_logits: logits[b,h,t, col0 + i*block + r] = sm_scale * q[b,h,t,:] . rot(K[idx[b,h,t,i], r, :]),
 *     q dense [B,H,T,D] already rotated; keys rotated at the slot positions and with the rounding steps of
 *     lmk_gather_kv, the dot product accumulated in fp32; D * sizeof(dtype) must be 64, 128, 256 or 512 bytes;
 *     logits in `dtype`, row stride `ld` elements, so the caller can point it into the buffer that also holds the
 *     local keys' logits.
 *   lmk_selected_pv: out[b,h,t,:] = sum_{i,r} probs[b,h,t, col0 + i*block + r] * V[idx[b,h,t,i], r, :];
 *     probs in `dtype` with row stride `ld`; out dense [B,H,T,D] in `dtype`, fp32 accumulation.
 */
int lmk_selected_logits(const void* q, const void* k_cache, const lmk_cache_desc* kdesc, const int32_t* idx,
                        const void* cos_table, const void* sin_table, int n_pos, int rotary, void* logits,
                        int64_t ld, int64_t col0, int B, int H, int T, int D, float sm_scale, int dtype,
                        void* stream);
int lmk_selected_pv(const void* probs, int64_t ld, int64_t col0, const void* v_cache, const lmk_cache_desc* vdesc,
                    const int32_t* idx, void* out, int B, int H, int T, int D, int dtype, void* stream);

/*
 * Attention over the selected blocks in ONE kernel, merged with the attention over the local keys: replaces the
 * gather + rotary + q k^T of llama/llama_mem.py:386-404, the prefix columns of the grouped softmax (:415-420, 462-466)
 * and the prefix value product (:468-474) without writing logits or probabilities to memory.
 *   Every selected block is a closed landmark group: its rows 0..block-2 share the probability of its landmark (row
 *   block-1), split by a softmax inside the block; the landmark rows themselves carry no value weight.
 *   o_local [B,H,local_rows,D] (dtype) and R_local [B*H, local_rows] (fp32), local_rows >= T, of which rows 0..T-1 are
 *   read: the attention output over the local keys normalised on its own, and log2 of its share of the outer softmax
 *   (what lmk_attn_mask_fwd writes as o and R, possibly for a query count padded to its tile size).  Both NULL:
 *   attention over the selected blocks alone.
 *   out [B,H,T,D] dense = (2^R o_local + sum_i 2^(x_i) o_i) / (2^R + sum_i 2^(x_i)), x_i the landmark logits (log2
 *   domain), o_i the in-block softmax-weighted value sums.  q, caches, idx, rotary arguments as for lmk_selected_logits.
 */
int lmk_selected_attend(const void* q, const void* k_cache, const lmk_cache_desc* kdesc, const void* v_cache,
                        const lmk_cache_desc* vdesc, const int32_t* idx, const void* cos_table, const void* sin_table,
                        int n_pos, int rotary, const void* o_local, const float* R_local, int64_t local_rows, void* out,
                        int B, int H, int T, int D, float sm_scale, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200LMK_H */
