"""Landmark grouped softmax on materialised attention scores, with the reference's two signatures.

llama flavour:        landmark_grouped_softmax(x, dim, is_mem, last_section_mask)           llama/llama_mem.py:222-243
lm_benchmark flavour: landmark_grouped_softmax_lm(x, dim, is_mem, attn_mask, last_section_mask, return_group_prob,
                                                  max_mem_cnt, p_group_dropout=None)       lm_benchmark/models/landmark.py:88-119
Both return fp32 probabilities and are differentiable w.r.t. x.  Masks may be broadcast views; they are never
expanded in memory and no int64 index tensor is built.
"""
import torch

from . import _lib as L


def _as_u8(mask):
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        return mask.view(torch.uint8) if mask.is_contiguous() or mask.dim() == 0 else mask.to(torch.uint8)
    return (mask != 0).to(torch.uint8)        # the kernels read bit 0 of every byte


def _prep(x, is_mem, last, hidden):
    if x.dim() != 4:
        raise ValueError("expected scores of shape [B, H, Lq, Lk]")
    if x.stride(3) != 1:
        x = x.contiguous()
    shape = x.shape
    masks = []
    for m in (is_mem, last, hidden):
        if m is None:
            masks.append((None, None))
            continue
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m8 = _as_u8(m)
        m8, st = L.strides4_broadcast(m8, shape)
        masks.append((m8, st))
    return x, masks


class _GroupedSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, is_mem, last, hidden, guards, max_groups, max_mem_cnt):
        L.require_cuda(x, is_mem, last, hidden)
        x, masks = _prep(x, is_mem, last, hidden)
        B, H, Lq, Lk = x.shape
        probs = torch.empty((B, H, Lq, Lk), device=x.device, dtype=torch.float32)
        gp = torch.empty((B, H, Lq, max_mem_cnt), device=x.device, dtype=torch.float32) if max_mem_cnt else None
        (m8, ms), (l8, ls), (h8, hs) = masks
        rc = L.lib().lmk_grouped_softmax_fwd(L.ptr(x), L.strides3(x), L.ptr(m8), ms, L.ptr(l8), ls, L.ptr(h8), hs,
                                             L.ptr(probs), L.ptr(gp), max_mem_cnt or 0, B, H, Lq, Lk,
                                             L.dtype_code(x), int(guards), max_groups, L.stream_ptr(x.device))
        L.check(rc, "lmk_grouped_softmax_fwd")
        ctx.save_for_backward(x, is_mem, last, hidden if hidden is not None else torch.empty(0))
        ctx.has_hidden = hidden is not None
        ctx.guards, ctx.max_groups = guards, max_groups
        if gp is not None:
            ctx.mark_non_differentiable(gp)
            return probs, gp
        return probs, None

    @staticmethod
    def backward(ctx, gprobs, _ggp):
        x, is_mem, last, hidden = ctx.saved_tensors
        hidden = hidden if ctx.has_hidden else None
        x, masks = _prep(x, is_mem, last, hidden)
        B, H, Lq, Lk = x.shape
        gprobs = gprobs.to(torch.float32).contiguous()
        gx = torch.empty((B, H, Lq, Lk), device=x.device, dtype=torch.float32)
        (m8, ms), (l8, ls), (h8, hs) = masks
        rc = L.lib().lmk_grouped_softmax_bwd(L.ptr(x), L.strides3(x), L.ptr(m8), ms, L.ptr(l8), ls, L.ptr(h8), hs,
                                             L.ptr(gprobs), L.ptr(gx), B, H, Lq, Lk, L.dtype_code(x),
                                             int(ctx.guards), ctx.max_groups, L.stream_ptr(x.device))
        L.check(rc, "lmk_grouped_softmax_bwd")
        return gx.to(x.dtype), None, None, None, None, None, None


_CAUSAL_MAX_KEYS = 4096      # rows the mask-free kernel takes (include/b200lmk.h, lmk_grouped_softmax_causal_fwd)


class _GroupedSoftmaxCausal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, is_mem_row, max_groups):
        L.require_cuda(x, is_mem_row)
        if x.stride(3) != 1:
            x = x.contiguous()
        B, H, Lq, Lk = x.shape
        flags = _as_u8(is_mem_row)
        flags = flags if flags.stride(-1) == 1 else flags.contiguous()
        probs = torch.empty((B, H, Lq, Lk), device=x.device, dtype=torch.float32)
        rc = L.lib().lmk_grouped_softmax_causal_fwd(L.ptr(x), L.strides3(x), L.ptr(flags), flags.stride(0), L.ptr(probs),
                                                    B, H, Lq, Lk, L.dtype_code(x), max_groups, L.stream_ptr(x.device))
        L.check(rc, "lmk_grouped_softmax_causal_fwd")
        ctx.save_for_backward(x, flags)
        ctx.max_groups = max_groups
        return probs

    @staticmethod
    def backward(ctx, gprobs):
        x, flags = ctx.saved_tensors
        B, H, Lq, Lk = x.shape
        gprobs = gprobs.to(torch.float32).contiguous()
        gx = torch.empty((B, H, Lq, Lk), device=x.device, dtype=torch.float32)
        rc = L.lib().lmk_grouped_softmax_causal_bwd(L.ptr(x), L.strides3(x), L.ptr(flags), flags.stride(0), L.ptr(gprobs),
                                                    L.ptr(gx), B, H, Lq, Lk, L.dtype_code(x), ctx.max_groups,
                                                    L.stream_ptr(x.device))
        L.check(rc, "lmk_grouped_softmax_causal_bwd")
        return gx.to(x.dtype), None, None


def landmark_grouped_softmax_causal(x, is_mem_row, max_mem_cnt=None):
    """Mask block, masked_fill and grouped softmax of lm_benchmark's call site (lm_benchmark/models/landmark.py:210-232)
    from the RAW scores x [B,H,Lq,Lk] and one landmark flag per (batch row, key), is_mem_row [B,Lk]: query i sees keys
    0 .. i + Lk - Lq (a cache prefix of Lk - Lq columns is visible to every query).  No [Lq,Lk] mask is built or read,
    hidden scores need not be filled with -inf beforehand, and rows are only read up to their last visible key.
    fp32 probabilities, differentiable w.r.t. x.  Rows longer than 4096 keys go through the masks."""
    B, H, Lq, Lk = x.shape
    if max_mem_cnt is None:
        max_mem_cnt = min(2048, Lk + 1)
    max_groups = min(2048, max(int(max_mem_cnt), 2))
    if Lk <= _CAUSAL_MAX_KEYS and (Lk + 255) // 256 * 1280 * 4 + 64 * max_groups <= 96 * 1024:
        return _GroupedSoftmaxCausal.apply(x, is_mem_row, max_groups)
    hidden = torch.ones(Lq, Lk, dtype=torch.bool, device=x.device).triu(Lk - Lq + 1)
    mask, is_mem, last = prepare_landmark_masks(is_mem_row, hidden)
    probs, _ = _GroupedSoftmax.apply(x.masked_fill(mask, float("-inf")), is_mem, last, mask, True, max_groups, 0)
    return probs


def _check_dim(x, dim):
    if dim not in (-1, x.dim() - 1):
        raise NotImplementedError("the grouped softmax runs over the last dimension")


def landmark_grouped_softmax(x, dim, is_mem, last_section_mask, max_groups=None):
    """llama flavour (llama/llama_mem.py:222-243).  The reference hard-codes room for 63 landmarks per row
    (max_mem_cnt = 64, :228); here `max_groups` bounds 1 + the number of landmarks in a row.  Default: the row length + 1,
    capped at 256 so that rows of up to 4096 keys stay on the fast kernel; a row with more landmarks than that sets
    the device status word (501, see `_lib.device_status`) instead of passing unnoticed -- give `max_groups` then."""
    _check_dim(x, dim)
    if max_groups is None:
        max_groups = min(256, x.shape[-1] + 1)
    probs, _ = _GroupedSoftmax.apply(x, is_mem, last_section_mask, None, False, max_groups, 0)
    return probs


def landmark_grouped_softmax_lm(x, dim, is_mem, attn_mask, last_section_mask, return_group_prob, max_mem_cnt,
                                p_group_dropout=None):
    """lm_benchmark flavour (lm_benchmark/models/landmark.py:88-119).

    Group dropout (:110-114, a training-time regulariser): every landmark's group weight is dropped with probability p
    or scaled by 1/(1-p); last-section keys are untouched.  The kernel computes the probabilities without dropout and
    the keep factors are applied per (row, group) afterwards -- the same function of x as the reference's formulation,
    with this package's own random draw (one `torch.rand` of shape [B,H,Lq,max_mem_cnt-1] from the default generator)."""
    _check_dim(x, dim)
    max_groups = min(2048, max(int(max_mem_cnt), 2))
    drop = p_group_dropout is not None and p_group_dropout > 0
    probs, gp = _GroupedSoftmax.apply(x, is_mem, last_section_mask, attn_mask, True, max_groups,
                                      int(max_mem_cnt) if (return_group_prob or drop) else 0)
    if drop:
        p = float(p_group_dropout)
        B, H, Lq, Lk = probs.shape
        keep = (torch.rand((B, H, Lq, int(max_mem_cnt) - 1), device=probs.device) >= p).to(probs.dtype) / (1.0 - p)
        group = torch.cumsum(is_mem.expand(B, H, Lq, Lk).to(torch.int64), dim=-1).clamp_(max=int(max_mem_cnt) - 2)
        factor = torch.gather(keep, -1, group)
        bucket = is_mem | last_section_mask | attn_mask
        probs = torch.where(bucket, probs, probs * factor)
        if return_group_prob:
            gp = torch.cat((gp[..., :-1] * keep, gp[..., -1:] / (1.0 - p)), dim=-1)
    return probs, (gp if return_group_prob else None)


def prepare_landmark_masks(is_mem_row, attn_mask):
    """Mask block of the call sites (lm_benchmark/models/landmark.py:210-224; llama/llama_mem.py:807-815).
    is_mem_row: bool [B, Lk]; attn_mask: bool [..., Lq, Lk] (True = hidden).
    Returns (mask, is_mem, last_section), bool [B, 1, Lq, Lk]."""
    B, Lk = is_mem_row.shape
    im = is_mem_row.view(B, 1, 1, Lk)
    while attn_mask.dim() < 4:
        attn_mask = attn_mask.unsqueeze(0)
    imi = im.to(torch.int32)
    before = torch.cumsum(imi, dim=-1) - imi
    mem_ids = torch.where(attn_mask, torch.zeros_like(before), before)
    last = mem_ids == mem_ids.amax(dim=-1, keepdim=True)
    mask = attn_mask | (im & last)
    last = last & ~mask
    is_mem = im & ~mask
    return mask, is_mem, last


def lm_landmark_attention(q, k, v, is_mem_row, sm_scale=None, max_groups=None, att_prefix=None, cache_values=None):
    """Attention of lm_benchmark's CausalSelfAttention.forward (landmark.py:196-243): q, k rotated, landmarks at
    arbitrary per-row positions is_mem_row [B, T].

    Without a cache, bf16/fp16 with head dim 128 and T a multiple of 128 runs as ONE fused operator on the tensor
    cores (masked.landmark_attention_masked: no score, mask or probability tensor exists).  Other shapes and fp32 use
    the unfused route: library matmuls around this package's grouped-softmax kernel, masks as broadcast views.

    With a cache (the evaluation branch, :182-209 and :236-243): `att_prefix` [B,H,T,P] and `cache_values`
    {'v': [B,H,T,P,D] or [B,H,P,D], 'is_mem': [B,P] (optional)} are what `MemLMCacheStorage.retrieve_for_query`
    returns; the prefix columns are visible to every query and go through the same grouped softmax in front of the
    chunk's own keys.  This branch takes the unfused route."""
    from .masked import DEFAULT_MAX_GROUPS, landmark_attention_masked, masked_attention_supported
    B, H, T, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / (D ** 0.5)
    n_pre = 0 if att_prefix is None else att_prefix.shape[-1]
    fused_groups = DEFAULT_MAX_GROUPS if max_groups is None else int(max_groups)
    if n_pre == 0 and masked_attention_supported(q, k, fused_groups):
        return landmark_attention_masked(q, k, v, is_mem_row, sm_scale, fused_groups)
    att = torch.matmul(q, k.transpose(-2, -1)) * sm_scale
    if n_pre:
        att = torch.cat((att_prefix.to(att.dtype), att), dim=-1)
        pre_mem = cache_values.get('is_mem')
        if pre_mem is None:
            pre_mem = torch.zeros((B, n_pre), dtype=torch.bool, device=q.device)
        is_mem_row = torch.cat((pre_mem.to(torch.bool), is_mem_row.to(torch.bool)), dim=-1)
    # mask block + masked_fill + grouped softmax in one kernel, from the raw scores and the row flags
    probs = landmark_grouped_softmax_causal(att, is_mem_row, max_groups if max_groups is not None
                                            else min(2048, T + n_pre + 1))
    probs = probs.to(v.dtype)
    y = torch.matmul(probs[..., n_pre:], v)
    if n_pre:
        cache_v = cache_values['v']
        pp = probs[..., :n_pre]
        if cache_v.dim() == v.dim():
            y = y + torch.matmul(pp, cache_v)
        elif cache_v.dim() == v.dim() + 1:
            y = y + torch.matmul(pp.unsqueeze(3), cache_v).squeeze(3)
        else:
            raise NotImplementedError("cache values must be [B,H,P,D] or [B,H,T,P,D]")
    return y
