"""Inference-time landmark retrieval: scores -> top-k -> gather, and the LLaMA cache branch built from them.

Reference: LlamaAttention.forward cache branch, llama/llama_mem.py:318-430, 447-474.
"""
import ctypes
import math

import torch

from . import _lib as L
from .grouped_softmax import landmark_grouped_softmax, prepare_landmark_masks


def rotary_tables_half(n_pos, dim, dtype, device, base=10000.0):
    """cos/sin tables [n_pos, dim] built as LlamaRotaryEmbedding does (llama/llama_mem.py:96-122)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, device=device).float() / dim))
    t = torch.arange(n_pos, device=device, dtype=inv_freq.dtype)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype).contiguous(), emb.sin().to(dtype).contiguous()


def rotary_tables_interleaved(n_pos, dim, dtype, device):
    """cos/sin tables [n_pos, dim] for lm_benchmark's rotary (positional_encoders/rotary.py:24-55)."""
    freqs = 10 ** (-4 * torch.arange(0, dim, 2, device=device)[: dim // 2].float() / dim)
    t = torch.arange(n_pos, device=device, dtype=torch.float32)
    ang = (t.unsqueeze(-1) * freqs.view(1, -1)).unsqueeze(-1).expand(n_pos, dim // 2, 2).reshape(n_pos, dim)
    return ang.cos().to(dtype).contiguous(), ang.sin().to(dtype).contiguous()


class _RotaryPair(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, pos0, mode):
        ctx.save_for_backward(cos, sin)
        ctx.pos0, ctx.mode = pos0, mode
        return _rotary_launch(q, k, cos, sin, pos0, mode, False)

    @staticmethod
    def backward(ctx, gq, gk):
        cos, sin = ctx.saved_tensors
        dq, dk = _rotary_launch(gq, gk, cos, sin, ctx.pos0, ctx.mode, True)      # rotation by the negative angle
        return dq, dk, None, None, None, None


def _rotary_launch(q, k, cos, sin, pos0, mode, inverse):
    L.require_cuda(q, k, cos, sin)
    B, H, T, D = q.shape
    q, k = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k)]
    assert k.shape == q.shape and q.dtype == k.dtype == cos.dtype == sin.dtype
    assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == D
    qo, ko = torch.empty((B, H, T, D), dtype=q.dtype, device=q.device), torch.empty((B, H, T, D), dtype=q.dtype, device=q.device)
    rc = L.lib().lmk_rotary_apply(L.ptr(q), L.ptr(k), L.strides3(q), L.strides3(k), L.ptr(cos), L.ptr(sin), cos.shape[0],
                                  int(pos0), mode, int(inverse), L.ptr(qo), L.ptr(ko), B, H, T, D, L.dtype_code(q),
                                  L.stream_ptr(q.device))
    L.check(rc, "lmk_rotary_apply")
    return qo, ko


def rotary_apply(q, k, cos, sin, pos0=0, interleaved=True):
    """Rotary position embedding of q and k [B,H,T,D] (any batch/head/row strides) at positions pos0 .. pos0+T-1 in one
    launch, differentiable (the backward pass is the inverse rotation, one launch as well).  interleaved=True is
    lm_benchmark's adapt_queries / adapt_keys (positional_encoders/rotary.py:35-55 with rotary_utils.py:17-31);
    False is LLaMA's rotate-half (llama/llama_mem.py:127-149).  cos, sin: tables [n_pos, D] of q's dtype
    (rotary_tables_interleaved / rotary_tables_half).  Returns dense (q_rot, k_rot)."""
    return _RotaryPair.apply(q, k, cos, sin, int(pos0), L.ROTARY_INTERLEAVED if interleaved else L.ROTARY_HALF)


def apply_rotary_half(x, cos, sin, positions):
    """x*cos + rotate_half(x)*sin with tables gathered at `positions` (llama/llama_mem.py:127-149)."""
    c, s = cos[positions], sin[positions]
    d = x.shape[-1]
    rot = torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return x * c + rot * s


def make_desc(cache_view, block, n_blocks, top_k, ring_start=0, pos_base=0, strides=None):
    """Cache descriptor for a tensor addressed as [b, h, block index, row, d]."""
    if strides is None:
        strides = cache_view.stride()[:4]
    return L.CacheDesc(int(strides[0]), int(strides[1]), int(strides[2]), int(strides[3]),
                       int(n_blocks), int(ring_start), int(block), int(top_k), int(pos_base))


def landmark_scores(q, k_cache, desc, cos=None, sin=None, rotary=L.ROTARY_NONE, sm_scale=None, softmax=False):
    """fp32 scores [B,H,T,n_blocks] of rotated queries against the cached landmark keys (rotated at slot positions)."""
    L.require_cuda(q, k_cache)
    q = q.contiguous()
    B, H, T, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    scores = torch.empty((B, H, T, desc.n_blocks), device=q.device, dtype=torch.float32)
    n_pos = 0 if cos is None else cos.shape[0]
    need = L.lib().lmk_landmark_scores_workspace(B, H, T, D, desc.n_blocks, L.dtype_code(q))
    ws = torch.empty(int(need), dtype=torch.uint8, device=q.device) if need else None
    rc = L.lib().lmk_landmark_scores(L.ptr(q), L.ptr(k_cache), ctypes.byref(desc), L.ptr(cos), L.ptr(sin), n_pos,
                                     rotary, L.ptr(scores), B, H, T, D, float(sm_scale), int(softmax),
                                     L.dtype_code(q), L.ptr(ws), int(need), L.stream_ptr(q.device))
    L.check(rc, "lmk_landmark_scores")
    return scores


def topk_sorted(scores, k, mode="per_token_and_head", ring_start=0):
    """Indices (int32, ascending logical age) of the k best blocks.
    scores: fp32 [B,H,T,N].  mode: per_token_and_head -> [B,H,T,k]; max_over_tokens -> [B,H,1,k];
    max_over_heads -> [B,1,T,k] (lm_benchmark/models/caches/mem_cache.py:63-70; llama/llama_mem.py:373-384)."""
    L.require_cuda(scores)
    assert scores.dtype == torch.float32 and scores.is_contiguous()
    B, H, T, N = scores.shape
    if mode == "per_token_and_head":
        shape, args = (B, H, T, k), (B * H * T, 1, N, 0, 1, 0)
    elif mode == "max_over_tokens":
        shape, args = (B, H, 1, k), (B * H, 1, T * N, 0, T, N)
    elif mode == "max_over_heads":
        shape, args = (B, 1, T, k), (B, T, H * T * N, N, H, T * N)
    else:
        raise NotImplementedError(mode)
    idx = torch.empty(shape, device=scores.device, dtype=torch.int32)
    outer, inner, ostride, istride, reduce, rstride = args
    rc = L.lib().lmk_topk_sorted(L.ptr(scores), L.ptr(idx), outer, inner, ostride, istride, reduce, rstride, N, k,
                                 ring_start, L.stream_ptr(scores.device))
    L.check(rc, "lmk_topk_sorted")
    return idx


def gather_kv(k_cache, v_cache, kdesc, vdesc, idx, cos=None, sin=None, rotary=L.ROTARY_NONE, dim=None):
    """Gather the selected blocks: returns (k_sel rotated at slot positions, v_sel), each [B,H,T,top_k*block,D]."""
    L.require_cuda(k_cache, v_cache, idx)
    assert idx.dtype == torch.int32 and idx.is_contiguous()
    B, H, T, top_k = idx.shape
    D = dim if dim is not None else k_cache.shape[-1]
    k_out = torch.empty((B, H, T, top_k * kdesc.block, D), device=idx.device, dtype=k_cache.dtype)
    v_out = torch.empty_like(k_out)
    n_pos = 0 if cos is None else cos.shape[0]
    rc = L.lib().lmk_gather_kv(L.ptr(k_cache), L.ptr(v_cache), ctypes.byref(kdesc), ctypes.byref(vdesc), L.ptr(idx),
                               L.ptr(cos), L.ptr(sin), n_pos, rotary, L.ptr(k_out), L.ptr(v_out), B, H, T, D,
                               L.dtype_code(k_cache), L.stream_ptr(idx.device))
    L.check(rc, "lmk_gather_kv")
    return k_out, v_out


def selected_logits(q, k_cache, kdesc, idx, out, col0=0, cos=None, sin=None, rotary=L.ROTARY_NONE, sm_scale=None):
    """Logits of each query against the keys of ITS selected blocks, read in place from the cache (no gathered copy):
    out[b,h,t, col0 + i*block + r] = sm_scale * q[b,h,t] . rot(K[idx[b,h,t,i], r]).  `out` is a [B,H,T,W] tensor of
    q's dtype that may be wider than top_k*block, so the logits of local keys can live in the same buffer.
    Fuses llama/llama_mem.py:386-404 (gather, rotary at slot positions, q k^T)."""
    L.require_cuda(q, k_cache, idx, out)
    q = q.contiguous()
    B, H, T, D = q.shape
    assert idx.dtype == torch.int32 and idx.is_contiguous() and idx.shape == (B, H, T, kdesc.top_k)
    assert out.dtype == q.dtype and out.shape[:3] == (B, H, T) and out.is_contiguous()
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    n_pos = 0 if cos is None else cos.shape[0]
    rc = L.lib().lmk_selected_logits(L.ptr(q), L.ptr(k_cache), ctypes.byref(kdesc), L.ptr(idx), L.ptr(cos), L.ptr(sin),
                                     n_pos, rotary, L.ptr(out), out.shape[3], col0, B, H, T, D, float(sm_scale),
                                     L.dtype_code(q), L.stream_ptr(q.device))
    L.check(rc, "lmk_selected_logits")
    return out


def selected_pv(probs, v_cache, vdesc, idx, col0=0, dim=None):
    """sum_j probs[b,h,t, col0 + j] * V[selected row j] -> [B,H,T,D], the value rows read in place from the cache.
    Fuses the gather with the p_prefix @ v matmul of llama/llama_mem.py:468-474."""
    L.require_cuda(probs, v_cache, idx)
    assert probs.is_contiguous() and probs.dtype == v_cache.dtype
    B, H, T, W = probs.shape
    D = dim if dim is not None else v_cache.shape[-1]
    out = torch.empty((B, H, T, D), device=probs.device, dtype=probs.dtype)
    rc = L.lib().lmk_selected_pv(L.ptr(probs), W, col0, L.ptr(v_cache), ctypes.byref(vdesc), L.ptr(idx), L.ptr(out),
                                 B, H, T, D, L.dtype_code(probs), L.stream_ptr(probs.device))
    L.check(rc, "lmk_selected_pv")
    return out


_SYMMETRIC = {}       # (id(cos), id(sin)) -> (weakref to cos, weakref to sin, versions, verdict)


def _halves_equal(cos, sin, check=True):
    """Whether cos[p, d] == cos[p, d + D/2] and the same for sin (tables built as cat(freqs, freqs), as LLaMA's rotary
    embedding does).  One device comparison per pair of table tensors, remembered while those tensor objects live and
    are not written to; check=False only looks the verdict up (None if unknown)."""
    import weakref
    key = (id(cos), id(sin))
    hit = _SYMMETRIC.get(key)
    if hit is not None and hit[0]() is cos and hit[1]() is sin and hit[2] == (cos._version, sin._version):
        return hit[3]
    if not check:
        return None
    h = cos.shape[1] // 2
    verdict = bool(torch.equal(cos[:, :h], cos[:, h:]) and torch.equal(sin[:, :h], sin[:, h:]))
    if len(_SYMMETRIC) > 64:
        _SYMMETRIC.clear()
    _SYMMETRIC[key] = (weakref.ref(cos), weakref.ref(sin), (cos._version, sin._version), verdict)
    return verdict


def selected_attend(q, k_cache, v_cache, kdesc, vdesc, idx, cos=None, sin=None, rotary=L.ROTARY_NONE, sm_scale=None,
                    o_local=None, R_local=None):
    """Attention of every query over ITS selected blocks in one kernel, merged with the attention over the local keys.

    o_local [B,H,Tl,D] / R_local [B*H,Tl] (Tl >= T) are the output and the log2 outer-softmax share of the local keys as
    `lmk::masked_attention_fwd` returns them; None: attend over the selected blocks alone.  No logits or probabilities
    are written to memory.  Fuses llama/llama_mem.py:386-404, the prefix part of :462-466 and :468-474."""
    L.require_cuda(q, k_cache, v_cache, idx)
    q = q.contiguous()
    B, H, T, D = q.shape
    assert idx.dtype == torch.int32 and idx.is_contiguous() and idx.shape == (B, H, T, kdesc.top_k)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    local_rows = 0
    if o_local is not None:
        assert o_local.is_contiguous() and R_local.is_contiguous() and o_local.dtype == q.dtype
        local_rows = o_local.shape[2]
        assert o_local.shape == (B, H, local_rows, D) and R_local.shape == (B * H, local_rows)
    out = torch.empty((B, H, T, D), device=q.device, dtype=q.dtype)
    n_pos = 0 if cos is None else cos.shape[0]
    if rotary == L.ROTARY_HALF and _halves_equal(cos, sin, check=not torch.cuda.is_current_stream_capturing()):
        rotary = L.ROTARY_HALF_SYM              # the kernel then reads half of the table bytes
    rc = L.lib().lmk_selected_attend(L.ptr(q), L.ptr(k_cache), ctypes.byref(kdesc), L.ptr(v_cache), ctypes.byref(vdesc),
                                     L.ptr(idx), L.ptr(cos), L.ptr(sin), n_pos, rotary, L.ptr(o_local), L.ptr(R_local),
                                     local_rows, L.ptr(out), B, H, T, D, float(sm_scale), L.dtype_code(q),
                                     L.stream_ptr(q.device))
    L.check(rc, "lmk_selected_attend")
    return out


def chunk_prepare(q, k_new, v_new, cos, sin, pos0, chunk_is_mem, block, t_pad, cache=None):
    """One launch for what a layer does to a chunk's projections before its attention (lmk_chunk_prepare): rotate-half
    rotary of q and k at positions pos0 .. pos0+T-1 (llama/llama_mem.py:127-149), copies padded with zero rows to t_pad
    rows, the landmark flags of those rows, and -- with `cache`, a LandmarkKVCache -- the append of the un-rotated keys
    and values (:424-425).  Returns (q_rot [B,H,T,D], q_pad, k_pad, v_pad [B,H,t_pad,D], flags uint8 [B,t_pad])."""
    L.require_cuda(q, k_new, v_new, cos, sin)
    B, H, T, D = q.shape
    q, k_new, v_new = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k_new, v_new)]
    assert cos.dtype == q.dtype and cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == D
    dev = q.device
    q_rot = torch.empty((B, H, T, D), dtype=q.dtype, device=dev)
    q_pad, k_pad, v_pad = [torch.empty((B, H, t_pad, D), dtype=q.dtype, device=dev) for _ in range(3)]
    flags = torch.empty((B, t_pad), dtype=torch.uint8, device=dev)
    cf = None
    if chunk_is_mem is not None:
        cf = chunk_is_mem.reshape(-1)[:T].to(torch.uint8).contiguous()
    ck = cv = cst = None
    cache_pos = 0
    if cache is not None:
        if cache.length + T > cache.k.shape[2]:
            raise ValueError(f"cache capacity {cache.k.shape[2]} exceeded ({cache.length} + {T})")
        assert cache.k.stride() == cache.v.stride() and cache.k.stride(3) == 1
        ck, cv, cst, cache_pos = cache.k, cache.v, L.strides3(cache.k), cache.length
    rc = L.lib().lmk_chunk_prepare(L.ptr(q), L.ptr(k_new), L.ptr(v_new), L.strides3(q), L.strides3(k_new),
                                   L.strides3(v_new), L.ptr(cos), L.ptr(sin), cos.shape[0], int(pos0), L.ptr(cf),
                                   int(block), L.ptr(q_rot), L.ptr(q_pad), L.ptr(k_pad), L.ptr(v_pad), L.ptr(flags),
                                   L.ptr(ck), L.ptr(cv), cst, int(cache_pos), B, H, T, t_pad, D, L.dtype_code(q),
                                   L.stream_ptr(dev))
    L.check(rc, "lmk_chunk_prepare")
    if cache is not None:
        cache.length += T
    return q_rot, q_pad, k_pad, v_pad, flags


class LandmarkKVCache:
    """Preallocated un-rotated key/value cache [B,H,capacity,D] for chunked inference: `append` copies only the new
    chunk, so a layer never re-copies what it already holds (the reference re-concatenates the whole cache on every call,
    llama/llama_mem.py:424-425)."""

    def __init__(self, batch, heads, capacity, dim, dtype, device):
        self.k = torch.empty((batch, heads, capacity, dim), dtype=dtype, device=device)
        self.v = torch.empty((batch, heads, capacity, dim), dtype=dtype, device=device)
        self.length = 0

    def views(self):
        return self.k[:, :, :self.length], self.v[:, :, :self.length]

    def append(self, k_new, v_new):
        n = k_new.shape[2]
        if self.length + n > self.k.shape[2]:
            raise ValueError(f"cache capacity {self.k.shape[2]} exceeded ({self.length} + {n})")
        self.k[:, :, self.length:self.length + n].copy_(k_new)
        self.v[:, :, self.length:self.length + n].copy_(v_new)
        self.length += n
        return self.views()


def _pad_rows(x, rows):
    if x.shape[2] == rows:
        return x.contiguous()
    out = x.new_zeros((*x.shape[:2], rows, x.shape[3]))
    out[:, :, :x.shape[2]] = x
    return out


def llama_retrieval_attention(q, k_new, v_new, past_k=None, past_v=None, mem_freq=None, cache_top_k=None,
                              position_ids=None, chunk_is_mem=None, cos=None, sin=None, return_debug=False,
                              materialize=None, cache=None, aggregate=None, fused=None):
    """Attention of one chunk against a landmark block cache, as LlamaAttention.forward does with
    `mem_freq`/`cache_top_k` set (llama/llama_mem.py:296-298, 318-430, 447-474).

    q, k_new, v_new: [B,H,T,D] projections of the chunk BEFORE rotary; past_k/past_v: [B,H,C,D] un-rotated cache
    (:424,436), or `cache`, a LandmarkKVCache that is appended to in place.  chunk_is_mem: bool [1,T] landmark flags of
    the chunk (default: regular in absolute position).
    aggregate: None = one block selection per (head, token) on the raw scores (the reference's default, :378-384);
      "max_over_tokens" = one selection per head from the softmax of the scores maximised over the chunk's tokens, the
      selected blocks prepended to the keys and the whole thing run through fused landmark attention (the reference's
      route with offload_cache_to_cpu, :369-377, 400-406, 445).
    Three implementations of the default mode, same results within the 16-bit tolerances:
      fused (default where it applies: 16-bit, D=128, no partial block in the cache): local keys through the
        tensor-core operator for arbitrary landmark positions, selected blocks read in place by one kernel that also
        merges the two parts -- no logits, probabilities or gathered copies in memory;
      materialize=False: selected-block logits / value sums read in place, grouped softmax on a logits buffer;
      materialize=True (what the reference does, :386-398): gathered [B,H,T,top_k*block,D] copies and matmuls.
    Returns (attn_output [B,H,T,D], new (past_k, past_v)).
    """
    if cache is not None:
        past_k, past_v = cache.views()
    if materialize is None:
        materialize = return_debug
    B, H, T, D = q.shape
    C = past_k.shape[2]
    block = mem_freq + 1
    dev = q.device
    default_positions = position_ids is None
    if position_ids is None:
        position_ids = torch.arange(C, C + T, device=dev)
    if cos is None:
        cos, sin = rotary_tables_half(C + T + 1, D, q.dtype, dev)
    scale = 1.0 / math.sqrt(D)
    inc = C % block
    t_pad = ((T + 127) // 128) * 128
    if fused is None:
        fused = (not materialize and not return_debug and aggregate is None and inc == 0 and cache_top_k >= 1
                 and C >= block and q.dtype != torch.float32 and D == 128 and t_pad <= 32768)
    one_launch = fused and default_positions and aggregate is None and q.dtype != torch.float32
    if one_launch:
        # rotary of q and k, padded tiles, landmark flags and the cache append in one kernel
        qr, qp, kp, vp, im = chunk_prepare(q, k_new, v_new, cos, sin, C, chunk_is_mem, block, t_pad, cache)
        kr = None
    else:
        qr = apply_rotary_half(q, cos, sin, position_ids)
        kr = apply_rotary_half(k_new, cos, sin, position_ids)
    full = C - inc
    if inc > 0:
        assert T + inc <= block
    num_mems = full // block
    top_k = min(cache_top_k, num_mems)
    prefix_len = full - (top_k + 1) * block
    past_k = past_k if past_k.stride(3) == 1 else past_k.contiguous()
    past_v = past_v if past_v.stride(3) == 1 else past_v.contiguous()
    kst, vst = past_k.stride(), past_v.stride()
    kdesc = L.CacheDesc(kst[0], kst[1], kst[2] * block, kst[2], num_mems, 0, block, top_k, prefix_len)
    vdesc = L.CacheDesc(vst[0], vst[1], vst[2] * block, vst[2], num_mems, 0, block, top_k, prefix_len)

    def new_cache():
        if cache is not None:
            return cache.views() if one_launch else cache.append(k_new, v_new)   # chunk_prepare appended already
        return torch.cat((past_k, k_new), dim=2), torch.cat((past_v, v_new), dim=2)

    if aggregate == "max_over_tokens":
        # one set of blocks per head; the chunk then attends to [selected blocks | chunk] with the regular landmark
        # pattern, which is fused landmark attention with top_k history blocks (:400-406, 445)
        assert inc == 0, "max_over_tokens needs whole blocks in the cache (the fused kernel's history is whole blocks)"
        probs = landmark_scores(qr, past_k, kdesc, cos, sin, L.ROTARY_HALF, scale, softmax=True)
        sel = topk_sorted(probs, top_k, mode="max_over_tokens")                       # [B,H,1,top_k]
        sel_k, sel_v = gather_kv(past_k, past_v, kdesc, vdesc, sel, cos, sin, L.ROTARY_HALF, dim=D)
        from .fused import fused_landmark_attention
        keys = torch.cat((sel_k.view(B, H, top_k * block, D), kr), dim=2)
        vals = torch.cat((sel_v.view(B, H, top_k * block, D), v_new), dim=2)
        out = fused_landmark_attention(qr, keys, vals, None, sm_scale=scale, block_size=block)
        if return_debug:
            return out, new_cache(), dict(scores=probs, sel=sel, sel_k=sel_k, sel_v=sel_v)
        return out, new_cache()
    if aggregate is not None:
        raise NotImplementedError(f"aggregate={aggregate!r}")

    scores = landmark_scores(qr, past_k, kdesc, cos, sin, L.ROTARY_HALF, scale)
    sel = topk_sorted(scores, top_k)
    if chunk_is_mem is None and not one_launch:
        chunk_is_mem = (position_ids % block == block - 1).view(1, T)

    from .masked import _fwd as masked_fwd
    if fused:
        # local part: landmark attention of the chunk over itself on the tensor cores, rows padded to whole tiles
        # (padding keys lie after every real query, so causality hides them); then one kernel for the selected blocks
        # and the merge of the two parts
        assert inc == 0 and not materialize and top_k >= 1
        if not one_launch:
            qp, kp, vp = _pad_rows(qr, t_pad), _pad_rows(kr, t_pad), _pad_rows(v_new, t_pad)
            im = torch.zeros((B, t_pad), dtype=torch.uint8, device=dev)
            im[:, :T] = chunk_is_mem.to(torch.uint8).expand(B, T)
        o_loc, r_loc, _ = masked_fwd(qp, kp, vp, im, scale, 64)
        out = selected_attend(qr, past_k, past_v, kdesc, vdesc, sel, cos, sin, L.ROTARY_HALF, scale, o_loc, r_loc)
        return out, new_cache()

    n_pre = top_k * block
    sel_k = sel_v = None
    if materialize:
        sel_k, sel_v = gather_kv(past_k, past_v, kdesc, vdesc, sel, cos, sin, L.ROTARY_HALF, dim=D)
        prefix = torch.matmul(qr.unsqueeze(3), sel_k.transpose(3, 4)).squeeze(3) * scale      # [B,H,T,top_k*block]

    inc_pos = torch.arange(full, full + inc, device=dev)
    k_inc = apply_rotary_half(past_k[:, :, full:], cos, sin, inc_pos)
    keys = torch.cat((k_inc, kr), dim=2)
    vals = torch.cat((past_v[:, :, full:], v_new), dim=2)
    local = torch.matmul(qr, keys.transpose(2, 3)) * scale
    hidden = torch.ones(T, T, dtype=torch.bool, device=dev).triu(1)
    mask_c, is_mem_c, last_c = prepare_landmark_masks(chunk_is_mem, hidden)
    fmin = torch.finfo(local.dtype).min
    local = torch.cat((local[..., :inc], local[..., inc:].masked_fill(mask_c, fmin)), dim=-1)
    pre_pat = torch.zeros(top_k, block, dtype=torch.bool, device=dev)
    pre_pat[:, block - 1] = True
    is_mem_full = torch.cat((pre_pat.view(1, 1, 1, -1).expand(1, 1, T, -1),
                             torch.zeros(1, 1, T, inc, dtype=torch.bool, device=dev), is_mem_c), dim=-1)
    last_full = torch.cat((torch.zeros(1, 1, T, top_k * block, dtype=torch.bool, device=dev),
                           torch.ones(1, 1, T, inc, dtype=torch.bool, device=dev), last_c), dim=-1)
    if materialize:
        logits = torch.cat((prefix, local), dim=-1)
    else:
        logits = torch.empty((B, H, T, n_pre + local.shape[-1]), device=dev, dtype=q.dtype)
        logits[..., n_pre:] = local
        selected_logits(qr, past_k, kdesc, sel, logits, 0, cos, sin, L.ROTARY_HALF, scale)
    probs = landmark_grouped_softmax(logits, -1, is_mem_full, last_full).to(q.dtype)
    p_local = probs[..., n_pre:]
    if materialize:
        out = torch.matmul(p_local, vals) + torch.matmul(probs[..., :n_pre].unsqueeze(3), sel_v).squeeze(3)
    else:
        out = torch.matmul(p_local, vals) + selected_pv(probs.contiguous(), past_v, vdesc, sel, 0, dim=D)
    if return_debug:
        return out, new_cache(), dict(scores=scores, sel=sel, sel_k=sel_k, sel_v=sel_v, probs=probs)
    return out, new_cache()


class OffloadedLandmarkCache:
    """Landmark block cache whose whole blocks live in pinned HOST memory (llama/llama_mem.py:326-327, 393-398, 427-428:
    the reference's `offload_cache_to_cpu`).

    What stays on the device: the landmark key of every block (1/block of the keys: enough to score all blocks) and the
    unfinished tail block.  What crosses the host link per chunk and layer: only the top_k blocks each head selects
    (one selection per head, the maximum over the chunk's tokens of the softmaxed scores, as the reference does with
    offloading), read by the gather kernel straight from the mapped pinned buffers -- no host round trip for the indices,
    no staging copy -- and, in the other direction, the chunk's finished blocks.
    """

    def __init__(self, batch, heads, capacity_blocks, block, dim, dtype, device):
        self.block, self.capacity = block, capacity_blocks
        self.k_host = torch.empty((batch, heads, capacity_blocks * block, dim), dtype=dtype).pin_memory()
        self.v_host = torch.empty((batch, heads, capacity_blocks * block, dim), dtype=dtype).pin_memory()
        self.lm_keys = torch.empty((batch, heads, capacity_blocks, dim), dtype=dtype, device=device)
        self.tail_k = torch.empty((batch, heads, block, dim), dtype=dtype, device=device)
        self.tail_v = torch.empty((batch, heads, block, dim), dtype=dtype, device=device)
        self.n_blocks, self.tail_len = 0, 0
        self.device = torch.device(device)

    @property
    def length(self):
        return self.n_blocks * self.block + self.tail_len

    def append(self, k_new, v_new):
        """Append un-rotated keys / values [B,H,T,D]: finished blocks go to the host buffers (asynchronous copies on the
        current stream) and their landmark keys to the device array; the rest waits in the device tail."""
        blk = self.block
        k = torch.cat((self.tail_k[:, :, :self.tail_len], k_new), dim=2)
        v = torch.cat((self.tail_v[:, :, :self.tail_len], v_new), dim=2)
        n_full = k.shape[2] // blk
        if self.n_blocks + n_full > self.capacity:
            raise ValueError(f"cache capacity of {self.capacity} blocks exceeded")
        if n_full:
            lo, hi = self.n_blocks * blk, (self.n_blocks + n_full) * blk
            self.k_host[:, :, lo:hi].copy_(k[:, :, :n_full * blk], non_blocking=True)
            self.v_host[:, :, lo:hi].copy_(v[:, :, :n_full * blk], non_blocking=True)
            self.lm_keys[:, :, self.n_blocks:self.n_blocks + n_full].copy_(k[:, :, blk - 1:n_full * blk:blk])
            self.n_blocks += n_full
        self.tail_len = k.shape[2] - n_full * blk
        self.tail_k[:, :, :self.tail_len].copy_(k[:, :, n_full * blk:])
        self.tail_v[:, :, :self.tail_len].copy_(v[:, :, n_full * blk:])

    def attend(self, q, k_new, v_new, cache_top_k, cos=None, sin=None, return_debug=False):
        """Attention of the chunk q, k_new, v_new [B,H,T,D] (before rotary) over [selected blocks | chunk], then
        `append`.  Same result as llama_retrieval_attention(..., aggregate="max_over_tokens") on a device-resident
        cache with the same contents."""
        from .fused import fused_landmark_attention
        assert self.tail_len == 0, "offloaded attention needs whole blocks in the cache (as the fused route does)"
        B, H, T, D = q.shape
        blk, n, C = self.block, self.n_blocks, self.n_blocks * self.block
        dev = q.device
        if cos is None:
            cos, sin = rotary_tables_half(C + T + 1, D, q.dtype, dev)
        scale = 1.0 / math.sqrt(D)
        pos = torch.arange(C, C + T, device=dev)
        qr, kr = apply_rotary_half(q, cos, sin, pos), apply_rotary_half(k_new, cos, sin, pos)
        top_k = min(cache_top_k, n)
        prefix_len = C - (top_k + 1) * blk
        ls = self.lm_keys.stride()
        lmdesc = L.CacheDesc(ls[0], ls[1], ls[2], 0, n, 0, blk, top_k, prefix_len)
        hs = self.k_host.stride()
        hdesc = L.CacheDesc(hs[0], hs[1], hs[2] * blk, hs[2], n, 0, blk, top_k, prefix_len)
        probs = landmark_scores(qr, self.lm_keys, lmdesc, cos, sin, L.ROTARY_HALF, scale, softmax=True)
        sel = topk_sorted(probs, top_k, mode="max_over_tokens")                       # [B,H,1,top_k], on the device
        # the gather kernel reads the selected blocks from the mapped pinned buffers: top_k * block rows per head
        sel_k, sel_v = _gather_from_host(self.k_host, self.v_host, hdesc, sel, cos, sin, D, dev)
        keys = torch.cat((sel_k.view(B, H, top_k * blk, D), kr), dim=2)
        vals = torch.cat((sel_v.view(B, H, top_k * blk, D), v_new), dim=2)
        out = fused_landmark_attention(qr, keys, vals, None, sm_scale=scale, block_size=blk)
        self.append(k_new, v_new)
        if return_debug:
            return out, dict(sel=sel, sel_k=sel_k, sel_v=sel_v)
        return out


def _gather_from_host(k_host, v_host, desc, idx, cos, sin, dim, device):
    """lmk_gather_kv with the cache pointers in pinned (mapped) host memory and the outputs on the device."""
    B, H, T, top_k = idx.shape
    k_out = torch.empty((B, H, T, top_k * desc.block, dim), device=device, dtype=k_host.dtype)
    v_out = torch.empty_like(k_out)
    assert k_host.is_pinned() and v_host.is_pinned()
    rc = L.lib().lmk_gather_kv(L.ptr(k_host), L.ptr(v_host), ctypes.byref(desc), ctypes.byref(desc), L.ptr(idx),
                               L.ptr(cos), L.ptr(sin), cos.shape[0], L.ROTARY_HALF, L.ptr(k_out), L.ptr(v_out), B, H, T,
                               dim, L.dtype_code(k_host), L.stream_ptr(device))
    L.check(rc, "lmk_gather_kv")
    return k_out, v_out
