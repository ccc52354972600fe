"""CPU oracle for the landmark-attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-on-CPU tensor code, what the reference
(epfml/landmark-attention) computes on its hot path.  Nothing in the shipped
package may import it: it exists so that tests, the smoke check and the CPU
baseline leg of the benchmark have something independent to compare the CUDA
kernels with.  Every function names the reference lines it follows.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
Python (its high-level grouped softmax, its Triton kernels under the Triton
interpreter, its LLaMA retrieval branch and its lm_benchmark block cache) on
seeded inputs and stores the results; `tests/test_oracle_golden.py` checks this
oracle against those stored results.

The restatement is deliberately written differently from the reference (direct
per-group arithmetic on a [.., n_blocks, block] view instead of
scatter/gather on an int64 index tensor) so that agreement means something.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

NEG_INF = float("-inf")


# ----------------------------------------------------------------------------
# Fused landmark attention (regular landmark pattern)
# ----------------------------------------------------------------------------

def regular_is_mem(length: int, block_size: int, device="cpu") -> torch.Tensor:
    """Landmark = last token of every block.
    Reference: llama/ltriton/flash_landmark_attention.py:393."""
    return torch.arange(length, device=device) % block_size == block_size - 1


def landmark_attention_probs(q, k, block_size: int, sm_scale: Optional[float] = None,
                             return_stats: bool = False):
    """Attention probabilities of fused landmark attention, [B,H,Lq,Lk].

    Semantics (llama/ltriton/flash_landmark_attention.py:47-113, equal to the
    high-level recipe llama/ltriton/test_flash_landmark_attention.py:105-125):
    query row i sits at key position p = (Lk-Lq)+i in block b = p // block.
      * keys of its own block are visible causally (j <= p) except the block's
        own landmark, which no row sees (the landmark query is shifted back one
        position, :29-30,94);
      * every earlier block n < b contributes its landmark score l_n to an outer
        softmax taken over {l_n} U {visible own-block scores};
      * the non-landmark keys of an earlier block share that block's outer
        probability, split by a softmax inside the block (:57-61,76);
      * landmark keys themselves carry no value weight.
    With return_stats, also returns (M, L): the max and the sum of exponentials
    of the outer softmax, which the reference kernel stores (:116-119).
    """
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    blk = block_size
    assert (Lk - Lq) % blk == 0 and Lk % blk == 0
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    nb = Lk // blk
    s = torch.matmul(q, k.transpose(-1, -2)) * sm_scale          # [B,H,Lq,Lk]
    s4 = s.view(B, H, Lq, nb, blk)
    pos = torch.arange(Lq, device=q.device) + (Lk - Lq)           # key position of each query
    own = pos // blk                                              # own block of each query
    blocks = torch.arange(nb, device=q.device)
    earlier = blocks[None, :] < own[:, None]                      # [Lq, nb]

    inner = torch.softmax(s4[..., : blk - 1], dim=-1)             # softmax inside every block
    lm = s4[..., blk - 1].masked_fill(~earlier, NEG_INF)          # landmark scores of earlier blocks

    own_scores = torch.gather(
        s4, 3, own.view(1, 1, Lq, 1, 1).expand(B, H, Lq, 1, blk)).squeeze(3)   # [B,H,Lq,blk]
    local = torch.arange(blk, device=q.device)
    own_visible = (local[None, :] <= (pos - own * blk)[:, None]) & (local[None, :] != blk - 1)
    own_scores = own_scores.masked_fill(~own_visible, NEG_INF)

    outer_logits = torch.cat((lm, own_scores), dim=-1)            # [B,H,Lq,nb+blk]
    outer = torch.softmax(outer_logits, dim=-1)
    w, p_own = outer[..., :nb], outer[..., nb:]

    p4 = torch.cat((inner * w.unsqueeze(-1), torch.zeros_like(w).unsqueeze(-1)), dim=-1)
    own_onehot = (blocks[None, :] == own[:, None]).view(1, 1, Lq, nb, 1)
    p4 = torch.where(own_onehot, p_own.unsqueeze(3), p4)
    probs = p4.reshape(B, H, Lq, Lk)
    if return_stats:
        m = outer_logits.amax(dim=-1)
        l = torch.exp(outer_logits - m.unsqueeze(-1)).sum(dim=-1)
        return probs, m, l
    return probs


def landmark_attention(q, k, v, block_size: int, sm_scale: Optional[float] = None,
                       return_stats: bool = False):
    """out = P @ V with P from landmark_attention_probs.
    Reference: `fused_landmark_attention`, flash_landmark_attention.py:391-403."""
    if return_stats:
        p, m, l = landmark_attention_probs(q, k, block_size, sm_scale, True)
        return torch.matmul(p, v), m, l
    return torch.matmul(landmark_attention_probs(q, k, block_size, sm_scale), v)


def landmark_attention_grads(q, k, v, do, block_size: int, sm_scale: Optional[float] = None):
    """(out, dq, dk, dv) by autograd through the restatement above.
    Stands for FusedLandmarkAttention.backward, flash_landmark_attention.py:356-389."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    out = landmark_attention(q, k, v, block_size, sm_scale)
    dq, dk, dv = torch.autograd.grad(out, [q, k, v], do)
    return out.detach(), dq, dk, dv


# ----------------------------------------------------------------------------
# Mask preparation done by the call sites
# ----------------------------------------------------------------------------

def prepare_landmark_masks(is_mem_row: torch.Tensor, attn_mask: torch.Tensor):
    """Mask block of the attention call sites.

    is_mem_row: bool [B, Lk] (per batch row); attn_mask: bool [.., Lq, Lk], True = hidden.
    Returns (mask, is_mem, last_section) each bool [B, 1, Lq, Lk] as the reference
    builds them: lm_benchmark/models/landmark.py:210-224 and llama/llama_mem.py:807-815.
      mem_ids      = number of landmarks strictly before each key (0 where hidden)
      last_section = keys whose mem_ids equals the row maximum (the query's own block)
      mask         = hidden OR (landmark of the own block)
    """
    B, Lk = is_mem_row.shape
    im = is_mem_row.view(B, 1, 1, Lk)
    attn_mask = attn_mask.view(*([1] * (4 - attn_mask.dim())), *attn_mask.shape)
    before = torch.cumsum(im.to(torch.int64), dim=-1) - im.to(torch.int64)
    mem_ids = torch.where(attn_mask, torch.zeros_like(before), before)
    last = mem_ids == mem_ids.amax(dim=-1, keepdim=True)
    mask = attn_mask | (im & last)
    last = last & ~mask
    is_mem = im & ~mask
    return mask, is_mem, last


# ----------------------------------------------------------------------------
# Stand-alone grouped softmax (arbitrary landmark positions)
# ----------------------------------------------------------------------------

def grouped_softmax(x, is_mem, last_section, attn_mask=None, guards: bool = False,
                    return_group_prob: bool = False, max_mem_cnt: Optional[int] = None):
    """Landmark grouped softmax over the last dim.

    llama flavour (guards=False): llama/llama_mem.py:168-243.
    lm_benchmark flavour (guards=True, attn_mask given): lm_benchmark/models/landmark.py:37-119.

    Per row: keys that are neither landmark nor "last section" (nor, in the
    lm_benchmark flavour, hidden by attn_mask) fall into group g = number of
    landmarks at or before them; the bucket holds last-section keys, landmarks
    and (lm_benchmark) hidden keys.  A softmax is taken inside every group and
    inside the bucket (:175-186).  The landmark that closes group g carries
    that group's probability (:238-239); each grouped key's inner probability
    is multiplied by it; bucket members keep their probability only if they are
    last-section keys (:240).  guards: an all -inf group gives 0 instead of NaN
    (landmark.py:48,54).
    Returns probs in fp32 (and group_prob [.., max_mem_cnt] when asked:
    landmark.py:107-116, slot g = landmark closing group g, last slot = total
    last-section probability).
    """
    xf = x.to(torch.float32) if x.dtype not in (torch.float32, torch.float64) else x
    shape = torch.broadcast_shapes(x.shape, is_mem.shape, last_section.shape)
    is_mem = is_mem.expand(shape)
    last_section = last_section.expand(shape)
    hidden = attn_mask.expand(shape) if attn_mask is not None else torch.zeros(shape, dtype=torch.bool)
    Lk = shape[-1]
    csum = torch.cumsum(is_mem.to(torch.int64), dim=-1)
    bucket = last_section | hidden | is_mem
    n_groups = int(csum.max().item()) + 1
    gid = torch.where(bucket, torch.full_like(csum, n_groups), csum)     # bucket id = n_groups
    onehot = torch.nn.functional.one_hot(gid, n_groups + 1).to(torch.bool)   # [.., Lk, G+1]
    xg = xf.unsqueeze(-1).masked_fill(~onehot, NEG_INF)
    gmax = xg.amax(dim=-2)                                                # [.., G+1]
    mx = torch.gather(gmax, -1, gid)
    if guards:
        mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    e = torch.exp(xf - mx)
    gsum = (e.unsqueeze(-1) * onehot).sum(dim=-2)
    den = torch.gather(gsum, -1, gid)
    inner = e / den
    if guards:
        inner = torch.where(den < 0.5, torch.zeros_like(inner), inner)
    # probability of the landmark closing each group: landmark j closes group csum[j]-1
    closes = torch.where(is_mem, csum - 1, torch.full_like(csum, n_groups))
    gp = torch.zeros(*shape[:-1], n_groups + 1, dtype=inner.dtype)
    gp.scatter_(-1, closes, torch.where(is_mem, inner, torch.zeros_like(inner)))
    weight = torch.gather(gp, -1, torch.clamp(gid, max=n_groups))
    probs = torch.where(bucket, inner * last_section.to(inner.dtype), inner * weight)
    if return_group_prob:
        assert max_mem_cnt is not None and max_mem_cnt >= n_groups + 1
        out = torch.zeros(*shape[:-1], max_mem_cnt, dtype=inner.dtype)
        out[..., : n_groups] = gp[..., : n_groups]
        out[..., max_mem_cnt - 1] = (inner * last_section.to(inner.dtype)).sum(dim=-1)
        return probs, out
    return probs


# ----------------------------------------------------------------------------
# Rotary position helpers
# ----------------------------------------------------------------------------

def rotary_half_split(x, positions, base: float = 10000.0):
    """LLaMA rotary: pair (d, d + D/2), angle = pos * base^(-2d/D).
    Reference: llama/llama_mem.py:96-149.  positions broadcast against x[..., :-1].
    The tables are built in fp32 and cast to x's dtype before use (:121-122)."""
    D = x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = positions.to(torch.float32).unsqueeze(-1) * inv
    emb = torch.cat((ang, ang), dim=-1)
    cos, sin = emb.cos().to(x.dtype), emb.sin().to(x.dtype)
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat((-x2, x1), dim=-1) * sin


def rotary_interleaved(x, positions):
    """lm_benchmark rotary: pair (2d, 2d+1), angle = pos * 10^(-4*2d/D).
    Reference: lm_benchmark/models/positional_encoders/rotary.py:24-55 and
    rotary_utils.py:17-31.  cos/sin are cast to x's dtype before the multiply."""
    D = x.shape[-1]
    freqs = 10.0 ** (-4.0 * torch.arange(0, D, 2, dtype=torch.float32)[: D // 2] / D)
    ang = (positions.unsqueeze(-1) * freqs).unsqueeze(-1).expand(*positions.shape, D // 2, 2)
    ang = ang.reshape(*positions.shape, D)
    xr = x.reshape(*x.shape[:-1], D // 2, 2)
    rot = torch.stack((-xr[..., 1], xr[..., 0]), dim=-1).reshape(x.shape)
    return x * ang.cos().to(x.dtype) + rot * ang.sin().to(x.dtype)


# ----------------------------------------------------------------------------
# Retrieval: LLaMA cache branch
# ----------------------------------------------------------------------------

def sorted_topk(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries along the last dim, in ascending index order.
    Reference: llama/llama_mem.py:384 (`topk(...)[1].sort(...)[0]`)."""
    return scores.topk(k, dim=-1).indices.sort(dim=-1).values


def llama_slot_positions(num_mems: int, top_k: int, full_len: int, block: int):
    """Positions at which cached landmark keys are rotated for scoring.
    Reference: llama/llama_mem.py:359-366.  All but the newest top_k landmarks share slot 0;
    the newest top_k take slots 1..top_k of a window of top_k+1 blocks ending at full_len."""
    prefix_len = full_len - (top_k + 1) * block
    slots = torch.cat((torch.zeros(max(0, num_mems - top_k), dtype=torch.long),
                       torch.arange(1, top_k + 1, dtype=torch.long)))
    return slots * block + (block - 1) + prefix_len, prefix_len


def llama_selected_key_positions(sel_idx, num_mems: int, top_k: int, prefix_len: int, block: int):
    """Positions of the keys of retrieved blocks: the i-th (ascending) retrieved block sits in slot i,
    or slot i+1 if it is one of the newest top_k.  Reference: llama/llama_mem.py:386-388."""
    base = torch.arange(top_k * block, dtype=torch.long).view(top_k, block)
    shift = torch.where(sel_idx >= num_mems - top_k, block, 0).unsqueeze(-1)
    return (shift + base).flatten(-2) + prefix_len


def llama_retrieval_attention(q, k_new, v_new, past_k, past_v, block: int, top_k: int,
                              position_ids=None, chunk_is_mem=None, return_debug: bool = False, sel=None):
    """LLaMA long-context attention with landmark retrieval (mode A: per head and token).

    Reference: LlamaAttention.forward cache branch, llama/llama_mem.py:296-298,318-430,447-474,
    with the mask preparation of LlamaModel.forward :807-815.
    q,k_new,v_new: [B,H,T,D] un-rotated projections of the current chunk, chunk tokens at
    positions position_ids (default: cache_len.. as the model does, :789-793);
    past_k/past_v: [B,H,C,D] un-rotated cache.  The chunk's landmark pattern is regular in
    absolute position (token at position p is a landmark iff p % block == block-1) unless
    chunk_is_mem (bool [1,T]) says otherwise.
    sel (int64 [B,H,T,top_k], optional): use this block selection instead of the top-k of this function's own scores
    (parity of 16-bit kernels is defined "given the same landmark scores": near-ties would otherwise flip).
    Returns [B,H,T,D].
    """
    B, H, T, D = q.shape
    C = past_k.shape[2]
    scale = 1.0 / math.sqrt(D)
    sel_given = sel
    if position_ids is None:
        position_ids = torch.arange(C, C + T, dtype=torch.long)
    qr = rotary_half_split(q, position_ids.view(1, 1, T))
    kr = rotary_half_split(k_new, position_ids.view(1, 1, T))
    inc = C % block
    full = C - inc
    past_k_full, past_k_inc = past_k[:, :, :full], past_k[:, :, full:]
    past_v_full, past_v_inc = past_v[:, :, :full], past_v[:, :, full:]
    if inc > 0:
        assert T + inc <= block
    inc_pos = torch.arange(full, full + inc, dtype=torch.long)
    k_inc = rotary_half_split(past_k_inc, inc_pos.view(1, 1, inc))
    keys = torch.cat((k_inc, kr), dim=2)
    vals = torch.cat((past_v_inc, v_new), dim=2)
    kb = past_k_full.view(B, H, -1, block, D)
    vb = past_v_full.view(B, H, -1, block, D)
    num_mems = kb.shape[2]
    tk = min(top_k, num_mems)
    mem_pos, prefix_len = llama_slot_positions(num_mems, tk, full, block)
    lm_keys = rotary_half_split(kb[:, :, :, block - 1], mem_pos.view(1, 1, num_mems))
    scores = torch.matmul(qr, lm_keys.transpose(2, 3)) / math.sqrt(D)       # [B,H,T,num_mems]
    sel = sorted_topk(scores, tk) if sel_given is None else sel_given       # [B,H,T,tk]
    key_pos = llama_selected_key_positions(sel, num_mems, tk, prefix_len, block)  # [B,H,T,tk*block]
    gidx = sel.view(B, H, T, tk, 1, 1).expand(B, H, T, tk, block, D)
    sel_k = torch.take_along_dim(kb.unsqueeze(2).expand(B, H, T, num_mems, block, D), gidx, dim=3)
    sel_v = torch.take_along_dim(vb.unsqueeze(2).expand(B, H, T, num_mems, block, D), gidx, dim=3)
    sel_k = rotary_half_split(sel_k.reshape(B, H, T, tk * block, D), key_pos)
    sel_v = sel_v.reshape(B, H, T, tk * block, D)
    prefix = torch.matmul(qr.unsqueeze(3), sel_k.transpose(3, 4)).squeeze(3) / math.sqrt(D)
    local = torch.matmul(qr, keys.transpose(2, 3)) / math.sqrt(D)           # [B,H,T,inc+T]

    # masks: local part (model-level prep on the chunk, then cache columns prepended)
    causal_hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    if chunk_is_mem is None:
        chunk_is_mem = (position_ids % block == block - 1).view(1, T)
    mask_c, is_mem_c, last_c = prepare_landmark_masks(chunk_is_mem, causal_hidden)
    local = torch.cat((local[..., :inc], local[..., inc:].masked_fill(mask_c, torch.finfo(local.dtype).min)), -1)
    is_mem_full = torch.cat((
        torch.cat((torch.zeros(block - 1, dtype=torch.bool), torch.ones(1, dtype=torch.bool))).repeat(tk)
        .view(1, 1, 1, -1).expand(1, 1, T, -1),
        torch.zeros(1, 1, T, inc, dtype=torch.bool), is_mem_c), dim=-1)
    last_full = torch.cat((torch.zeros(1, 1, T, tk * block, dtype=torch.bool),
                           torch.ones(1, 1, T, inc, dtype=torch.bool), last_c), dim=-1)
    logits = torch.cat((prefix, local), dim=-1)
    probs = grouped_softmax(logits, is_mem_full, last_full).to(q.dtype)
    p_prefix, p_local = probs[..., : tk * block], probs[..., tk * block:]
    out = torch.matmul(p_local, vals) + torch.matmul(p_prefix.unsqueeze(3), sel_v).squeeze(3)
    if return_debug:
        return out, dict(scores=scores, sel=sel, key_pos=key_pos, mem_pos=mem_pos, probs=probs)
    return out


# ----------------------------------------------------------------------------
# Retrieval: lm_benchmark block cache
# ----------------------------------------------------------------------------

class BlockCacheOracle:
    """Restatement of MemLMCacheStorage (lm_benchmark/models/caches/mem_cache.py:21-158).

    Keeps the cached blocks as a plain Python list in LOGICAL order (oldest first) instead of a
    ring buffer; physical slot numbers are derived when indices have to be reported the way the
    reference reports them.
    """

    def __init__(self, capacity: int, block: int, top_k: int, selection: str = "per_token_and_head"):
        self.capacity, self.block, self.top_k, self.selection = capacity, block, top_k, selection
        self.clear_state()

    def clear_state(self):                       # mem_cache.py:36-39
        self.blocks_k, self.blocks_v = [], []    # each [B,H,block,D], logical order
        self.tail_k = self.tail_v = self.tail_is_mem = None
        self.total_blocks = 0

    @property
    def cache_iter(self):                        # next physical slot, mem_cache.py:140-158
        return self.total_blocks % self.capacity

    def store(self, k, v, is_mem):               # mem_cache.py:111-158
        if self.tail_k is not None:
            k = torch.cat((self.tail_k, k), dim=2)
            v = torch.cat((self.tail_v, v), dim=2)
            is_mem = torch.cat((self.tail_is_mem, is_mem), dim=1)
        T = k.shape[2]
        inc = T % self.block
        full = T - inc
        self.tail_k, self.tail_v, self.tail_is_mem = k[:, :, full:], v[:, :, full:], is_mem[:, full:]
        if inc == 0:
            self.tail_k = self.tail_v = self.tail_is_mem = None
        im = is_mem[:, :full].view(is_mem.shape[0], -1, self.block)
        assert bool(im[..., -1].all()) and not bool(im[..., :-1].any())
        for n in range(full // self.block):
            self.blocks_k.append(k[:, :, n * self.block:(n + 1) * self.block])
            self.blocks_v.append(v[:, :, n * self.block:(n + 1) * self.block])
            self.total_blocks += 1
        self.blocks_k = self.blocks_k[-self.capacity:]
        self.blocks_v = self.blocks_v[-self.capacity:]

    def retrieve(self, q, start_index: int):
        """q: [B,H,T,D] rotated queries.  Returns (att_prefix, v_prefix, is_mem_prefix, debug).
        Follows retrieve_for_query, mem_cache.py:41-109 (rotary = lm_benchmark interleaved)."""
        B, H, T, D = q.shape
        blk, scale = self.block, 1.0 / math.sqrt(D)
        tail_len = 0 if self.tail_k is None else self.tail_k.shape[2]
        if tail_len:
            pos = torch.arange(start_index - tail_len, start_index)
            tk_ = rotary_interleaved(self.tail_k, pos.view(1, 1, tail_len).expand(B, H, tail_len).to(torch.float32))
            att_inc = torch.matmul(q, tk_.transpose(-2, -1)) * scale
            v_inc = self.tail_v.unsqueeze(2).expand(B, H, T, tail_len, D)
            mem_inc = self.tail_is_mem
        else:
            att_inc = q.new_zeros(B, H, T, 0)
            v_inc = q.new_zeros(B, H, T, 0, D)
            mem_inc = torch.zeros(B, 0, dtype=torch.bool)
        n = len(self.blocks_k)
        if n == 0 or self.top_k == 0:
            return att_inc, v_inc, mem_inc, {}
        top_k = self.top_k
        kb = torch.stack(self.blocks_k, dim=2)                 # [B,H,n,blk,D] logical order
        vb = torch.stack(self.blocks_v, dim=2)
        logical = torch.arange(n)
        slot = torch.where(logical >= n - top_k, logical - (n - top_k) + 1, torch.zeros_like(logical))
        lm_pos = (slot * blk + blk - 1).to(torch.float32)
        lm = rotary_interleaved(kb[:, :, :, blk - 1], lm_pos.view(1, 1, n).expand(B, H, n))
        att = torch.softmax(torch.matmul(q, lm.transpose(-2, -1)) * scale, dim=-1)   # [B,H,T,n]
        if self.selection == "max_over_heads":
            att = att.amax(dim=1, keepdim=True).expand(B, H, T, n)
        elif self.selection == "max_over_tokens":
            att = att.amax(dim=2, keepdim=True).expand(B, H, T, n)
        elif self.selection != "per_token_and_head":
            raise NotImplementedError
        sel = att.topk(top_k, dim=-1).indices.sort(dim=-1).values             # logical, ascending
        gi = sel.view(B, H, T, top_k, 1, 1).expand(B, H, T, top_k, blk, D)
        sk = torch.take_along_dim(kb.unsqueeze(2).expand(B, H, T, n, blk, D), gi, dim=3)
        sv = torch.take_along_dim(vb.unsqueeze(2).expand(B, H, T, n, blk, D), gi, dim=3)
        chosen_slot = slot[sel]                                               # [B,H,T,top_k]
        kpos = ((chosen_slot > 0).to(torch.long) * blk).unsqueeze(-1) + \
            torch.arange(top_k * blk).view(top_k, blk)
        kpos = kpos.reshape(B, H, T, top_k * blk)
        sk = rotary_interleaved(sk.reshape(B, H, T, top_k * blk, D), kpos.to(torch.float32))
        att_k = torch.matmul(q.unsqueeze(3), sk.transpose(-2, -1)).squeeze(3) * scale
        is_mem = torch.cat((torch.zeros(B, top_k, blk - 1, dtype=torch.bool),
                            torch.ones(B, top_k, 1, dtype=torch.bool)), dim=-1).view(B, -1)
        # physical slot of logical block i: the oldest surviving block sits at cache_iter once full
        first_phys = self.cache_iter if self.total_blocks >= self.capacity else 0
        phys = (sel + first_phys) % max(n, 1)
        dbg = dict(sel_logical=sel, sel_physical=phys, key_pos=kpos, lm_pos=lm_pos)
        return (torch.cat((att_k, att_inc), dim=-1),
                torch.cat((sv.reshape(B, H, T, top_k * blk, D), v_inc), dim=-2),
                torch.cat((is_mem, mem_inc), dim=-1), dbg)


def insert_landmarks(ids: torch.Tensor, mem_freq: int, landmark_id: int, carry: int = 0):
    """Insert landmark_id after every mem_freq real tokens; `carry` real tokens of an unfinished
    block precede this chunk.  Returns (new ids, new carry).
    Reference: MemLMCache.forward, lm_benchmark/models/caches/mem_cache.py:178-200."""
    out = []
    B, T = ids.shape
    c = carry
    for t in range(T):
        out.append(ids[:, t:t + 1])
        c += 1
        if c == mem_freq:
            out.append(torch.full((B, 1), landmark_id, dtype=ids.dtype))
            c = 0
    return torch.cat(out, dim=1) if out else ids, c


def strip_landmarks(x: torch.Tensor, mem_freq: int, carry_before: int):
    """Drop the positions insert_landmarks added (x: [B,T',C]).
    Reference: MemLMCache.get_final_logits, mem_cache.py:202-217."""
    keep, c = [], carry_before
    for t in range(x.shape[1]):
        if c == mem_freq:
            c = 0
            continue
        keep.append(t)
        c += 1
    return x[:, keep]


# ----------------------------------------------------------------------------
# lm_benchmark attention call site (training path, arbitrary landmark positions)
# ----------------------------------------------------------------------------

def lm_attention(q, k, v, is_mem_row, sm_scale: Optional[float] = None, att_prefix=None, v_prefix=None,
                 is_mem_prefix=None):
    """Attention of lm_benchmark's CausalSelfAttention: q,k already rotated.
    Reference: lm_benchmark/models/landmark.py:196-236 (softmax_func = landmark_grouped_softmax).
    With a cache (landmark.py:182-209, 236-243): att_prefix [B,H,T,P] are the scaled scores against the retrieved
    keys, v_prefix [B,H,T,P,D] (or [B,H,P,D]) their values and is_mem_prefix [B,P] their landmark flags; the prefix
    columns are visible to every query and join the same grouped softmax in front of the chunk's own keys."""
    B, H, T, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    att = torch.matmul(q, k.transpose(-2, -1)) * sm_scale
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    n_pre = 0
    if att_prefix is not None:
        n_pre = att_prefix.shape[-1]
        att = torch.cat((att_prefix, att), dim=-1)                                     # :201-203
        pre_mem = is_mem_prefix if is_mem_prefix is not None else torch.zeros(B, n_pre, dtype=torch.bool)
        is_mem_row = torch.cat((pre_mem, is_mem_row), dim=-1)                          # :204-207
        hidden = torch.cat((torch.zeros(T, n_pre, dtype=torch.bool), hidden), dim=-1)  # :208
    mask, is_mem, last = prepare_landmark_masks(is_mem_row, hidden)
    att = att.masked_fill(mask, NEG_INF)
    p = grouped_softmax(att, is_mem, last, attn_mask=mask, guards=True)
    y = torch.matmul(p[..., n_pre:].to(v.dtype), v)
    if n_pre:
        pp = p[..., :n_pre].to(v.dtype)
        y = y + (torch.matmul(pp, v_prefix) if v_prefix.dim() == 4                    # :238-243
                 else torch.matmul(pp.unsqueeze(3), v_prefix).squeeze(3))
    return y
