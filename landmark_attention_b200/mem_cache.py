"""lm_benchmark's landmark block cache on this package's retrieval kernels.

Same interface as the reference (lm_benchmark/models/caches/cache.py:17-35, mem_cache.py:21-217):
`retrieve_for_query(q, cache_context, pos_emb_closure, start_index)`, `store_in_cache(keys, values_dict)`,
`clear_state()`, and the id bookkeeping of `MemLMCache.forward / get_final_logits`.
The ring buffer keeps the reference's layout [B, capacity, block, H, D] by default; `layout="head_major"` stores it as
[B, H, capacity, block, D], where a block of one head is one contiguous run of block * D elements (the gather then reads
whole blocks instead of `block` separate rows).  In both layouts `store_in_cache` also keeps the blocks' landmark keys
in a dense [B, H, capacity, D] array, which is what the scoring kernel reads.  Selection, the gather, the rotation of
gathered keys and the block writes run in CUDA kernels; the rotary convention is lm_benchmark's interleaved one.
"""
import ctypes
import math

import torch
from torch import nn

from . import _lib as L
from .retrieval import gather_kv, landmark_scores, rotary_tables_interleaved, topk_sorted


def _rotate_interleaved(x, cos, sin, positions):
    c, s = cos[positions], sin[positions]
    xr = x.reshape(*x.shape[:-1], x.shape[-1] // 2, 2)
    rot = torch.stack((-xr[..., 1], xr[..., 0]), dim=-1).reshape(x.shape)
    return x * c + rot * s


def _require_plain_rotary(closure, hs):
    """Accept None or a closure whose encoder is lm_benchmark's RotaryPositionalEncoder: same class name, the
    interleaved-pair frequencies 10^(-4 i / hs), and no attention-matrix adaptation."""
    if closure is None:
        return
    enc = getattr(closure, "encoder", None)
    freqs = getattr(enc, "freqs", None)
    ok = type(closure).__name__ == "RotaryPositionalEncoderClosure" and freqs is not None and freqs.numel() == hs // 2
    if ok:
        want = 10 ** (-4 * torch.arange(0, hs, 2, device=freqs.device)[: hs // 2].float() / hs)
        ok = torch.allclose(freqs.float(), want, rtol=1e-6, atol=0)
    if not ok:
        raise NotImplementedError("MemLMCacheStorage applies lm_benchmark's plain rotary encoding inside its kernels; "
                                  f"the positional encoder closure {type(closure).__name__} is not supported")


class MemLMCacheStorage(nn.Module):
    """Per-layer storage (mem_cache.py:21-158).  `config` needs batch_size, mem_cache_size, mem_cache_freq, n_head,
    n_embd, cache_topk, cache_selection_method."""

    def __init__(self, config, layer=None, dtype=torch.float32, device="cuda", layout="reference"):
        super().__init__()
        self.config = config
        hs = config.n_embd // config.n_head
        blk = config.mem_cache_freq + 1
        if layout == "reference":
            shape = (config.batch_size, config.mem_cache_size, blk, config.n_head, hs)
        elif layout == "head_major":
            shape = (config.batch_size, config.n_head, config.mem_cache_size, blk, hs)
        else:
            raise ValueError(f"unknown cache layout {layout!r}")
        self.layout = layout
        self.register_buffer("cache_mem_k", torch.empty(shape, dtype=dtype, device=device), persistent=False)
        self.register_buffer("cache_mem_v", torch.empty(shape, dtype=dtype, device=device), persistent=False)
        lm_shape = (config.batch_size, config.n_head, config.mem_cache_size, hs)
        self.register_buffer("cache_lm_k", torch.empty(lm_shape, dtype=dtype, device=device), persistent=False)
        tail = (config.batch_size, config.n_head, blk, hs)
        self.register_buffer("last_incomplete_k", torch.empty(tail, dtype=dtype, device=device), persistent=False)
        self.register_buffer("last_incomplete_v", torch.empty(tail, dtype=dtype, device=device), persistent=False)
        self.register_buffer("last_incomplete_ismem",
                             torch.empty((config.batch_size, blk), dtype=torch.bool, device=device), persistent=False)
        self._tables = None
        self.clear_state()

    def clear_state(self):
        self.last_incomplete_len = 0
        self.cache_iter = 0
        self.cache_size = 0

    @property
    def block(self):
        return self.config.mem_cache_freq + 1

    @property
    def capacity(self):
        return self.config.mem_cache_size

    def _descs(self, n, ring_start, top_k):
        """(key, value, landmark-key) descriptors addressed as (batch, head, block slot, row)."""
        def order(st):
            return (st[0], st[3], st[1], st[2]) if self.layout == "reference" else (st[0], st[1], st[2], st[3])
        blk = self.block
        k = L.CacheDesc(*order(self.cache_mem_k.stride()), n, ring_start, blk, top_k, 0)
        v = L.CacheDesc(*order(self.cache_mem_v.stride()), n, ring_start, blk, top_k, 0)
        ls = self.cache_lm_k.stride()
        lm = L.CacheDesc(ls[0], ls[1], ls[2], 0, n, ring_start, blk, top_k, 0)      # every "row" of a slot is its landmark key
        return k, v, lm

    def _rotary(self, n_pos, dim, dtype, device):
        if self._tables is None or self._tables[0].shape[0] < n_pos or self._tables[0].dtype != dtype:
            self._tables = rotary_tables_interleaved(max(n_pos, 4096), dim, dtype, device)
        return self._tables

    def retrieve_for_query(self, q, cache_context, pos_emb_closure, start_index):
        """mem_cache.py:41-109.  Positions are applied inside the kernels with lm_benchmark's plain rotary tables
        (positional_encoders/rotary.py), so `pos_emb_closure` must be None or the closure of that encoder; any other
        encoder (rotary_mem_jump, or one that adapts the attention matrix) is refused instead of silently giving other
        key rotations than the model expects."""
        _require_plain_rotary(pos_emb_closure, q.shape[-1])
        B, nh, T, hs = q.shape
        blk, cap = self.block, self.capacity
        top_k = self.config.cache_topk
        scale = 1.0 / math.sqrt(hs)
        cos, sin = self._rotary(max(start_index + T, (top_k + 2) * blk) + 1, hs, q.dtype, q.device)
        inc = self.last_incomplete_len
        tail_pos = torch.arange(start_index - inc, start_index, device=q.device)
        tail_k = _rotate_interleaved(self.last_incomplete_k[:B, :, :inc], cos, sin, tail_pos)
        att_incomplete = (q @ tail_k.transpose(-2, -1)) * scale
        last_v = self.last_incomplete_v[:B, :, :inc].unsqueeze(2).expand(B, nh, T, inc, hs)
        last_mem = self.last_incomplete_ismem[:B, :inc]
        if self.cache_size == 0 or top_k == 0:
            return att_incomplete, {'v': last_v.clone(), 'is_mem': last_mem.clone()}
        n = min(self.cache_size, cap)
        ring_start = self.cache_iter % n if self.cache_size >= cap else 0
        kdesc, vdesc, lmdesc = self._descs(n, ring_start, min(top_k, n))
        scores = landmark_scores(q, self.cache_lm_k, lmdesc, cos, sin, L.ROTARY_INTERLEAVED, scale, softmax=True)
        sel = topk_sorted(scores, kdesc.top_k, self.config.cache_selection_method, ring_start)
        if sel.shape != (B, nh, T, kdesc.top_k):
            sel = sel.expand(B, nh, T, kdesc.top_k).contiguous()
        mem_k, mem_v = gather_kv(self.cache_mem_k, self.cache_mem_v, kdesc, vdesc, sel, cos, sin,
                                 L.ROTARY_INTERLEAVED, dim=hs)
        att_k = (q.unsqueeze(3) @ mem_k.transpose(-2, -1)).squeeze(3) * scale
        is_mem = torch.zeros((B, kdesc.top_k, blk), dtype=torch.bool, device=q.device)
        is_mem[:, :, blk - 1] = True
        att_prefix = torch.cat((att_k, att_incomplete), dim=-1)
        v_prefix = torch.cat((mem_v, last_v), dim=-2)
        is_mem_prefix = torch.cat((is_mem.view(B, -1), last_mem), dim=-1)
        return att_prefix, {'v': v_prefix, 'is_mem': is_mem_prefix}

    def store_in_cache(self, keys, values_dict):
        """mem_cache.py:111-158: append whole blocks to the ring buffer, keep the unfinished tail aside."""
        B = keys.shape[0]
        blk, cap = self.block, self.capacity
        inc0 = self.last_incomplete_len
        k = torch.cat((self.last_incomplete_k[:B, :, :inc0], keys), dim=-2)
        v = torch.cat((self.last_incomplete_v[:B, :, :inc0], values_dict['v']), dim=-2)
        is_mem = torch.cat((self.last_incomplete_ismem[:B, :inc0], values_dict['is_mem']), dim=-1)
        _, nh, T, hs = k.shape
        inc = T % blk
        full = T - inc
        self.last_incomplete_k[:B, :, :inc].copy_(k[:, :, full:])
        self.last_incomplete_v[:B, :, :inc].copy_(v[:, :, full:])
        self.last_incomplete_ismem[:B, :inc].copy_(is_mem[:, full:])
        self.last_incomplete_len = inc
        im = is_mem[:, :full].view(B, -1, blk)
        assert im[..., -1].all()
        assert not im[..., :-1].any()
        added = im.shape[1]
        dropped = max(0, added - cap)           # more blocks than the ring holds: only the newest `cap` are kept
        self.cache_iter = (self.cache_iter + dropped) % cap
        self.cache_size += dropped
        added -= dropped
        if added > 0:
            # one kernel writes the blocks into their ring slots (wrapping) and their landmark keys into the dense array
            ks, vs = k[:, :, dropped * blk:full], v[:, :, dropped * blk:full]
            if ks.stride(3) != 1 or ks.stride() != vs.stride():
                ks, vs = ks.contiguous(), vs.contiguous()
            kdesc, vdesc, _ = self._descs(cap, 0, 0)
            rc = L.lib().lmk_cache_store(L.ptr(ks), L.ptr(vs), L.I64x3(ks.stride(0), ks.stride(1), ks.stride(2)),
                                         L.ptr(self.cache_mem_k), L.ptr(self.cache_mem_v), ctypes.byref(kdesc),
                                         ctypes.byref(vdesc), L.ptr(self.cache_lm_k),
                                         L.I64x3(*self.cache_lm_k.stride()[:3]), B, nh, added, self.cache_iter, cap, hs,
                                         L.dtype_code(ks), L.stream_ptr(ks.device))
            L.check(rc, "lmk_cache_store")
        self.cache_iter = (self.cache_iter + added) % cap if self.cache_iter + added >= cap else self.cache_iter + added
        self.cache_size += added


class MemLMCache(nn.Module):
    """Token-id bookkeeping of the cache (mem_cache.py:166-223): inserts `landmark_id` after every
    `mem_cache_freq` tokens across chunk boundaries and strips those positions from the outputs."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.last_incomplete_len = 0
        self.total_len = 0

    def forward(self, x):
        freq = self.config.mem_cache_freq
        prev = self.last_incomplete_len
        B, T = x.shape
        n_total = prev + T
        n_full = n_total // freq
        out_len = T + ((prev + T) // freq)
        out = x.new_empty((B, out_len))
        # position of source token t in the output: t + number of landmarks inserted before it
        src = torch.arange(T, device=x.device)
        dst = src + (src + prev) // freq
        out[:, dst] = x
        lm_pos = (torch.arange(1, n_full + 1, device=x.device) * freq - prev - 1)
        lm_pos = lm_pos + (lm_pos + prev) // freq + 1
        out[:, lm_pos] = self.config.landmark_id
        self.last_incomplete_len = n_total % freq
        prev_total = self.total_len
        self.total_len += out_len
        blk = freq + 1
        start_index = min(prev_total // blk, self.config.cache_topk + 1) * blk + prev
        return out, start_index, None

    def get_final_logits(self, x):
        freq = self.config.mem_cache_freq
        B, T, C = x.shape
        # carry before this chunk = (real tokens before it) mod freq, recovered from the running totals
        blk = freq + 1
        start = self.total_len - T
        pos = torch.arange(start, start + T, device=x.device)
        keep = (pos % blk) != blk - 1
        return x[:, keep]

    def clear_state(self):
        self.last_incomplete_len = 0
        self.total_len = 0
