"""Fused landmark attention: same Python API as the reference's `fused_landmark_attention`
(llama/ltriton/flash_landmark_attention.py:391-403) and an SDPA-style alias.
"""
import math
from typing import Optional

import torch

from . import _lib as L


class FusedLandmarkAttention(torch.autograd.Function):
    """Mirrors FusedLandmarkAttention (flash_landmark_attention.py:308-389): forward keeps q, k, v, o and the
    softmax statistics L, M; backward recomputes the probabilities."""

    @staticmethod
    def forward(ctx, q, k, v, n_prefix_q, sm_scale, block_size, path=L.PATH_AUTO):
        L.require_cuda(q, k, v)
        batch, nheads, seqlen_q, d = q.shape
        seqlen_k = k.shape[2]
        assert k.shape == (batch, nheads, seqlen_k, d)
        assert v.shape == (batch, nheads, seqlen_k, d)
        assert d <= 128, 'FlashAttention only support head dimensions up to 128'
        assert q.dtype == k.dtype == v.dtype, 'All tensors must have the same type'
        assert seqlen_k - seqlen_q == n_prefix_q * block_size
        q, k, v = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v)]
        o = torch.empty((batch, nheads, seqlen_q, d), device=q.device, dtype=q.dtype)
        lse_l = torch.empty((batch * nheads, seqlen_q), device=q.device, dtype=torch.float32)
        lse_m = torch.empty((batch * nheads, seqlen_q), device=q.device, dtype=torch.float32)
        rc = L.lib().lmk_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse_l), L.ptr(lse_m),
                                  batch, nheads, seqlen_q, seqlen_k, d, L.strides3(q), L.strides3(k), L.strides3(v),
                                  block_size, float(sm_scale), L.dtype_code(q), path, L.stream_ptr(q.device))
        L.check(rc, "lmk_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse_l, lse_m)
        ctx.sm_scale, ctx.block, ctx.path = sm_scale, block_size, path
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse_l, lse_m = ctx.saved_tensors
        block = ctx.block
        assert q.shape[2] % block == 0, "Backward supported only for full blocks"
        assert k.shape[2] % block == 0, "Backward supported only for full blocks"
        batch, nheads, seqlen_q, d = q.shape
        seqlen_k = k.shape[2]
        do = do.contiguous()
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        dq = torch.empty((batch, nheads, seqlen_q, d), device=q.device, dtype=q.dtype)
        dk = torch.empty((batch, nheads, seqlen_k, d), device=q.device, dtype=q.dtype)
        dv = torch.empty((batch, nheads, seqlen_k, d), device=q.device, dtype=q.dtype)
        code = L.dtype_code(q)
        need = L.lib().lmk_attn_bwd_workspace(batch, nheads, seqlen_q, seqlen_k, d, block, code, ctx.path)
        ws = torch.empty(max(int(need), 256), device=q.device, dtype=torch.uint8)
        rc = L.lib().lmk_attn_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(do), L.ptr(lse_l), L.ptr(lse_m),
                                  L.ptr(dq), L.ptr(dk), L.ptr(dv), L.ptr(ws), ws.numel(),
                                  batch, nheads, seqlen_q, seqlen_k, d, L.strides3(q), L.strides3(k), L.strides3(v),
                                  block, float(ctx.sm_scale), code, ctx.path, L.stream_ptr(q.device))
        L.check(rc, "lmk_attn_bwd")
        return dq, dk, dv, None, None, None, None


def fused_landmark_attention(q, k, v, is_mem=None, sm_scale=None, block_size=64, path=L.PATH_AUTO):
    """Landmark attention over q [B,H,Lq,D], k/v [B,H,Lk,D]; the landmark is the last token of every block.

    Same call as the reference's `fused_landmark_attention(q, k, v, is_mem, sm_scale=None, block_size=64)`.
    `is_mem` may be None (fast path: no mask is read and the host is not synchronised); when given it must be the
    regular pattern over the keys, as the reference asserts (flash_landmark_attention.py:393-394).
    """
    if is_mem is not None:
        expected_is_mem = torch.arange(0, is_mem.shape[-1], device=is_mem.device) % block_size == (block_size - 1)
        assert (is_mem == expected_is_mem).all()
    n_history_kv = k.shape[-2] - q.shape[-2]
    assert n_history_kv % block_size == 0
    n_history_blocks = n_history_kv // block_size
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.size(-1))
    D = q.shape[-1]
    if (path == L.PATH_AUTO and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and D <= 128 and D % 8 == 0
            and q.shape[2] % 128 != 0 and n_history_kv % 64 == 0):
        # lengths that are not whole 128-row tiles: rows of zeros appended to q, k and v come after every real query,
        # so causality hides the extra keys and the extra query rows are dropped again
        extra = -q.shape[2] % 128
        if _tensor_core_route(q.shape[0], q.shape[1], q.shape[2] + extra, k.shape[2] + extra, block_size, q.dtype):
            qp, kp, vp = [torch.nn.functional.pad(t, (0, 0, 0, extra)) for t in (q, k, v)]
            return fused_landmark_attention(qp, kp, vp, None, sm_scale, block_size, path)[:, :, :q.shape[2]]
    if (path == L.PATH_AUTO and D < 128 and D % 8 == 0 and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16)
            and _tensor_core_route(q.shape[0], q.shape[1], q.shape[2], k.shape[2], block_size, q.dtype)):
        # head dims below 128: zero columns change neither q k^T nor the real columns of p v, and the tensor-core
        # kernels at twice the work beat the general kernels by an order of magnitude
        pad = (0, 128 - D)
        qp, kp, vp = [torch.nn.functional.pad(t, pad) for t in (q, k, v)]
        return fused_landmark_attention(qp, kp, vp, None, sm_scale, block_size, path)[..., :D]
    if path == L.PATH_AUTO and block_size != 64:
        # the tensor-core kernels of lmk_attn_fwd are built for blocks of 64; other block sizes run on the
        # arbitrary-landmark tensor-core kernels with the regular pattern as flags, where those take the shape
        from .masked import landmark_attention_masked, masked_attention_supported
        Lk = k.shape[2]
        groups = max(Lk // block_size, 1)          # landmarks in front of any query
        if groups <= 64 and sm_scale > 0 and masked_attention_supported(q, k, groups):
            return landmark_attention_masked(q, k, v, _regular_flags(q.shape[0], Lk, block_size, q.device), sm_scale,
                                             groups)
    return FusedLandmarkAttention.apply(q, k, v, n_history_blocks, sm_scale, block_size, path)


def _tensor_core_route(B, H, Lq, Lk, block_size, dtype):
    """Whether a head-dim-128 problem of this shape runs on one of the two tensor-core kernel families."""
    if block_size == 64:
        return bool(L.lib().lmk_attn_tcgen05_supported(B, H, Lq, Lk, 128, 64, L._DTYPES[dtype]))
    return (Lk // max(block_size, 1) <= 64 and Lq >= 128 and Lq % 128 == 0 and Lk % 64 == 0 and Lk >= Lq
            and (Lk - Lq) % 64 == 0 and Lk <= 32768)


_FLAGS = {}


def _regular_flags(batch, n_keys, block_size, device):
    """uint8 [batch, n_keys] with a landmark at the end of every block (one row, broadcast over the batch)."""
    key = (device, n_keys, block_size)
    row = _FLAGS.get(key)
    if row is None:
        if len(_FLAGS) > 64:
            _FLAGS.clear()
        row = (torch.arange(n_keys, device=device) % block_size == block_size - 1).to(torch.uint8).view(1, n_keys)
        _FLAGS[key] = row
    return row.expand(batch, n_keys)


def landmark_sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=True, scale=None, *,
                  is_mem: Optional[torch.Tensor] = None, block_size: int = 64):
    """`torch.nn.functional.scaled_dot_product_attention` signature on top of fused landmark attention.
    Landmark attention is causal by construction; masks and dropout are not part of the operator."""
    if attn_mask is not None:
        raise ValueError("landmark_sdpa does not take attn_mask (the landmark pattern defines the mask)")
    if dropout_p != 0.0:
        raise ValueError("landmark_sdpa does not support dropout")
    if not is_causal:
        raise ValueError("landmark attention is causal; pass is_causal=True")
    return fused_landmark_attention(query, key, value, is_mem, sm_scale=scale, block_size=block_size)


def attn_forward_with_stats(q, k, v, block_size=64, sm_scale=None, path=L.PATH_AUTO):
    """Forward only; also returns the stored statistics (L, M) [B*H, Lq] for inspection and tests."""
    L.require_cuda(q, k, v)
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v)]
    o = torch.empty((B, H, Lq, D), device=q.device, dtype=q.dtype)
    l = torch.empty((B * H, Lq), device=q.device, dtype=torch.float32)
    m = torch.empty((B * H, Lq), device=q.device, dtype=torch.float32)
    rc = L.lib().lmk_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(l), L.ptr(m), B, H, Lq, Lk, D,
                              L.strides3(q), L.strides3(k), L.strides3(v), block_size, float(sm_scale),
                              L.dtype_code(q), path, L.stream_ptr(q.device))
    L.check(rc, "lmk_attn_fwd")
    return o, l, m
