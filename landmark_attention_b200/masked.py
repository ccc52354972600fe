"""Fused landmark attention with landmarks at arbitrary positions (one flag per batch row and key).

This is the attention of lm_benchmark's `CausalSelfAttention.forward` without cache -- scores, causal fill, mask block,
grouped softmax, att @ v (lm_benchmark/models/landmark.py:196-236, :210-224, :37-119) -- as one differentiable operator
on the tensor cores.  No [B,H,T,T] tensor exists at any point; the group ids are derived inside the kernels from
`is_mem [B, T]`.

The operator is registered with `torch.library` (`lmk::masked_attention`, with a fake implementation and an autograd
formula), so a model that calls it can be wrapped in `torch.compile(fullgraph=True)` as the reference's trainer does
(lm_benchmark/optim/base.py:57-61) without a graph break.
"""
import math
from typing import Tuple

import torch

from . import _lib as L

DEFAULT_MAX_GROUPS = 64


def _u8(is_mem: torch.Tensor) -> torch.Tensor:
    m = is_mem if is_mem.dtype == torch.uint8 else is_mem.to(torch.uint8)
    return m if m.stride(-1) == 1 else m.contiguous()


@torch.library.custom_op("lmk::masked_attention_fwd", mutates_args=())
def _fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_mem: torch.Tensor, sm_scale: float,
         max_groups: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    L.require_cuda(q, k, v, is_mem)
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    assert k.shape == (B, H, Lk, D) and v.shape == (B, H, Lk, D)
    assert q.dtype == k.dtype == v.dtype, 'All tensors must have the same type'
    assert is_mem.shape == (B, Lk), "is_mem must hold one flag per (batch row, key)"
    q, k, v = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v)]
    m8 = _u8(is_mem)
    o = torch.empty((B, H, Lq, D), device=q.device, dtype=q.dtype)
    R = torch.empty((B * H, Lq), device=q.device, dtype=torch.float32)
    A = torch.empty((B * H, max_groups, Lq), device=q.device, dtype=torch.float32)
    rc = L.lib().lmk_attn_mask_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(m8), m8.stride(0), L.ptr(o), L.ptr(R), L.ptr(A),
                                   B, H, Lq, Lk, D, L.strides3(q), L.strides3(k), L.strides3(v), max_groups,
                                   float(sm_scale), L.dtype_code(q), L.stream_ptr(q.device))
    L.check(rc, "lmk_attn_mask_fwd")
    return o, R, A


@_fwd.register_fake
def _(q, k, v, is_mem, sm_scale, max_groups):
    B, H, Lq, D = q.shape
    return (q.new_empty((B, H, Lq, D)), q.new_empty((B * H, Lq), dtype=torch.float32),
            q.new_empty((B * H, max_groups, Lq), dtype=torch.float32))


@torch.library.custom_op("lmk::masked_attention_bwd", mutates_args=())
def _bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_mem: torch.Tensor, o: torch.Tensor, do: torch.Tensor,
         R: torch.Tensor, A: torch.Tensor, sm_scale: float,
         max_groups: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    q, k, v = [t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v)]
    do = do.contiguous()
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    o = o.contiguous()
    m8 = _u8(is_mem)
    dq = torch.empty((B, H, Lq, D), device=q.device, dtype=q.dtype)
    dk = torch.empty((B, H, Lk, D), device=q.device, dtype=q.dtype)
    dv = torch.empty((B, H, Lk, D), device=q.device, dtype=q.dtype)
    need = L.lib().lmk_attn_mask_bwd_workspace(B, H, Lq, max_groups)
    ws = torch.empty(max(int(need), 256), device=q.device, dtype=torch.uint8)
    rc = L.lib().lmk_attn_mask_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(m8), m8.stride(0), L.ptr(o), L.ptr(do), L.ptr(R),
                                   L.ptr(A), L.ptr(dq), L.ptr(dk), L.ptr(dv), L.ptr(ws), ws.numel(), B, H, Lq, Lk, D,
                                   L.strides3(q), L.strides3(k), L.strides3(v), max_groups, float(sm_scale),
                                   L.dtype_code(q), L.stream_ptr(q.device))
    L.check(rc, "lmk_attn_mask_bwd")
    return dq, dk, dv


@_bwd.register_fake
def _(q, k, v, is_mem, o, do, R, A, sm_scale, max_groups):
    return (q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape))


def _setup_context(ctx, inputs, output):
    q, k, v, is_mem, sm_scale, max_groups = inputs
    o, R, A = output
    ctx.save_for_backward(q, k, v, is_mem, o, R, A)
    ctx.sm_scale, ctx.max_groups = sm_scale, max_groups


def _backward(ctx, do, _dR, _dA):
    q, k, v, is_mem, o, R, A = ctx.saved_tensors
    dq, dk, dv = _bwd(q, k, v, is_mem, o, do, R, A, ctx.sm_scale, ctx.max_groups)
    return dq, dk, dv, None, None, None


_fwd.register_autograd(_backward, setup_context=_setup_context)


# the kernels' shape contract (include/b200lmk.h, lmk_attn_mask_fwd); kept in Python so that the check is traceable
_HEAD_DIM, _Q_TILE, _K_TILE, _MAX_KEYS, _MAX_GROUPS = 128, 128, 64, 32768, 64


def masked_attention_supported(q, k, max_groups=DEFAULT_MAX_GROUPS) -> bool:
    """True when the tensor-core kernels take this problem (bf16/fp16, D = 128, whole 128-row query tiles, 64-key
    tiles, max_groups within the build's limit).  Pure shape logic: no library call, so torch.compile can trace it."""
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    Lq, D, Lk = q.shape[2], q.shape[3], k.shape[2]
    return (D == _HEAD_DIM and Lq >= _Q_TILE and Lq % _Q_TILE == 0 and Lk % _K_TILE == 0 and Lk >= Lq
            and (Lk - Lq) % _K_TILE == 0 and Lk <= _MAX_KEYS and 0 < max_groups <= _MAX_GROUPS)


def landmark_attention_masked(q, k, v, is_mem, sm_scale=None, max_groups=DEFAULT_MAX_GROUPS):
    """Landmark attention of q [B,H,Lq,D] over k, v [B,H,Lk,D] with landmark flags is_mem [B, Lk] (bool or uint8).

    `max_groups` bounds the number of landmarks before any query (lm_benchmark's max_groups_for_softmax - 1); it sizes
    the statistics kept for the backward pass.  Raises NotImplementedError for shapes outside the kernels' contract."""
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.size(-1))
    o, _, _ = _fwd(q, k, v, is_mem, float(sm_scale), int(max_groups))
    return o
