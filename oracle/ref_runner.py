"""Drive the reference's own code staged under oracle/_ref/ (see make_ref.py).  TEST INFRASTRUCTURE ONLY.

Used by the benchmark's reference arm / CPU baseline and by the reference-on-GPU timing script; never by the package.
`available()` is False where oracle/_ref/ has not been staged; callers then fall back to the restatement in
landmark_oracle.py and say so.
"""
import importlib
import math
import os
import sys
import types

import torch

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "llama", "llama_mem.py"))


def llama_mem():
    """The reference's llama/llama_mem.py module (imports transformers and triton, both only at module level)."""
    p = os.path.join(REF_DIR, "llama")
    if p not in sys.path:
        sys.path.insert(0, p)
    return importlib.import_module("llama_mem")


def triton_kernels():
    """The reference's llama/ltriton/flash_landmark_attention.py module (needs a CUDA device to run)."""
    p = os.path.join(REF_DIR, "llama")
    if p not in sys.path:
        sys.path.insert(0, p)
    return importlib.import_module("ltriton.flash_landmark_attention")


def lm_landmark():
    """The reference's lm_benchmark/models/landmark.py.  It imports tiktoken only to build a tokenizer for text
    generation (landmark.py:298), which needs a download; a stub module stands in when tiktoken is missing, and
    get_encoding is replaced either way."""
    p = os.path.join(REF_DIR, "lm_benchmark")
    if p not in sys.path:
        sys.path.insert(0, p)
    try:
        import tiktoken
    except ImportError:
        tiktoken = types.ModuleType("tiktoken")
        sys.modules["tiktoken"] = tiktoken
    tiktoken.get_encoding = lambda name: None
    return importlib.import_module("models.landmark")


def highlevel_attention(q, k, v, block):
    """The high-level path exactly as the reference's own test drives it
    (llama/ltriton/test_flash_landmark_attention.py:105-125, which cannot be imported because it runs CUDA code at
    import): masks, llama_mem.landmark_grouped_softmax (llama/llama_mem.py:222-243), P @ V."""
    lm = llama_mem()
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    dev = q.device
    att = q @ k.transpose(-1, -2) / math.sqrt(D)
    att_mask = torch.tril(torch.ones((1, 1, Lq, Lk), device=dev), diagonal=Lk - Lq) == 1.
    kb = torch.arange(0, Lk, device=dev) // block
    last = (kb[None, :] == kb[Lk - Lq:, None]).unsqueeze(0).unsqueeze(1)
    is_mem = (torch.arange(0, Lk, device=dev) % block == block - 1).view(1, 1, 1, Lk)
    mask = att_mask & ~(last & is_mem)
    last = last & mask
    is_mem = (is_mem & mask).expand(B, H, Lq, Lk)
    att = att.masked_fill(~mask, float("-inf"))
    att = lm.landmark_grouped_softmax(att, -1, is_mem, last).to(q.dtype)
    att = att.masked_fill(~mask, 0.0)
    return att @ v


def highlevel_fwd_bwd(q, k, v, do, block):
    q, k, v = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out = highlevel_attention(q, k, v, block)
    dq, dk, dv = torch.autograd.grad(out, [q, k, v], do)
    return out.detach(), dq, dk, dv
