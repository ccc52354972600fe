"""Parity of the stand-alone grouped softmax kernels (both reference flavours) against the oracle and golden data."""
import pytest
import torch

import landmark_attention_b200 as P
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_llama_flavour_against_golden(golden):
    g = golden("gsm_llama.pt")
    x = g["x"].to(DEV).detach().requires_grad_(True)
    p = P.landmark_grouped_softmax(x, -1, g["is_mem"].to(DEV), g["last"].to(DEV))
    assert (p.detach().cpu() - g["probs"]).abs().max().item() < 1e-6
    (gx,) = torch.autograd.grad(p, [x], g["gprobs"].to(DEV))
    assert (gx.cpu() - g["gx"]).abs().max().item() < 1e-5


def test_lm_flavour_against_golden(golden):
    g = golden("gsm_lm.pt")
    x = g["x"].to(DEV).detach().requires_grad_(True)
    p, gp = P.landmark_grouped_softmax_lm(x, -1, g["is_mem"].to(DEV), g["mask"].to(DEV), g["last"].to(DEV), True,
                                          g["max_mem_cnt"])
    assert (p.detach().cpu() - g["probs"]).abs().max().item() < 1e-6
    assert (gp.cpu() - g["group_prob"]).abs().max().item() < 1e-6
    (gx,) = torch.autograd.grad(p, [x], g["gprobs"].to(DEV))
    assert (gx.cpu() - g["gx"]).abs().max().item() < 1e-5


def test_lm_call_site_against_golden(golden):
    g = golden("lm_attn.pt")
    q, k, v = [g[n].to(DEV).detach().requires_grad_(True) for n in ("q_rot", "k_rot", "v")]
    B, H, T, D = q.shape
    y = P.lm_landmark_attention(q, k, v, g["is_mem_row"].to(DEV)).transpose(1, 2).reshape(B, T, H * D)
    assert (y.detach().cpu() - g["y"]).abs().max().item() < 1e-5
    dq, dk, dv = torch.autograd.grad(y, [q, k, v], g["gy"].to(DEV))
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert (got.cpu() - g[key]).abs().max().item() < 2e-5


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-6)])
def test_regular_pattern_equals_fused_probabilities(dtype, tol):
    # on the regular landmark pattern the grouped softmax of masked scores is the fused kernel's probability matrix
    torch.manual_seed(0)
    B, H, L, D, blk = 1, 2, 320, 32, 64
    q, k = torch.randn(B, H, L, D), torch.randn(B, H, L, D)
    s = ((q @ k.transpose(-1, -2)) / D ** 0.5).to(dtype)
    hidden = torch.ones(L, L, dtype=torch.bool).triu(1)
    mask, is_mem, last = O.prepare_landmark_masks(O.regular_is_mem(L, blk).view(1, L), hidden)
    x = s.masked_fill(mask, float("-inf"))
    exp = O.grouped_softmax(x.float(), is_mem, last, attn_mask=mask, guards=True)
    got, _ = P.landmark_grouped_softmax_lm(x.to(DEV), -1, is_mem.to(DEV), mask.to(DEV), last.to(DEV), False, L // blk + 3)
    assert (got.cpu() - exp).abs().max().item() < tol
    assert (got.sum(-1).cpu() - 1).abs().max().item() < 1e-5


def test_long_rows_and_many_groups():
    torch.manual_seed(1)
    B, H, Lq, Lk = 1, 1, 8, 4096
    is_mem_row = torch.zeros(1, Lk, dtype=torch.bool)
    is_mem_row[0, 31::32] = True
    x = torch.randn(B, H, Lq, Lk)
    hidden = torch.zeros(Lq, Lk, dtype=torch.bool)
    hidden[:, Lk - 5:] = True
    mask, is_mem, last = O.prepare_landmark_masks(is_mem_row, hidden)
    xm = x.masked_fill(mask, float("-inf"))
    exp = O.grouped_softmax(xm, is_mem, last, attn_mask=mask, guards=True)
    got, _ = P.landmark_grouped_softmax_lm(xm.to(DEV), -1, is_mem.to(DEV), mask.to(DEV), last.to(DEV), False, 130)
    assert (got.cpu() - exp).abs().max().item() < 1e-6


@pytest.mark.parametrize("Lk,density,dtype", [(333, 0.3, torch.float32), (1000, 0.05, torch.float32),
                                               (2048, 0.02, torch.bfloat16), (777, 0.5, torch.float16),
                                               (4096, 0.01, torch.float32), (5000, 0.01, torch.float32)])
@pytest.mark.parametrize("guards", [True, False])
def test_random_masks_any_length(Lk, density, dtype, guards):
    # arbitrary landmark positions (several per eight keys at the higher densities), row lengths that are not a
    # multiple of the vector width, rows that start at unaligned addresses, both flavours, forward and backward
    g = torch.Generator().manual_seed(Lk)
    B, H, Lq = 2, 2, 5
    is_mem = torch.rand(B, 1, Lq, Lk, generator=g) < density
    last = (torch.rand(B, 1, Lq, Lk, generator=g) < 0.1) & ~is_mem
    last[..., 0] = True
    is_mem[..., 0] = False
    hidden = (torch.rand(1, 1, Lq, Lk, generator=g) < 0.2) & ~last & ~is_mem if guards else None
    x = (torch.randn(B, H, Lq, Lk, generator=g) * 3).to(dtype)
    if guards:
        x = x.masked_fill(hidden, float("-inf"))
    gp = torch.randn(B, H, Lq, Lk, generator=g)
    n_lm = int(is_mem.sum(-1).max()) + 2
    xo = x.float().detach().requires_grad_(True)
    exp = O.grouped_softmax(xo, is_mem, last, attn_mask=hidden, guards=guards)
    (gx_exp,) = torch.autograd.grad(exp, [xo], gp)
    xd = x.to(DEV).detach().requires_grad_(True)
    if guards:
        got, _ = P.landmark_grouped_softmax_lm(xd, -1, is_mem.to(DEV), hidden.to(DEV), last.to(DEV), False, n_lm)
    else:
        got = P.landmark_grouped_softmax(xd, -1, is_mem.to(DEV), last.to(DEV), max_groups=n_lm)
    assert (got.detach().cpu() - exp.detach()).abs().max().item() < 2e-6
    (gx,) = torch.autograd.grad(got, [xd], gp.to(DEV))
    tol = 2e-5 if dtype == torch.float32 else 2e-2          # the gradient is rounded to the 16-bit input type
    assert (gx.float().cpu() - gx_exp).abs().max().item() < tol
    again = P.landmark_grouped_softmax_lm(xd, -1, is_mem.to(DEV), hidden.to(DEV), last.to(DEV), False, n_lm)[0] \
        if guards else P.landmark_grouped_softmax(xd, -1, is_mem.to(DEV), last.to(DEV), max_groups=n_lm)
    assert torch.equal(again, got)                           # sums are taken in a fixed order


def test_lm_call_site_with_cache_against_golden(golden):
    # CausalSelfAttention.forward with a block cache attached (landmark.py:182-253): four chunks; the cache kernels
    # supply the prefix scores / values, lm_landmark_attention joins prefix and chunk in one grouped softmax
    g = golden("lm_attn_cache.pt")
    r0 = g["records"][0]
    B, H, _, D = r0["q_rot"].shape
    cfg = type("C", (), dict(batch_size=B, mem_cache_size=g["capacity"], mem_cache_freq=g["blk"] - 1, n_head=H,
                             n_embd=H * D, cache_topk=g["top_k"], cache_selection_method=g["method"]))()
    store = P.MemLMCacheStorage(cfg, None, dtype=torch.float32, device=DEV)
    widest = 0
    for r in g["records"]:
        q, k_rot, k, v, im = [r[n].to(DEV) for n in ("q_rot", "k_rot", "k", "v", "is_mem")]
        T = q.shape[2]
        att_prefix, cv = store.retrieve_for_query(q, None, None, r["start_index"])
        widest = max(widest, att_prefix.shape[-1])
        y = P.lm_landmark_attention(q, k_rot, v, im, att_prefix=att_prefix, cache_values=cv)
        y = y.transpose(1, 2).reshape(B, T, H * D)
        assert (y.cpu() - r["y"]).abs().max().item() < 2e-5
        store.store_in_cache(k, {"v": v, "is_mem": im})
    assert widest >= g["top_k"] * g["blk"]


def test_group_dropout_scales_whole_groups():
    # landmark.py:110-114: each landmark's group weight is dropped or scaled by 1/(1-p); last-section keys untouched.
    # Same draw as the implementation (one torch.rand from the default generator), applied to the oracle's result.
    B, H, T, blk, p, mmc = 2, 2, 96, 8, 0.4, 16
    g = torch.Generator().manual_seed(9)
    x = torch.randn(B, H, T, T, generator=g)
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    mask, is_mem, last = O.prepare_landmark_masks(O.regular_is_mem(T, blk).view(1, T).expand(B, T), hidden)
    x = x.masked_fill(mask, float("-inf"))
    base = O.grouped_softmax(x, is_mem, last, attn_mask=mask, guards=True)
    xd = x.to(DEV).requires_grad_(True)
    torch.manual_seed(77)
    got, gp = P.landmark_grouped_softmax_lm(xd, -1, is_mem.to(DEV), mask.to(DEV), last.to(DEV), True, mmc, p_group_dropout=p)
    torch.manual_seed(77)
    keep = (torch.rand((B, H, T, mmc - 1), device=DEV) >= p).float().cpu() / (1 - p)
    group = torch.cumsum(is_mem.expand(B, H, T, T).long(), -1).clamp(max=mmc - 2)
    exp = torch.where(is_mem | last | mask, base, base * torch.gather(keep, -1, group))
    assert (got.detach().cpu() - exp).abs().max().item() < 1e-6
    assert 0.2 < (keep == 0).float().mean().item() < 0.6                       # groups were dropped indeed
    assert (gp[..., -1].cpu() - (base * last).sum(-1) / (1 - p)).abs().max().item() < 1e-5
    (gx,) = torch.autograd.grad(got.sum(), [xd])                                 # differentiable through the factors
    assert torch.isfinite(gx).all()


@pytest.mark.parametrize("B,H,Lq,Lk,dtype", [(2, 2, 512, 512, torch.float32), (2, 3, 200, 333, torch.float32),
                                             (1, 2, 257, 1024, torch.bfloat16), (2, 1, 64, 64, torch.float16),
                                             (1, 1, 300, 4096, torch.float32), (1, 1, 40, 4500, torch.float32)])
def test_causal_form_needs_no_masks(B, H, Lq, Lk, dtype):
    # landmark_grouped_softmax_causal(raw scores, row flags) against the oracle's mask block + masked_fill + grouped
    # softmax (landmark.py:210-232); landmarks at random positions incl. the query's own key, a visible prefix of
    # Lk - Lq keys, garbage (not -inf) at the hidden positions, forward and backward
    g = torch.Generator().manual_seed(Lq * 7 + Lk)
    flags = torch.rand(B, Lk, generator=g) < 0.06
    x = (torch.randn(B, H, Lq, Lk, generator=g) * 3).to(dtype)
    hidden = torch.ones(Lq, Lk, dtype=torch.bool).triu(Lk - Lq + 1)
    mask, is_mem, last = O.prepare_landmark_masks(flags, hidden)
    xo = x.float().detach().requires_grad_(True)
    exp = O.grouped_softmax(xo.masked_fill(mask, float("-inf")), is_mem, last, attn_mask=mask, guards=True)
    gp = torch.randn(B, H, Lq, Lk, generator=g)
    (gx_exp,) = torch.autograd.grad(exp, [xo], gp)
    xd = x.to(DEV).detach().requires_grad_(True)
    got = P.landmark_grouped_softmax_causal(xd, flags.to(DEV), int(flags.sum(-1).max()) + 2)
    assert (got.detach().cpu() - exp.detach()).abs().max().item() < 2e-6
    (gx,) = torch.autograd.grad(got, [xd], gp.to(DEV))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (gx.float().cpu() - gx_exp).abs().max().item() < tol
    assert not gx.float().cpu()[..., hidden].any()              # nothing flows to hidden scores


def test_too_many_landmarks_for_max_groups_are_reported():
    # max_groups bounds 1 + landmarks per row; a row beyond it must not pass unnoticed: device status word 501
    from landmark_attention_b200 import _lib as L
    g = torch.Generator().manual_seed(4)
    B, H, Lq, Lk = 1, 1, 4, 300
    is_mem = torch.zeros(B, 1, Lq, Lk, dtype=torch.bool)
    is_mem[..., 9::10] = True                                   # 30 landmarks
    last = torch.zeros_like(is_mem)
    last[..., 0] = True
    x = torch.randn(B, H, Lq, Lk, generator=g).to(DEV)
    L.device_status()
    P.landmark_grouped_softmax(x, -1, is_mem.to(DEV), last.to(DEV), max_groups=31)
    assert L.device_status() == 0
    P.landmark_grouped_softmax(x, -1, is_mem.to(DEV), last.to(DEV), max_groups=30)
    assert L.device_status() == 501
    assert L.device_status() == 0                               # reading clears it
    flags = torch.zeros(B, Lk, dtype=torch.bool)
    flags[:, 9::10] = True
    P.landmark_grouped_softmax_causal(x, flags.to(DEV), 30)     # the last query sees 29 landmarks in front of its own key
    assert L.device_status() == 0
    P.landmark_grouped_softmax_causal(x, flags.to(DEV), 29)
    assert L.device_status() == 501
