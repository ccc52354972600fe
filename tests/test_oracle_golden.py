"""Pin the CPU oracle against results recorded from the reference's own code (tests/golden)."""
import math

import pytest
import torch

from oracle import landmark_oracle as O


@pytest.mark.parametrize("name", ["fused_square", "fused_prefix", "fused_blk32", "fused_blk16_d128"])
def test_fused_against_highlevel_reference(golden, name):
    g = golden(name + ".pt")
    out, dq, dk, dv = O.landmark_attention_grads(g["q"], g["k"], g["v"], g["do"], g["blk"])
    for a, b in ((out, g["out"]), (dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert (a - b).abs().max().item() < 2e-5


@pytest.mark.parametrize("name", ["triton_square", "triton_prefix"])
def test_fused_against_reference_triton_kernels(golden, name):
    g = golden(name + ".pt")
    out, m, l = O.landmark_attention(g["q"], g["k"], g["v"], g["blk"], return_stats=True)
    B, H, Lq, D = g["q"].shape
    assert (out - g["out"]).abs().max().item() < 1e-5
    assert (m.reshape(B * H, Lq) - g["M"]).abs().max().item() < 1e-5
    assert ((l.reshape(B * H, Lq) - g["L"]).abs() / g["L"]).max().item() < 1e-5
    _, dq, dk, dv = O.landmark_attention_grads(g["q"], g["k"], g["v"], g["do"], g["blk"])
    for a, b in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert (a - b).abs().max().item() < 2e-5


def test_grouped_softmax_llama(golden):
    g = golden("gsm_llama.pt")
    x = g["x"].detach().clone().requires_grad_(True)
    p = O.grouped_softmax(x, g["is_mem"], g["last"])
    assert (p - g["probs"]).abs().max().item() < 1e-6
    (gx,) = torch.autograd.grad(p, [x], g["gprobs"])
    assert (gx - g["gx"]).abs().max().item() < 1e-5


def test_grouped_softmax_lm(golden):
    g = golden("gsm_lm.pt")
    x = g["x"].detach().clone().requires_grad_(True)
    p, gp = O.grouped_softmax(x, g["is_mem"], g["last"], attn_mask=g["mask"], guards=True,
                              return_group_prob=True, max_mem_cnt=g["max_mem_cnt"])
    assert (p - g["probs"]).abs().max().item() < 1e-6
    assert (gp - g["group_prob"]).abs().max().item() < 1e-6
    (gx,) = torch.autograd.grad(p, [x], g["gprobs"])
    assert (gx - g["gx"]).abs().max().item() < 1e-5


def test_mask_preparation(golden):
    g = golden("gsm_lm.pt")
    T = g["x"].shape[-1]
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    mask, is_mem, last = O.prepare_landmark_masks(g["is_mem_row"], hidden)
    H = g["x"].shape[1]
    assert torch.equal(mask.expand(-1, H, -1, -1), g["mask"])
    assert torch.equal(is_mem.expand(-1, H, -1, -1), g["is_mem"])
    assert torch.equal(last.expand(-1, H, -1, -1), g["last"])
    g2 = golden("gsm_llama.pt")
    _, is_mem2, last2 = O.prepare_landmark_masks(g2["is_mem_row"], hidden)
    assert torch.equal(is_mem2, g2["is_mem"]) and torch.equal(last2, g2["last"])


def test_lm_attention_call_site(golden):
    g = golden("lm_attn.pt")
    q = g["q_rot"].detach().clone().requires_grad_(True)
    k = g["k_rot"].detach().clone().requires_grad_(True)
    v = g["v"].detach().clone().requires_grad_(True)
    B, H, T, D = q.shape
    y = O.lm_attention(q, k, v, g["is_mem_row"]).transpose(1, 2).reshape(B, T, H * D)
    assert (y - g["y"]).abs().max().item() < 1e-5
    dq, dk, dv = torch.autograd.grad(y, [q, k, v], g["gy"])
    for a, b in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert (a - b).abs().max().item() < 2e-5


@pytest.mark.parametrize("method", ["per_token_and_head", "max_over_heads", "max_over_tokens"])
def test_block_cache(golden, method):
    g = golden(f"memcache_{method}.pt")
    cache = O.BlockCacheOracle(g["capacity"], g["blk"], g["top_k"], method)
    for r in g["records"]:
        att, vp, im, _ = cache.retrieve(r["q"], r["start_index"])
        assert att.shape == r["att_prefix"].shape
        assert (att - r["att_prefix"]).abs().max().item() < 1e-5 if att.numel() else True
        assert torch.equal(im, r["is_mem_prefix"])
        assert (vp - r["v_prefix"]).abs().max().item() == 0 if vp.numel() else True
        assert cache.cache_iter == r["cache_iter"]
        cache.store(r["k"], r["v"], r["is_mem"])


def test_lm_call_site_with_cache(golden):
    # CausalSelfAttention.forward with a block cache attached: the oracle's cache supplies the prefix, the oracle's
    # attention joins prefix and chunk in one grouped softmax; four chunks against the reference's outputs
    g = golden("lm_attn_cache.pt")
    cache = O.BlockCacheOracle(g["capacity"], g["blk"], g["top_k"], g["method"])
    saw_blocks = False
    for r in g["records"]:
        B, H, T, D = r["q_rot"].shape
        att, vp, im, _ = cache.retrieve(r["q_rot"], r["start_index"])
        saw_blocks = saw_blocks or att.shape[-1] >= g["blk"]
        y = O.lm_attention(r["q_rot"], r["k_rot"], r["v"], r["is_mem"], att_prefix=att, v_prefix=vp, is_mem_prefix=im)
        y = y.transpose(1, 2).reshape(B, T, H * D)
        assert (y - r["y"]).abs().max().item() < 1e-5
        cache.store(r["k"], r["v"], r["is_mem"])
    assert saw_blocks


def test_landmark_id_bookkeeping(golden):
    g = golden("memcache_ids.pt")
    carry, total = 0, 0
    blk = g["mem_freq"] + 1
    for r in g["records"]:
        start_index = min(total // blk, g["top_k"] + 1) * blk + carry
        ids, new_carry = O.insert_landmarks(r["ids"], g["mem_freq"], g["landmark_id"], carry)
        assert torch.equal(ids, r["out_ids"])
        assert start_index == r["start_index"]
        assert torch.equal(O.strip_landmarks(r["feats"], g["mem_freq"], carry), r["stripped"])
        total += ids.shape[1]
        carry = new_carry


@pytest.mark.parametrize("name", ["llama_retr_blocks", "llama_retr_tail"])
def test_llama_retrieval_branch(golden, name):
    g = golden(name + ".pt")
    out = O.llama_retrieval_attention(g["q"], g["k"], g["v"], g["past_k"], g["past_v"], g["blk"], g["top_k"],
                                      chunk_is_mem=g["is_mem_row"])
    assert (out - g["out"]).abs().max().item() < 1e-5
