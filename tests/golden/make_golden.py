"""Generate the golden fixtures in this folder by running the REFERENCE's own Python on CPU.

Usage (only where a checkout of epfml/landmark-attention is available):
    python tests/golden/make_golden.py --reference /path/to/landmark-attention

Each fixture is a small .pt file holding seeded inputs and the outputs the reference computed
for them.  The tests never need the reference checkout: they only read these files.

What is recorded, and from which reference code:
  fused_*.pt       high-level recipe of llama/ltriton/test_flash_landmark_attention.py:105-125
                   driving llama/llama_mem.py:222-243 (out, dq, dk, dv)
  triton_*.pt      the reference Triton kernels (llama/ltriton/flash_landmark_attention.py) run
                   under TRITON_INTERPRET=1: out, L, M, dq, dk, dv
  gsm_llama.pt     llama_mem.landmark_grouped_softmax on irregular landmark positions with the
                   model-level mask preparation of llama_mem.py:807-815
  gsm_lm.pt        lm_benchmark landmark_grouped_softmax (landmark.py:88-119) with the mask block
                   of landmark.py:210-224, probs + group_prob + grad
  lm_attn.pt       lm_benchmark CausalSelfAttention.forward (landmark.py:171-255), no cache
  memcache_*.pt    MemLMCacheStorage.store_in_cache / retrieve_for_query (mem_cache.py:41-158)
  lm_attn_cache.pt lm_benchmark CausalSelfAttention.forward with a MemLMCacheStorage attached (landmark.py:182-253):
                   four chunks, the attention output of each given the blocks retrieved from the earlier ones
                   for the three selection methods; MemLMCache.forward / get_final_logits
  llama_retr_*.pt  LlamaModel.forward -> LlamaAttention.forward cache branch (llama_mem.py:318-430)
"""
import argparse
import math
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, **kw):
    kw = {k: (v.detach().clone().contiguous() if torch.is_tensor(v) else v) for k, v in kw.items()}
    torch.save(kw, os.path.join(HERE, name))
    size = os.path.getsize(os.path.join(HERE, name))
    print(f"wrote {name}: {size / 1024:.1f} KiB")


# --------------------------------------------------------------------------- fused, high level
def highlevel_recipe(llama_mem, q, k, v, blk):
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    att = q @ k.transpose(-1, -2) / math.sqrt(D)
    att_mask = torch.tril(torch.ones((1, 1, Lq, Lk)), diagonal=Lk - Lq) == 1.
    last = (torch.arange(0, Lk) // blk)[None, :] == (torch.arange(Lk - Lq, Lk) // blk)[:, None]
    last = last.unsqueeze(0).unsqueeze(1)
    is_mem = (torch.arange(0, Lk) % blk == blk - 1).view(1, 1, 1, Lk)
    mask = att_mask & ~(last & is_mem)
    last = last & mask
    is_mem = (is_mem & mask).expand(B, H, Lq, Lk)
    att = att.masked_fill(~mask, float("-inf"))
    att = llama_mem.landmark_grouped_softmax(att, -1, is_mem, last).to(q.dtype)
    att = att.masked_fill(~mask, 0.0)
    return att @ v


def gen_fused(llama_mem):
    cases = dict(
        fused_square=dict(B=1, H=2, Lq=256, Lk=256, D=32, blk=64, seed=11),
        fused_prefix=dict(B=1, H=2, Lq=128, Lk=320, D=64, blk=64, seed=12),
        fused_blk32=dict(B=2, H=1, Lq=128, Lk=128, D=32, blk=32, seed=13),
        fused_blk16_d128=dict(B=1, H=1, Lq=64, Lk=96, D=128, blk=16, seed=14),
    )
    for name, c in cases.items():
        g = torch.Generator().manual_seed(c["seed"])
        q = torch.randn(c["B"], c["H"], c["Lq"], c["D"], generator=g)
        k = torch.randn(c["B"], c["H"], c["Lk"], c["D"], generator=g)
        v = torch.randn(c["B"], c["H"], c["Lk"], c["D"], generator=g)
        do = torch.randn(c["B"], c["H"], c["Lq"], c["D"], generator=g)
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
        out = highlevel_recipe(llama_mem, q, k, v, c["blk"])
        dq, dk, dv = torch.autograd.grad(out, [q, k, v], do)
        save(name + ".pt", q=q, k=k, v=v, do=do, out=out, dq=dq, dk=dk, dv=dv, blk=c["blk"])


# --------------------------------------------------------------------------- fused, Triton kernels
def gen_triton(fla):
    import triton
    for name, (Lq, Lk, D, blk, seed) in dict(triton_square=(128, 128, 32, 64, 21),
                                             triton_prefix=(64, 128, 16, 32, 22)).items():
        g = torch.Generator().manual_seed(seed)
        B, H = 1, 2
        q = torch.randn(B, H, Lq, D, generator=g)
        k = torch.randn(B, H, Lk, D, generator=g)
        v = torch.randn(B, H, Lk, D, generator=g)
        do = torch.randn(B, H, Lq, D, generator=g)
        scale = 1.0 / math.sqrt(D)
        npre = (Lk - Lq) // blk
        o = torch.empty_like(q)
        L = torch.empty(B * H, Lq); M = torch.empty(B * H, Lq)
        grid = (triton.cdiv(Lq, blk), B * H, 1)
        fla._fwd_kernel[grid](q, k, v, scale, o, *q.stride(), *k.stride(), *v.stride(), *o.stride(),
                              L, M, B, H, Lq, Lk, BLOCK=blk, BLOCK_DMODEL=D, N_PREFIX_Q=npre)
        dq = torch.zeros_like(q); dk = torch.empty_like(k); dv = torch.empty_like(v)
        do_s = torch.empty_like(do); delta = torch.empty_like(L)
        fla._bwd_preprocess[(grid[0], grid[1])](o, *o.stride(), do, L, L.stride(0), L.stride(1),
                                                do_s, delta, Lq, BLOCK_M=blk, D_HEAD=D)
        fla._bwd_kernel[(grid[1],)](q, k, v, scale, o, do_s, dq, dk, dv, L, M, delta,
                                    *q.stride(), *k.stride(), *v.stride(), B, H, Lq, Lk,
                                    BLOCK=blk, BLOCK_DMODEL=D, N_PREFIX_Q=npre)
        save(name + ".pt", q=q, k=k, v=v, do=do, out=o, L=L, M=M, dq=dq, dk=dk, dv=dv, blk=blk)


# --------------------------------------------------------------------------- grouped softmax
def random_is_mem(B, T, g, lo=3, hi=9):
    im = torch.zeros(B, T, dtype=torch.bool)
    for b in range(B):
        p = int(torch.randint(lo, hi, (1,), generator=g))
        while p < T:
            im[b, p] = True
            p += int(torch.randint(lo, hi, (1,), generator=g))
    return im


def gen_gsm_llama(llama_mem):
    g = torch.Generator().manual_seed(31)
    B, H, T = 2, 2, 48
    is_mem_row = random_is_mem(B, T, g)
    x = torch.randn(B, H, T, T, generator=g)
    gp = torch.randn(B, H, T, T, generator=g)
    fmin = torch.finfo(torch.float32).min
    attention_mask = torch.triu(torch.full((T, T), fmin), diagonal=1).view(1, 1, T, T).expand(B, 1, T, T).clone()
    # model-level preparation, llama_mem.py:807-815
    is_mem = is_mem_row.unsqueeze(1).unsqueeze(2)
    mem_ids = torch.where(attention_mask < -1, 0, torch.cumsum(is_mem, -1) - is_mem.int())
    last = torch.amax(mem_ids, -1, keepdim=True) == mem_ids
    attention_mask.masked_fill_(last & is_mem, fmin)
    last.logical_and_(attention_mask > -1)
    is_mem = is_mem.logical_and(attention_mask > -1)
    xin = torch.max(x + attention_mask, torch.tensor(fmin)).requires_grad_(True)
    probs = llama_mem.landmark_grouped_softmax(xin, dim=-1, is_mem=is_mem.expand(-1, H, -1, -1), last_section_mask=last)
    (gx,) = torch.autograd.grad(probs, [xin], gp)
    save("gsm_llama.pt", x=xin, is_mem=is_mem, last=last, is_mem_row=is_mem_row, probs=probs, gprobs=gp, gx=gx)


def gen_gsm_lm(landmark):
    g = torch.Generator().manual_seed(32)
    B, H, T = 2, 2, 48
    is_mem_row = random_is_mem(B, T, g)
    x = torch.randn(B, H, T, T, generator=g)
    gp = torch.randn(B, H, T, T, generator=g)
    attn_mask = torch.triu(torch.ones(T, T), diagonal=1).view(1, 1, T, T) == 1
    is_mem = is_mem_row.unsqueeze(1).unsqueeze(2).repeat((1, H, 1, 1))
    mem_ids = torch.where(attn_mask, 0., torch.cumsum(is_mem, -1) - is_mem.int())
    last = torch.amax(mem_ids, -1, keepdim=True) == mem_ids
    mask = attn_mask.logical_or(is_mem & last)
    last.logical_and_(~mask)
    is_mem = is_mem.logical_and(~mask)
    xin = x.masked_fill(mask, float("-inf")).requires_grad_(True)
    probs, group_prob = landmark.landmark_grouped_softmax(xin, dim=-1, is_mem=is_mem, attn_mask=mask,
                                                          last_section_mask=last, return_group_prob=True,
                                                          max_mem_cnt=20)
    (gx,) = torch.autograd.grad(probs, [xin], gp)
    save("gsm_lm.pt", x=xin, is_mem=is_mem, last=last, mask=mask, is_mem_row=is_mem_row, probs=probs,
         group_prob=group_prob, gprobs=gp, gx=gx, max_mem_cnt=20)


# --------------------------------------------------------------------------- lm_benchmark pieces
def lm_config(**kw):
    c = types.SimpleNamespace(n_embd=64, n_head=2, bias=False, dropout=0.0, sequence_length=64,
                              softmax_func="mem_opt", enable_rem_score=False, postpone_lm_cache=True,
                              max_groups_for_softmax=16, group_dropout=None, batch_size=2,
                              mem_cache_size=4, mem_cache_freq=7, cache_topk=2,
                              cache_selection_method="per_token_and_head", landmark_id=999)
    c.__dict__.update(kw)
    return c


def gen_lm_attn(landmark, rotary):
    g = torch.Generator().manual_seed(41)
    cfg = lm_config()
    B, T, H, D = 2, 64, cfg.n_head, cfg.n_embd // cfg.n_head
    attn = landmark.CausalSelfAttention(cfg, None)
    with torch.no_grad():
        attn.c_attn.weight.copy_(torch.randn(3 * cfg.n_embd, cfg.n_embd, generator=g) * 0.3)
        attn.c_proj.weight.copy_(torch.eye(cfg.n_embd))
    enc = rotary.RotaryPositionalEncoder(cfg)
    _, closure = enc(None)
    x = torch.randn(B, T, cfg.n_embd, generator=g, requires_grad=True)
    is_mem_row = random_is_mem(B, T, g, 5, 9)
    y, _ = attn(x, is_mem_row, closure, None, 0)
    gy = torch.randn(B, T, cfg.n_embd, generator=g)
    qkv = attn.c_attn(x)
    q, k, v = [t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(cfg.n_embd, dim=2)]
    qr = closure.adapt_queries(q, start_index=0)
    kr = closure.adapt_keys(k, start_index=0)
    qr.retain_grad(); kr.retain_grad(); v.retain_grad()
    # same graph again through the module's code but from the rotated tensors, to get their grads
    att = (qr @ kr.transpose(-2, -1)) * (1.0 / math.sqrt(D))
    bias = attn.bias[:, :, :T, :T]
    att = att.masked_fill(bias == 0, float("-inf"))
    attn_mask = bias == 0
    im = is_mem_row.unsqueeze(1).unsqueeze(2).repeat((1, H, 1, 1))
    mem_ids = torch.where(attn_mask, 0., torch.cumsum(im, -1) - im.int())
    last = torch.amax(mem_ids, -1, keepdim=True) == mem_ids
    mask = attn_mask.logical_or(im & last)
    last.logical_and_(~mask)
    im = im.logical_and(~mask)
    att = att.masked_fill(mask, float("-inf"))
    p, _ = landmark.landmark_grouped_softmax(att, dim=-1, is_mem=im, attn_mask=mask, last_section_mask=last,
                                             return_group_prob=False, max_mem_cnt=16)
    y2 = (p @ v).transpose(1, 2).contiguous().view(B, T, cfg.n_embd)
    assert torch.equal(y2, y), "module output differs from its own recipe"
    y2.backward(gy)
    save("lm_attn.pt", q_rot=qr, k_rot=kr, v=v, is_mem_row=is_mem_row, y=y,
         gy=gy, dq=qr.grad, dk=kr.grad, dv=v.grad)


def gen_lm_attn_cache(landmark, mem_cache, rotary):
    g = torch.Generator().manual_seed(43)
    cfg = lm_config()
    B, H, D, blk = cfg.batch_size, cfg.n_head, cfg.n_embd // cfg.n_head, cfg.mem_cache_freq + 1
    attn = landmark.CausalSelfAttention(cfg, None)
    attn.cache_storage = mem_cache.MemLMCacheStorage(cfg, attn)
    attn.eval()
    with torch.no_grad():
        attn.c_attn.weight.copy_(torch.randn(3 * cfg.n_embd, cfg.n_embd, generator=g) * 0.3)
        attn.c_proj.weight.copy_(torch.eye(cfg.n_embd))
    enc = rotary.RotaryPositionalEncoder(cfg)
    _, closure = enc(None)
    records, pos = [], 0
    with torch.no_grad():
        for T in (19, 16, 13, 24):
            x = torch.randn(B, T, cfg.n_embd, generator=g)
            is_mem = ((torch.arange(pos, pos + T) % blk) == blk - 1).view(1, T).expand(B, T).clone()
            start_index = min((pos - pos % blk) // blk, cfg.cache_topk + 1) * blk + pos % blk
            q, k, v = [t.view(B, T, H, D).transpose(1, 2) for t in attn.c_attn(x).split(cfg.n_embd, dim=2)]
            qr = closure.adapt_queries(q, start_index=start_index)
            kr = closure.adapt_keys(k, start_index=start_index)
            y, _ = attn(x, is_mem, closure, mem_cache.MemLMCacheContext(), start_index)
            records.append(dict(q_rot=qr.clone(), k_rot=kr.clone(), k=k.clone(), v=v.clone(), is_mem=is_mem,
                                start_index=start_index, y=y.clone()))
            pos += T
    save("lm_attn_cache.pt", records=records, capacity=cfg.mem_cache_size, blk=blk, top_k=cfg.cache_topk,
         method=cfg.cache_selection_method, max_groups=cfg.max_groups_for_softmax)


def gen_memcache(mem_cache, rotary):
    for method in ("per_token_and_head", "max_over_heads", "max_over_tokens"):
        g = torch.Generator().manual_seed(51)
        cfg = lm_config(cache_selection_method=method)
        B, H, D, blk = cfg.batch_size, cfg.n_head, cfg.n_embd // cfg.n_head, cfg.mem_cache_freq + 1
        store = mem_cache.MemLMCacheStorage(cfg, None)
        enc = rotary.RotaryPositionalEncoder(cfg)
        _, closure = enc(None)
        chunks, records = [19, 16, 13, 24], []
        pos = 0                                                  # absolute position incl. landmarks
        for ci, T in enumerate(chunks):
            k = torch.randn(B, H, T, D, generator=g)
            v = torch.randn(B, H, T, D, generator=g)
            q = torch.randn(B, H, T, D, generator=g)
            is_mem = ((torch.arange(pos, pos + T) % blk) == blk - 1).view(1, T).expand(B, T).clone()
            start_index = min((pos - pos % blk) // blk, cfg.cache_topk + 1) * blk + pos % blk
            att_prefix, d = store.retrieve_for_query(q, None, closure, start_index)
            records.append(dict(q=q, k=k, v=v, is_mem=is_mem, start_index=start_index,
                                att_prefix=att_prefix.clone(), v_prefix=d["v"].clone(),
                                is_mem_prefix=d["is_mem"].clone(),
                                cache_iter=store.cache_iter, cache_size=store.cache_size))
            store.store_in_cache(k, {"v": v, "is_mem": is_mem})
            pos += T
        save(f"memcache_{method}.pt", records=records, capacity=cfg.mem_cache_size, blk=blk,
             top_k=cfg.cache_topk, method=method)
    # id-level bookkeeping of MemLMCache
    cfg = lm_config()
    cache = mem_cache.MemLMCache(cfg)
    g = torch.Generator().manual_seed(52)
    recs = []
    for T in (10, 7, 15, 3):
        ids = torch.randint(0, 900, (2, T), generator=g)
        x, start_index, _ = cache(ids)
        feats = torch.randn(2, x.shape[1], 5, generator=g)
        recs.append(dict(ids=ids, out_ids=x.clone(), start_index=start_index, feats=feats,
                         stripped=cache.get_final_logits(feats).clone()))
    save("memcache_ids.pt", records=recs, mem_freq=cfg.mem_cache_freq, landmark_id=cfg.landmark_id,
         top_k=cfg.cache_topk)


# --------------------------------------------------------------------------- LLaMA retrieval branch
def gen_llama_retrieval(llama_mem, LlamaLandmarkConfig):
    for name, (C, T, seed) in dict(llama_retr_blocks=(40, 16, 61), llama_retr_tail=(43, 3, 62)).items():
        torch.manual_seed(seed)
        H, D, mem_freq, top_k = 2, 16, 7, 2
        blk = mem_freq + 1
        cfg = LlamaLandmarkConfig(vocab_size=64, hidden_size=H * D, intermediate_size=48, num_hidden_layers=1,
                                  num_attention_heads=H, max_position_embeddings=256, mem_id=63, mem_freq=mem_freq,
                                  pad_token_id=0, bos_token_id=1, eos_token_id=2)
        model = llama_mem.LlamaModel(cfg).eval()
        attn = model.layers[0].self_attn
        cap = {}
        attn.q_proj.register_forward_hook(lambda m, i, o: cap.__setitem__("q", o))
        attn.k_proj.register_forward_hook(lambda m, i, o: cap.__setitem__("k", o))
        attn.v_proj.register_forward_hook(lambda m, i, o: cap.__setitem__("v", o))
        attn.o_proj.register_forward_hook(lambda m, i, o: cap.__setitem__("attn_out", i[0]))
        ids = torch.randint(3, 60, (1, T))
        pos = torch.arange(C, C + T)
        ids[0, pos % blk == blk - 1] = cfg.mem_id
        past_k = torch.randn(1, H, C, D)
        past_v = torch.randn(1, H, C, D)
        with torch.no_grad():
            model(input_ids=ids, past_key_values=((past_k, past_v),), use_cache=True, use_flash=False,
                  cache_top_k=top_k, mem_freq=mem_freq)
        q = cap["q"].view(1, T, H, D).transpose(1, 2)
        k = cap["k"].view(1, T, H, D).transpose(1, 2)
        v = cap["v"].view(1, T, H, D).transpose(1, 2)
        out = cap["attn_out"].view(1, T, H, D).transpose(1, 2)
        save(name + ".pt", q=q, k=k, v=v, past_k=past_k, past_v=past_v, out=out, blk=blk, top_k=top_k,
             is_mem_row=(ids == cfg.mem_id))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LMK_REFERENCE_CHECKOUT", ""))
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    sys.path.insert(0, os.path.join(a.reference, "llama"))
    sys.path.insert(0, os.path.join(a.reference, "llama", "ltriton"))
    import llama_mem
    from llama_landmark_config import LlamaLandmarkConfig
    import flash_landmark_attention as fla
    sys.path.insert(0, os.path.join(a.reference, "lm_benchmark"))
    import tiktoken
    tiktoken.get_encoding = lambda name: None     # needs the network; only used for text generation
    from models import landmark
    from models.caches import mem_cache
    from models.positional_encoders import rotary
    steps = dict(fused=lambda: gen_fused(llama_mem), triton=lambda: gen_triton(fla),
                 gsm_llama=lambda: gen_gsm_llama(llama_mem), gsm_lm=lambda: gen_gsm_lm(landmark),
                 lm_attn=lambda: gen_lm_attn(landmark, rotary), memcache=lambda: gen_memcache(mem_cache, rotary),
                 lm_attn_cache=lambda: gen_lm_attn_cache(landmark, mem_cache, rotary),
                 llama_retr=lambda: gen_llama_retrieval(llama_mem, LlamaLandmarkConfig))
    for name, fn in steps.items():
        if a.only and name not in a.only.split(","):
            continue
        print("==", name)
        fn()


if __name__ == "__main__":
    main()
