"""Parity of the retrieval kernels: landmark scores, top-k (bit-exact indices on identical fp32 scores), block gather
with rotary, the LLaMA cache branch and the lm_benchmark block cache."""
import ctypes
import math

import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("n,k", [(5, 2), (64, 4), (1024, 4), (1000, 8), (4096, 4), (33, 32)])
def test_topk_indices_bit_exact(n, k):
    torch.manual_seed(n + k)
    scores = torch.randn(2, 3, 17, n, device=DEV)
    got = P.topk_sorted(scores, k)
    exp = scores.topk(k, dim=-1).indices.sort(dim=-1).values
    assert torch.equal(got.long(), exp)


def test_topk_aggregations_and_ring_order():
    torch.manual_seed(0)
    s = torch.rand(2, 4, 9, 50, device=DEV)
    got = P.topk_sorted(s, 3, "max_over_tokens")
    exp = s.amax(dim=2, keepdim=True).topk(3, dim=-1).indices.sort(dim=-1).values
    assert torch.equal(got.long(), exp)
    got = P.topk_sorted(s, 3, "max_over_heads")
    exp = s.amax(dim=1, keepdim=True).topk(3, dim=-1).indices.sort(dim=-1).values
    assert torch.equal(got.long(), exp)
    # ring buffer: ascending by logical age, physical indices returned (mem_cache.py:73-83)
    ring = 20
    got = P.topk_sorted(s, 4, ring_start=ring).long()
    phys = s.topk(4, dim=-1).indices
    logical = torch.where(phys < ring, phys + 50 - ring, phys - ring).sort(dim=-1).values
    exp = torch.where(logical >= 50 - ring, logical - (50 - ring), logical + ring)
    assert torch.equal(got, exp)


@pytest.mark.parametrize("k", [3, 6])
def test_topk_with_ties_and_infinities(k):
    s = torch.full((1, 1, 4, 80), float("-inf"), device=DEV)
    s[0, 0, 0, 5] = 1.0
    s[0, 0, 1, :] = 0.5
    s[0, 0, 2, :] = torch.arange(80, device=DEV).float() % 7      # many exact ties spread over all lanes
    s[0, 0, 3, 40:] = float("nan")                                # NaN ranks lowest
    s[0, 0, 3, 77] = 2.0
    got = P.topk_sorted(s, k)
    assert got[0, 0, 0].tolist() == sorted([5] + list(range(k))[: k - 1] if 5 >= k - 1 else list(range(k)))
    assert got[0, 0, 1].tolist() == list(range(k))                # all equal: lowest indices
    assert got[0, 0, 2].tolist() == [6 + 7 * i for i in range(k)]
    assert got[0, 0, 3].tolist() == list(range(k - 1)) + [77]     # one finite value, then lowest indices among the rest


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scores_and_gather_llama_layout(dtype):
    torch.manual_seed(1)
    B, H, T, D, blk, nblk, top_k = 1, 3, 10, 64, 8, 12, 3
    C = nblk * blk
    q = torch.randn(B, H, T, D).to(dtype)
    pk = torch.randn(B, H, C, D).to(dtype)
    pv = torch.randn(B, H, C, D).to(dtype)
    prefix_len = C - (top_k + 1) * blk
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    pkc, pvc = pk.to(DEV), pv.to(DEV)
    st = pkc.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, prefix_len)
    scores = P.landmark_scores(q.to(DEV), pkc, desc, cos, sin, L.ROTARY_HALF)
    mem_pos, _ = O.llama_slot_positions(nblk, top_k, C, blk)
    lm = O.rotary_half_split(pk.view(B, H, nblk, blk, D)[:, :, :, blk - 1], mem_pos.view(1, 1, nblk))
    exp = torch.matmul(q.float(), lm.float().transpose(2, 3)) / math.sqrt(D)
    # Against the fp32-rotation oracle a bf16 run may differ by up to ~5e-2: the reference (and the kernel, on
    # purpose) rotates the landmark keys in bf16 -- x*cos + rotate_half(x)*sin with bf16 tables is three bf16
    # roundings per element -- before a 64-term dot product of N(0,1) values.  The 2e-2 bound of the attention
    # outputs does not apply to raw scores; the tight check is the next one.
    tol = 1e-4 if dtype == torch.float32 else 6e-2
    assert (scores.cpu() - exp).abs().max().item() < tol
    # closer to the reference's arithmetic in this dtype: keys rotated by torch on the same tables (rounded to the
    # dtype after every step), then an fp32 dot product.  The scoring kernel keeps the rotated key in fp32 (it skips
    # the last rounding), which leaves up to half a bf16 step on each of the 64 terms.
    from landmark_attention_b200.retrieval import apply_rotary_half as rot_same
    lm_same = rot_same(pk.view(B, H, nblk, blk, D)[:, :, :, blk - 1], cos.cpu(), sin.cpu(), mem_pos.view(1, 1, nblk))
    exp_same = torch.matmul(q.float(), lm_same.float().transpose(2, 3)) / math.sqrt(D)
    assert (scores.cpu() - exp_same).abs().max().item() < (1e-4 if dtype == torch.float32 else 1.5e-2)
    sel = P.topk_sorted(scores, top_k)
    assert torch.equal(sel.long(), scores.topk(top_k, dim=-1).indices.sort(dim=-1).values)
    sk, sv = P.gather_kv(pkc, pvc, desc, desc, sel, cos, sin, L.ROTARY_HALF)
    selc = sel.long().cpu()
    kpos = O.llama_selected_key_positions(selc, nblk, top_k, prefix_len, blk)
    gi = selc.view(B, H, T, top_k, 1, 1).expand(B, H, T, top_k, blk, D)
    ek = torch.take_along_dim(pk.view(B, H, 1, nblk, blk, D).expand(B, H, T, nblk, blk, D), gi, dim=3)
    ev = torch.take_along_dim(pv.view(B, H, 1, nblk, blk, D).expand(B, H, T, nblk, blk, D), gi, dim=3)
    ek = ek.reshape(B, H, T, top_k * blk, D)
    assert torch.equal(sv.cpu(), ev.reshape(B, H, T, top_k * blk, D))          # values: pure copy, bit-exact
    from landmark_attention_b200.retrieval import apply_rotary_half
    same_tables = apply_rotary_half(ek, cos.cpu(), sin.cpu(), kpos)            # torch arithmetic on the same tables
    assert torch.equal(sk.cpu(), same_tables)                                  # keys: same rounding steps as torch
    assert (sk.cpu().float() - O.rotary_half_split(ek.float(), kpos)).abs().max().item() < (1e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("materialize", [False, True])
@pytest.mark.parametrize("name", ["llama_retr_blocks", "llama_retr_tail"])
def test_llama_cache_branch_against_golden(golden, name, materialize):
    # materialize=True gathers the selected blocks as the reference does; False reads them in place (fused kernels)
    g = golden(name + ".pt")
    out, _ = P.llama_retrieval_attention(g["q"].to(DEV), g["k"].to(DEV), g["v"].to(DEV), g["past_k"].to(DEV),
                                         g["past_v"].to(DEV), g["blk"] - 1, g["top_k"],
                                         chunk_is_mem=g["is_mem_row"].to(DEV), materialize=materialize)
    assert (out.cpu() - g["out"]).abs().max().item() < 1e-5


@pytest.mark.parametrize("rotary", ["half", "interleaved", "none"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_selected_block_kernels_match_gather_then_matmul(dtype, rotary):
    # in-place logits / weighted value sums over the selected blocks == gather + rotary + matmul, on a ring-ordered
    # cache with ragged block size (24 rows: lanes 24..31 idle), written at a column offset into a wider buffer
    torch.manual_seed(5)
    B, H, T, D, blk, nblk, top_k, ring = 2, 3, 9, 64, 24, 11, 3, 4
    C = nblk * blk
    q = torch.randn(B, H, T, D).to(dtype).to(DEV)
    pk = torch.randn(B, H, C, D).to(dtype).to(DEV)
    pv = torch.randn(B, H, C, D).to(dtype).to(DEV)
    if rotary == "half":
        cos, sin, mode = *P.rotary_tables_half(C + T + 1, D, dtype, DEV), L.ROTARY_HALF
    elif rotary == "interleaved":
        cos, sin, mode = *P.rotary_tables_interleaved(C + T + 1, D, dtype, DEV), L.ROTARY_INTERLEAVED
    else:
        cos, sin, mode = None, None, L.ROTARY_NONE
    st = pk.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, ring, blk, top_k, C - (top_k + 1) * blk)
    scores = torch.randn(B, H, T, nblk, device=DEV)
    sel = P.topk_sorted(scores, top_k, ring_start=ring)
    sk, sv = P.gather_kv(pk, pv, desc, desc, sel, cos, sin, mode)
    scale = 0.3
    exp_logits = torch.matmul(q.float().unsqueeze(3), sk.float().transpose(3, 4)).squeeze(3) * scale
    col0, width = 5, top_k * blk + 12
    buf = torch.full((B, H, T, width), 7.0, dtype=dtype, device=DEV)
    P.selected_logits(q, pk, desc, sel, buf, col0, cos, sin, mode, scale)
    got = buf[..., col0:col0 + top_k * blk].float()
    tol = 1e-5 if dtype == torch.float32 else (6e-2 if dtype == torch.bfloat16 else 8e-3)
    assert (got - exp_logits).abs().max().item() < tol
    assert (buf[..., :col0] == 7).all() and (buf[..., col0 + top_k * blk:] == 7).all()       # nothing else touched
    probs = torch.softmax(torch.randn(B, H, T, width, device=DEV), dim=-1).to(dtype)
    out = P.selected_pv(probs, pv, desc, sel, col0)
    exp_out = torch.matmul(probs[..., col0:col0 + top_k * blk].float().unsqueeze(3), sv.float()).squeeze(3)
    assert (out.float() - exp_out).abs().max().item() < (1e-5 if dtype == torch.float32 else 1e-2)


def test_selected_block_kernels_per_head_selection():
    # max_over_tokens: one set of blocks per head, shared by every token of the chunk (indices expanded over tokens)
    torch.manual_seed(8)
    B, H, T, D, blk, nblk, top_k = 1, 3, 20, 64, 16, 24, 3
    C = nblk * blk
    dtype = torch.float32
    q = torch.randn(B, H, T, D, device=DEV)
    pk, pv = torch.randn(B, H, C, D, device=DEV), torch.randn(B, H, C, D, device=DEV)
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    st = pk.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, C - (top_k + 1) * blk)
    scores = P.landmark_scores(q, pk, desc, cos, sin, L.ROTARY_HALF)
    sel1 = P.topk_sorted(scores, top_k, mode="max_over_tokens")                       # [B,H,1,k]
    assert torch.equal(sel1[:, :, 0].long(), scores.amax(dim=2).topk(top_k, dim=-1).indices.sort(dim=-1).values)
    sel = sel1.expand(B, H, T, top_k).contiguous()
    sk, sv = P.gather_kv(pk, pv, desc, desc, sel1, cos, sin, L.ROTARY_HALF)          # [B,H,1,k*blk,D]
    buf = torch.empty((B, H, T, top_k * blk), dtype=dtype, device=DEV)
    P.selected_logits(q, pk, desc, sel, buf, 0, cos, sin, L.ROTARY_HALF)
    exp = torch.matmul(q, sk[:, :, 0].transpose(2, 3)) / math.sqrt(D)
    assert (buf - exp).abs().max().item() < 1e-4
    probs = torch.softmax(buf, dim=-1)
    out = P.selected_pv(probs, pv, desc, sel)
    assert (out - torch.matmul(probs, sv[:, :, 0])).abs().max().item() < 1e-5


def test_selected_block_kernels_config4_shape():
    # the long-context shape: D = 128, blocks of 32 rows, top-4 of 1024 blocks, one head group
    torch.manual_seed(6)
    B, H, T, D, blk, nblk, top_k = 1, 2, 64, 128, 32, 1024, 4
    C = nblk * blk
    dtype = torch.bfloat16
    q = torch.randn(B, H, T, D).to(dtype).to(DEV)
    pk = torch.randn(B, H, C, D).to(dtype).to(DEV)
    pv = torch.randn(B, H, C, D).to(dtype).to(DEV)
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    st = pk.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, C - (top_k + 1) * blk)
    sel = P.topk_sorted(P.landmark_scores(q, pk, desc, cos, sin, L.ROTARY_HALF), top_k)
    sk, sv = P.gather_kv(pk, pv, desc, desc, sel, cos, sin, L.ROTARY_HALF)
    buf = torch.empty((B, H, T, top_k * blk), dtype=dtype, device=DEV)
    P.selected_logits(q, pk, desc, sel, buf, 0, cos, sin, L.ROTARY_HALF)
    exp = torch.matmul(q.float().unsqueeze(3), sk.float().transpose(3, 4)).squeeze(3) / math.sqrt(D)
    assert (buf.float() - exp).abs().max().item() < 6e-2
    probs = torch.softmax(buf.float(), dim=-1).to(dtype)
    out = P.selected_pv(probs, pv, desc, sel)
    exp_out = torch.matmul(probs.float().unsqueeze(3), sv.float()).squeeze(3)
    assert (out.float() - exp_out).abs().max().item() < 2e-2


def test_llama_cache_branch_selected_blocks_match_oracle():
    torch.manual_seed(2)
    B, H, T, D, blk, C, top_k = 1, 4, 16, 32, 16, 16 * 40, 4
    q, k, v = [torch.randn(B, H, T, D) for _ in range(3)]
    pk, pv = torch.randn(B, H, C, D), torch.randn(B, H, C, D)
    out, _, dbg = P.llama_retrieval_attention(q.to(DEV), k.to(DEV), v.to(DEV), pk.to(DEV), pv.to(DEV), blk - 1, top_k,
                                              return_debug=True)
    exp, edbg = O.llama_retrieval_attention(q, k, v, pk, pv, blk, top_k, return_debug=True)
    assert (dbg["scores"].cpu() - edbg["scores"]).abs().max().item() < 1e-4
    assert torch.equal(dbg["sel"].long().cpu(), edbg["sel"])
    assert (out.cpu() - exp).abs().max().item() < 1e-4


@pytest.mark.parametrize("layout", ["reference", "head_major"])
@pytest.mark.parametrize("method", ["per_token_and_head", "max_over_heads", "max_over_tokens"])
def test_block_cache_against_golden(golden, method, layout):
    g = golden(f"memcache_{method}.pt")
    r0 = g["records"][0]
    B, H, _, D = r0["q"].shape
    cfg = type("C", (), dict(batch_size=B, mem_cache_size=g["capacity"], mem_cache_freq=g["blk"] - 1, n_head=H,
                             n_embd=H * D, cache_topk=g["top_k"], cache_selection_method=method))()
    store = P.MemLMCacheStorage(cfg, None, dtype=torch.float32, device=DEV, layout=layout)
    for r in g["records"]:
        att, d = store.retrieve_for_query(r["q"].to(DEV), None, None, r["start_index"])
        assert att.shape == r["att_prefix"].shape
        if att.numel():
            assert (att.cpu() - r["att_prefix"]).abs().max().item() < 1e-5
        assert torch.equal(d["is_mem"].cpu(), r["is_mem_prefix"])
        assert torch.equal(d["v"].cpu(), r["v_prefix"])
        assert (store.cache_iter, store.cache_size) == (r["cache_iter"], r["cache_size"])
        store.store_in_cache(r["k"].to(DEV), {"v": r["v"].to(DEV), "is_mem": r["is_mem"].to(DEV)})


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scores_on_tensor_cores(dtype):
    # D = 128, T >= 128 and n_blocks >= 128 take the tcgen05 scoring path (rotated landmarks staged in a workspace)
    torch.manual_seed(3)
    B, H, T, D, blk, nblk, top_k = 1, 3, 200, 128, 8, 160, 4
    C = nblk * blk
    q = torch.randn(B, H, T, D).to(dtype)
    pk = torch.randn(B, H, C, D).to(dtype)
    prefix_len = C - (top_k + 1) * blk
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    pkc = pk.to(DEV)
    st = pkc.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, prefix_len)
    assert L.lib().lmk_landmark_scores_workspace(B, H, T, D, nblk, L.dtype_code(q)) == B * H * nblk * D * 2
    scores = P.landmark_scores(q.to(DEV), pkc, desc, cos, sin, L.ROTARY_HALF)
    assert L.device_status() == 0
    mem_pos, _ = O.llama_slot_positions(nblk, top_k, C, blk)
    lm = O.rotary_half_split(pk.view(B, H, nblk, blk, D)[:, :, :, blk - 1], mem_pos.view(1, 1, nblk))
    exp = torch.matmul(q.float(), lm.float().transpose(2, 3)) / math.sqrt(D)
    assert (scores.cpu() - exp).abs().max().item() < 6e-2
    # same values as the CUDA-core kernel up to the rounding of the fp32 accumulation order
    n_pos = cos.shape[0]
    ref = torch.empty_like(scores)
    rc = L.lib().lmk_landmark_scores(L.ptr(q.to(DEV)), L.ptr(pkc), ctypes.byref(desc), L.ptr(cos), L.ptr(sin), n_pos,
                                     L.ROTARY_HALF, L.ptr(ref), B, H, T, D, 1.0 / math.sqrt(D), 0, L.dtype_code(q), None,
                                     0, L.stream_ptr(ref.device))
    L.check(rc, "lmk_landmark_scores")
    assert (scores - ref).abs().max().item() < 4e-2
    assert ((scores - ref).abs() > 0).float().mean().item() < 0.02
    sel = P.topk_sorted(scores, top_k)
    assert torch.equal(sel.long(), scores.topk(top_k, dim=-1).indices.sort(dim=-1).values)


def _blocks_attention_reference(q, pk, pv, sel, blk, key_pos, scale):
    """Attention over the selected blocks alone, each a closed landmark group (fp32 torch on CPU)."""
    B, H, T, D = q.shape
    top_k = sel.shape[-1]
    nblk = pk.shape[2] // blk
    gi = sel.view(B, H, T, top_k, 1, 1).expand(B, H, T, top_k, blk, D)
    ek = torch.take_along_dim(pk.view(B, H, 1, nblk, blk, D).expand(B, H, T, nblk, blk, D), gi, dim=3)
    ev = torch.take_along_dim(pv.view(B, H, 1, nblk, blk, D).expand(B, H, T, nblk, blk, D), gi, dim=3)
    ek = O.rotary_half_split(ek.reshape(B, H, T, top_k * blk, D).float(), key_pos).view(B, H, T, top_k, blk, D)
    logits = torch.einsum("bhtd,bhtird->bhtir", q.float(), ek) * scale
    inner = torch.softmax(logits[..., : blk - 1], dim=-1)
    outer = torch.softmax(logits[..., blk - 1], dim=-1)                       # over the landmarks of the blocks
    o_i = torch.einsum("bhtir,bhtird->bhtid", inner, ev.float()[..., : blk - 1, :])
    return torch.einsum("bhti,bhtid->bhtd", outer, o_i)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selected_attend_alone(dtype):
    # one kernel: logits of the selected blocks, softmax inside each block, outer softmax over their landmarks, value sums
    torch.manual_seed(8)
    B, H, T, D, blk, nblk, top_k = 2, 2, 7, 64, 8, 20, 3
    C = nblk * blk
    q = torch.randn(B, H, T, D).to(dtype)
    pk, pv = torch.randn(B, H, C, D).to(dtype), torch.randn(B, H, C, D).to(dtype)
    prefix_len = C - (top_k + 1) * blk
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    pkc, pvc = pk.to(DEV), pv.to(DEV)
    st = pkc.stride()
    desc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, prefix_len)
    sel = P.topk_sorted(P.landmark_scores(q.to(DEV), pkc, desc, cos, sin, L.ROTARY_HALF), top_k)
    out = P.selected_attend(q.to(DEV), pkc, pvc, desc, desc, sel, cos, sin, L.ROTARY_HALF)
    selc = sel.long().cpu()
    kpos = O.llama_selected_key_positions(selc, nblk, top_k, prefix_len, blk)
    exp = _blocks_attention_reference(q, pk, pv, selc, blk, kpos, 1.0 / math.sqrt(D))
    assert (out.float().cpu() - exp).abs().max().item() < (1e-4 if dtype == torch.float32 else 2e-2)


def test_retrieval_call_site_bf16_long_context_shape():
    # the long-context shape per head: cache of 32768 tokens in blocks of 32, chunk of 258, top-4 per (head, token), bf16.
    # Default route = fused (tensor-core local attention + one selected-block kernel); the oracle gets the kernel's own
    # selection (parity is defined given the same scores), which itself is checked bit-exactly against torch.topk.
    torch.manual_seed(12)
    B, H, T, D, blk, C, top_k = 1, 2, 258, 128, 32, 32768, 4
    dtype = torch.bfloat16
    q, k, v = [(torch.randn(B, H, T, D) * 0.5).to(dtype) for _ in range(3)]
    pk, pv = (torch.randn(B, H, C, D) * 0.5).to(dtype), torch.randn(B, H, C, D).to(dtype)
    qc, kc, vc, pkc, pvc = [t.to(DEV) for t in (q, k, v, pk, pv)]
    out_mat, _, dbg = P.llama_retrieval_attention(qc, kc, vc, pkc, pvc, blk - 1, top_k, return_debug=True)
    sel = dbg["sel"].long()
    assert torch.equal(sel, dbg["scores"].topk(top_k, dim=-1).indices.sort(dim=-1).values)
    out_fused, _ = P.llama_retrieval_attention(qc, kc, vc, pkc, pvc, blk - 1, top_k)
    out_inplace, _ = P.llama_retrieval_attention(qc, kc, vc, pkc, pvc, blk - 1, top_k, fused=False)
    exp = O.llama_retrieval_attention(q.float(), k.float(), v.float(), pk.float(), pv.float(), blk, top_k, sel=sel.cpu())
    for name, got in (("fused", out_fused), ("in place", out_inplace), ("materialised", out_mat)):
        err = (got.float().cpu() - exp).abs().max().item()
        assert err < 2e-2, f"{name}: {err}"
        rel = ((got.float().cpu() - exp).norm() / exp.norm()).item()
        assert rel < 1e-2, f"{name}: rel-L2 {rel}"
    # gather_kv at this shape against torch (values: pure copy; keys: torch's arithmetic on the same tables)
    nblk = C // blk
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    selc = sel[:, :, :16].cpu()
    kpos = O.llama_selected_key_positions(selc, nblk, top_k, C - (top_k + 1) * blk, blk)
    gi = selc.view(B, H, 16, top_k, 1, 1).expand(B, H, 16, top_k, blk, D)
    ek = torch.take_along_dim(pk.view(B, H, 1, nblk, blk, D).expand(B, H, 16, nblk, blk, D), gi, dim=3)
    ev = torch.take_along_dim(pv.view(B, H, 1, nblk, blk, D).expand(B, H, 16, nblk, blk, D), gi, dim=3)
    from landmark_attention_b200.retrieval import apply_rotary_half
    assert torch.equal(dbg["sel_v"][:, :, :16].cpu(), ev.reshape(B, H, 16, top_k * blk, D))
    assert torch.equal(dbg["sel_k"][:, :, :16].cpu(),
                       apply_rotary_half(ek.reshape(B, H, 16, top_k * blk, D), cos.cpu(), sin.cpu(), kpos))
    assert L.device_status() == 0


def test_preallocated_cache_appends_in_place():
    torch.manual_seed(13)
    B, H, D, blk, top_k = 1, 2, 128, 32, 2
    dtype = torch.bfloat16
    C0, T = 32 * 6, 64
    pk, pv = [torch.randn(B, H, C0, D).to(dtype).to(DEV) for _ in range(2)]
    chunks = [[torch.randn(B, H, T, D).to(dtype).to(DEV) for _ in range(3)] for _ in range(2)]
    cache = P.LandmarkKVCache(B, H, C0 + 2 * T, D, dtype, DEV)
    cache.append(pk, pv)
    base_k = cache.k.data_ptr()
    past = (pk, pv)
    for q, k, v in chunks:
        ref, past = P.llama_retrieval_attention(q, k, v, past[0], past[1], blk - 1, top_k)
        got, views = P.llama_retrieval_attention(q, k, v, mem_freq=blk - 1, cache_top_k=top_k, cache=cache)
        assert torch.equal(ref, got)
        assert views[0].data_ptr() == base_k and views[0].shape[2] == past[0].shape[2]
        assert torch.equal(views[0], past[0]) and torch.equal(views[1], past[1])


def test_max_over_tokens_route():
    # one block selection per head (softmax of the scores, maximum over the chunk's tokens), selected blocks prepended
    # to the chunk, regular fused landmark attention with top_k history blocks
    torch.manual_seed(14)
    B, H, T, D, blk, nblk, top_k = 1, 3, 32, 32, 16, 12, 2
    C = nblk * blk
    q, k, v = [torch.randn(B, H, T, D) for _ in range(3)]
    pk, pv = torch.randn(B, H, C, D), torch.randn(B, H, C, D)
    out, _, dbg = P.llama_retrieval_attention(q.to(DEV), k.to(DEV), v.to(DEV), pk.to(DEV), pv.to(DEV), blk - 1, top_k,
                                              aggregate="max_over_tokens", return_debug=True)
    pos = torch.arange(C, C + T)
    qr, kr = O.rotary_half_split(q, pos.view(1, 1, T)), O.rotary_half_split(k, pos.view(1, 1, T))
    mem_pos, prefix_len = O.llama_slot_positions(nblk, top_k, C, blk)
    lm = O.rotary_half_split(pk.view(B, H, nblk, blk, D)[:, :, :, blk - 1], mem_pos.view(1, 1, nblk))
    probs = torch.softmax(torch.matmul(qr, lm.transpose(2, 3)) / math.sqrt(D), dim=-1)
    sel = O.sorted_topk(probs.amax(dim=2, keepdim=True), top_k)                       # [B,H,1,top_k]
    assert torch.equal(dbg["sel"].long().cpu(), sel)
    kpos = O.llama_selected_key_positions(sel, nblk, top_k, prefix_len, blk)
    gi = sel.view(B, H, 1, top_k, 1, 1).expand(B, H, 1, top_k, blk, D)
    ek = torch.take_along_dim(pk.view(B, H, 1, nblk, blk, D), gi, dim=3).reshape(B, H, 1, top_k * blk, D)
    ev = torch.take_along_dim(pv.view(B, H, 1, nblk, blk, D), gi, dim=3).reshape(B, H, top_k * blk, D)
    ek = O.rotary_half_split(ek, kpos).view(B, H, top_k * blk, D)
    exp = O.landmark_attention(qr, torch.cat((ek, kr), 2), torch.cat((ev, v), 2), blk)
    assert (out.cpu() - exp).abs().max().item() < 1e-4


def test_offloaded_cache_reads_only_selected_blocks_from_host():
    # whole blocks in pinned host memory, landmark keys on the device; same attention as the device-resident cache
    torch.manual_seed(15)
    B, H, D, blk, top_k = 1, 3, 64, 16, 2
    dtype = torch.float32
    C0, T = blk * 10, 32
    pk, pv = torch.randn(B, H, C0, D).to(DEV), torch.randn(B, H, C0, D).to(DEV)
    off = P.OffloadedLandmarkCache(B, H, 16, blk, D, dtype, DEV)
    off.append(pk, pv)
    assert off.n_blocks == 10 and off.tail_len == 0 and off.k_host.is_pinned() and not off.k_host.is_cuda
    past = (pk, pv)
    for step in range(2):
        q, k, v = [torch.randn(B, H, T, D).to(DEV) for _ in range(3)]
        ref, past, dbg = P.llama_retrieval_attention(q, k, v, past[0], past[1], blk - 1, top_k,
                                                     aggregate="max_over_tokens", return_debug=True)
        got, odbg = off.attend(q, k, v, top_k, return_debug=True)
        assert torch.equal(odbg["sel"], dbg["sel"])
        assert torch.equal(odbg["sel_k"], dbg["sel_k"]) and torch.equal(odbg["sel_v"], dbg["sel_v"])
        assert torch.equal(got, ref)
    torch.cuda.synchronize()
    assert off.n_blocks == 14
    assert torch.equal(off.k_host[:, :, :off.length].to(DEV), past[0])
    assert torch.equal(off.lm_keys[:, :, :off.n_blocks], past[0][:, :, blk - 1::blk])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_chunk_prepare_equals_the_tensor_formulation(dtype):
    # rotary with the same three roundings, zero padding rows, flags, and the append of the un-rotated rows: bit-exact
    from landmark_attention_b200.retrieval import apply_rotary_half, chunk_prepare
    torch.manual_seed(21)
    B, H, T, D, blk, C = 2, 3, 77, 128, 32, 96
    q, k, v = [torch.randn(B, H, T, D).to(dtype).to(DEV) for _ in range(3)]
    k = k.transpose(1, 2).contiguous().transpose(1, 2)          # a strided input
    cos, sin = P.rotary_tables_half(C + T + 1, D, dtype, DEV)
    cache = P.LandmarkKVCache(B, H, C + T + 5, D, dtype, DEV)
    cache.k.zero_(); cache.v.zero_()
    cache.length = C
    q_rot, q_pad, k_pad, v_pad, flags = chunk_prepare(q, k, v, cos, sin, C, None, blk, 128, cache)
    pos = torch.arange(C, C + T, device=DEV)
    eq, ek = apply_rotary_half(q, cos, sin, pos), apply_rotary_half(k, cos, sin, pos)
    assert torch.equal(q_rot, eq)
    for got, exp in ((q_pad, eq), (k_pad, ek), (v_pad, v)):
        assert torch.equal(got[:, :, :T], exp) and not got[:, :, T:].any()
    ef = torch.zeros(B, 128, dtype=torch.uint8, device=DEV)
    ef[:, :T] = (pos % blk == blk - 1).to(torch.uint8)
    assert torch.equal(flags, ef)
    assert cache.length == C + T
    assert torch.equal(cache.k[:, :, C:C + T], k) and torch.equal(cache.v[:, :, C:C + T], v)
    assert not cache.k[:, :, :C].any() and not cache.k[:, :, C + T:].any()
    # explicit flags, no cache
    given = torch.rand(1, T, device=DEV) < 0.2
    _, _, _, _, flags2 = chunk_prepare(q, k, v, cos, sin, C, given, blk, 128)
    assert torch.equal(flags2[:, :T], given.to(torch.uint8).expand(B, T)) and not flags2[:, T:].any()


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rotary_apply_equals_the_tensor_formulation(dtype, interleaved):
    # q and k of one layer in one launch, strided [B,T,H,D] projections viewed as [B,H,T,D]; 16-bit results bit-exact
    # against x * cos + rotate(x) * sin in the tensor dtype; the backward pass against autograd of that formulation
    torch.manual_seed(31)
    B, H, T, D, pos0 = 2, 3, 70, 64, 5
    qkv = torch.randn(B, T, 3 * H * D).to(dtype).to(DEV)
    q, k, _ = [t.view(B, T, H, D).transpose(1, 2) for t in qkv.split(H * D, dim=2)]
    tables = P.rotary_tables_interleaved if interleaved else P.rotary_tables_half
    cos, sin = tables(pos0 + T, D, dtype, DEV)
    c, s = cos[pos0:pos0 + T], sin[pos0:pos0 + T]

    def rotate(x):
        if interleaved:
            xr = x.reshape(*x.shape[:-1], -1, 2)
            return torch.stack((-xr[..., 1], xr[..., 0]), dim=-1).reshape(x.shape)
        return torch.cat((-x[..., D // 2:], x[..., : D // 2]), dim=-1)

    qd, kd = q.detach().clone().requires_grad_(True), k.detach().clone().requires_grad_(True)
    eq, ek = qd * c + rotate(qd) * s, kd * c + rotate(kd) * s
    qg, kg = q.detach().requires_grad_(True), k.detach().requires_grad_(True)
    gq, gk_ = P.rotary_apply(qg, kg, cos, sin, pos0, interleaved=interleaved)
    if dtype == torch.float32:
        assert (gq - eq).abs().max().item() < 1e-6 and (gk_ - ek).abs().max().item() < 1e-6
    else:
        assert torch.equal(gq, eq) and torch.equal(gk_, ek)
    wq, wk = torch.randn_like(eq), torch.randn_like(ek)
    e_dq, e_dk = torch.autograd.grad((eq.float() * wq.float()).sum() + (ek.float() * wk.float()).sum(), [qd, kd])
    g_dq, g_dk = torch.autograd.grad((gq.float() * wq.float()).sum() + (gk_.float() * wk.float()).sum(), [qg, kg])
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (g_dq.float() - e_dq.float()).abs().max().item() < tol
    assert (g_dk.float() - e_dk.float()).abs().max().item() < tol


@pytest.mark.parametrize("n,k", [(1024, 4), (1000, 7), (256, 32), (64, 1), (1024, 16)])
def test_topk_register_rows_ties_runs_and_ring(n, k):
    # rows of at most 1024 scores take the register-resident selection (threshold from the lanes' maxima, a few
    # candidates); runs of equal scores overflow the candidate buffer and must fall back to the general selection with
    # the same result; bf16-rounded scores (many exact ties), -inf / NaN tails and a ring start are covered
    g = torch.Generator(device=DEV).manual_seed(n * 31 + k)
    s = torch.randn(3, 2, 9, n, device=DEV, generator=g)
    s[0] = s[0].to(torch.bfloat16).float() * 0.25                # coarse values: ties everywhere
    s[1, 0, 0] = 0.5                                             # all equal: lowest indices win
    s[1, 0, 1, : n // 2] = 3.0                                   # a run longer than the candidate buffer
    s[1, 0, 2, 5:] = float("-inf")
    s[1, 0, 3, 3:] = float("nan")
    exp = torch.where(s != s, torch.full_like(s, float("-inf")), s)
    # reference order: value descending, index ascending (a stable sort on the negated values)
    order = torch.sort(-exp, dim=-1, stable=True).indices[..., :k]
    for ring in (0, n // 3):
        got = P.topk_sorted(s, k, ring_start=ring).long()
        logical = torch.where(order < ring, order + n - ring, order - ring).sort(dim=-1).values
        want = torch.where(logical >= n - ring, logical - (n - ring), logical + ring)
        assert torch.equal(got, want), f"ring {ring}"


def test_selected_attend_with_equal_table_halves_reads_half_of_them():
    # tables built as cat(freqs, freqs) take LMK_ROTARY_HALF_SYM (second halves not read): same output bit for bit as
    # the general rotate-half mode; tables without that property stay on the general mode
    from landmark_attention_b200 import retrieval as R
    torch.manual_seed(5)
    B, H, T, D, blk, nblk, top_k = 1, 2, 130, 128, 32, 40, 4
    C = nblk * blk
    q = (torch.randn(B, H, T, D) * 0.5).to(torch.bfloat16).to(DEV)
    pk, pv = [torch.randn(B, H, C, D).to(torch.bfloat16).to(DEV) for _ in range(2)]
    cos, sin = P.rotary_tables_half(C + T + 1, D, torch.bfloat16, DEV)
    st = pk.stride()
    kdesc = L.CacheDesc(st[0], st[1], st[2] * blk, st[2], nblk, 0, blk, top_k, C - (top_k + 1) * blk)
    sel = P.topk_sorted(P.landmark_scores(q, pk, kdesc, cos, sin, L.ROTARY_HALF), top_k)
    assert R._halves_equal(cos, sin)
    got = P.selected_attend(q, pk, pv, kdesc, kdesc, sel, cos, sin, L.ROTARY_HALF)          # upgraded to the SYM mode
    cos2, sin2 = cos.clone(), sin.clone()
    cos2[0, D // 2:] += 0.5                                                                   # position 0 is never used
    assert not R._halves_equal(cos2, sin2)
    ref = P.selected_attend(q, pk, pv, kdesc, kdesc, sel, cos2, sin2, L.ROTARY_HALF)        # general mode
    assert torch.equal(got, ref)
