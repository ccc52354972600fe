"""CPU-only checks: the C-ABI library loads, exports what include/b200lmk.h declares, rejects bad arguments before
touching a GPU, and the pure host logic matches the golden fixtures."""
import ctypes
import os
import re

import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L
from oracle import landmark_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200lmk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lmk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert "lmk_attn_fwd" in names and "lmk_gather_kv" in names
    handle = ctypes.CDLL(L.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in b200lmk.h but not exported"
    assert set(names) == set(L.PROTOTYPES), "ctypes prototypes and header disagree"
    assert P.lib().lmk_version() == 100


def test_attention_argument_checks_return_codes():
    lib = P.lib()
    s = L.I64x3(1, 1, 1)
    one = ctypes.c_void_p(256)     # never dereferenced: every call below must fail validation first
    def fwd(**kw):
        a = dict(q=one, k=one, v=one, o=one, l=one, m=one, B=1, H=1, Lq=64, Lk=64, D=64, blk=64, dt=L.LMK_BF16, path=0)
        a.update(kw)
        return lib.lmk_attn_fwd(a["q"], a["k"], a["v"], a["o"], a["l"], a["m"], a["B"], a["H"], a["Lq"], a["Lk"],
                                a["D"], s, s, s, a["blk"], 0.125, a["dt"], a["path"], None)
    assert fwd(q=None) == L.LMK_ERR_INVALID
    assert fwd(D=256) == L.LMK_ERR_INVALID and b"128" in lib.lmk_last_error()
    assert fwd(Lk=100) == L.LMK_ERR_INVALID          # history not a multiple of the block
    assert fwd(Lq=128, Lk=64) == L.LMK_ERR_INVALID
    assert fwd(dt=7) == L.LMK_ERR_INVALID
    assert fwd(path=L.PATH_TCGEN05) == L.LMK_ERR_UNSUPPORTED   # D=64 is not a tcgen05 shape
    rc = lib.lmk_attn_bwd(one, one, one, one, one, one, one, one, one, one, None, 0, 1, 1, 96, 96, 64, s, s, s, 64,
                          0.125, L.LMK_F32, L.PATH_GENERAL, None)
    assert rc == L.LMK_ERR_INVALID and b"full blocks" in lib.lmk_last_error()
    rc = lib.lmk_attn_bwd(one, one, one, one, one, one, one, one, one, one, None, 0, 1, 1, 64, 64, 64, s, s, s, 64,
                          0.125, L.LMK_F32, L.PATH_GENERAL, None)
    assert rc == L.LMK_ERR_WORKSPACE
    assert lib.lmk_attn_bwd_workspace(1, 2, 64, 64, 64, 64, L.LMK_F32, L.PATH_GENERAL) == 2 * 64 * 4


def test_retrieval_argument_checks():
    lib = P.lib()
    one = ctypes.c_void_p(256)
    d = L.CacheDesc(1, 1, 1, 1, 4, 0, 8, 9, 0)        # top_k > n_blocks
    rc = lib.lmk_landmark_scores(one, one, ctypes.byref(d), None, None, 0, 0, one, 1, 1, 1, 64, 1.0, 0, 0, None, 0, None)
    assert rc == L.LMK_ERR_INVALID
    assert lib.lmk_topk_sorted(one, one, 1, 1, 0, 0, 1, 0, 8, 9, 0, None) == L.LMK_ERR_INVALID
    d = L.CacheDesc(8, 8, 8, 8, 4, 0, 8, 2, 0)
    rc = lib.lmk_gather_kv(one, one, ctypes.byref(d), ctypes.byref(d), one, None, None, 0, L.ROTARY_HALF, one, one,
                           1, 1, 1, 64, L.LMK_BF16, None)
    assert rc == L.LMK_ERR_INVALID and b"rotary" in lib.lmk_last_error()
    # fused selected-block attention: row stride too small for top_k * block columns at the offset; odd head dim
    rc = lib.lmk_selected_logits(one, one, ctypes.byref(d), one, None, None, 0, L.ROTARY_NONE, one, 16, 4, 1, 1, 1, 64,
                                 1.0, L.LMK_BF16, None)
    assert rc == L.LMK_ERR_INVALID and b"row stride" in lib.lmk_last_error()
    rc = lib.lmk_selected_logits(one, one, ctypes.byref(d), one, None, None, 0, L.ROTARY_NONE, one, 16, 0, 1, 1, 1, 24,
                                 1.0, L.LMK_BF16, None)
    assert rc == L.LMK_ERR_INVALID
    assert lib.lmk_selected_pv(one, 8, 0, one, ctypes.byref(d), one, one, 1, 1, 1, 64, L.LMK_BF16, None) == L.LMK_ERR_INVALID
    assert lib.lmk_selected_pv(one, 16, 0, one, ctypes.byref(d), None, one, 1, 1, 1, 64, L.LMK_BF16, None) == L.LMK_ERR_INVALID


def test_python_wrappers_refuse_cpu_tensors():
    q = torch.randn(1, 1, 64, 64)
    with pytest.raises(AssertionError):
        P.fused_landmark_attention(q, q, q, None)
    with pytest.raises(AssertionError):        # same check as the reference: history must be whole blocks
        P.fused_landmark_attention(q, torch.randn(1, 1, 100, 64), torch.randn(1, 1, 100, 64), None)
    with pytest.raises(ValueError):
        P.landmark_sdpa(q, q, q, attn_mask=torch.ones(64, 64, dtype=torch.bool))


def test_landmark_id_bookkeeping_matches_reference(golden):
    g = golden("memcache_ids.pt")
    cfg = type("C", (), dict(mem_cache_freq=g["mem_freq"], landmark_id=g["landmark_id"], cache_topk=g["top_k"]))()
    cache = P.MemLMCache(cfg)
    for r in g["records"]:
        ids, start_index, _ = cache(r["ids"])
        assert torch.equal(ids, r["out_ids"]) and start_index == r["start_index"]
        assert torch.equal(cache.get_final_logits(r["feats"]), r["stripped"])


def test_mask_preparation_matches_reference(golden):
    g = golden("gsm_lm.pt")
    T = g["x"].shape[-1]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    mask, is_mem, last = P.prepare_landmark_masks(g["is_mem_row"], hidden)
    H = g["x"].shape[1]
    assert torch.equal(mask.expand(-1, H, -1, -1), g["mask"])
    assert torch.equal(is_mem.expand(-1, H, -1, -1), g["is_mem"])
    assert torch.equal(last.expand(-1, H, -1, -1), g["last"])


def test_rotary_tables_match_oracle():
    x = torch.randn(2, 3, 5, 16)
    pos = torch.tensor([0, 3, 7, 20, 31])
    cos, sin = P.rotary_tables_half(32, 16, torch.float32, "cpu")
    from landmark_attention_b200.retrieval import apply_rotary_half
    assert torch.allclose(apply_rotary_half(x, cos, sin, pos), O.rotary_half_split(x, pos.view(1, 1, 5)), atol=1e-6)
    cos, sin = P.rotary_tables_interleaved(32, 16, torch.float32, "cpu")
    from landmark_attention_b200.mem_cache import _rotate_interleaved
    ref = O.rotary_interleaved(x, pos.view(1, 1, 5).expand(2, 3, 5).to(torch.float32))
    assert torch.allclose(_rotate_interleaved(x, cos, sin, pos), ref, atol=1e-6)
