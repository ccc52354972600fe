"""lmk_attn_bwd_static: the backward entry point for callers that cannot allocate device memory (a plugin without an
allocator, code inside a no-allocation region, a real-time loop).  It must give the same gradients as lmk_attn_bwd,
call after call, while using only the scratch array built into the library.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _problem(B, H, Lq, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = [(torch.randn(B, H, Lq, D, generator=g) * 0.5).to(dtype).to(DEV) for _ in range(3)]
    do = torch.randn(B, H, Lq, D, generator=g).to(dtype).to(DEV)
    return q, k, v, do


def _backward(entry, q, k, v, do, path, block=64):
    """Forward through the C ABI, then one backward through `entry` ('workspace' or 'static')."""
    lib = L.lib()
    B, H, Lq, D = q.shape
    code = L.dtype_code(q)
    scale = D ** -0.5
    o = torch.empty_like(q)
    l = torch.empty(B * H, Lq, device=DEV)
    m = torch.empty(B * H, Lq, device=DEV)
    s3, st = L.strides3(q), L.stream_ptr(q.device)
    L.check(lib.lmk_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(l), L.ptr(m), B, H, Lq, Lq, D, s3, s3, s3,
                             block, scale, code, path, st), "lmk_attn_fwd")
    dq, dk, dv = [torch.full_like(q, float("nan")) for _ in range(3)]
    if entry == "workspace":
        need = lib.lmk_attn_bwd_workspace(B, H, Lq, Lq, D, block, code, path)
        ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=DEV)
        rc = lib.lmk_attn_bwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(do), L.ptr(l), L.ptr(m), L.ptr(dq), L.ptr(dk),
                              L.ptr(dv), L.ptr(ws), ws.numel(), B, H, Lq, Lq, D, s3, s3, s3, block, scale, code, path, st)
    else:
        rc = lib.lmk_attn_bwd_static(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(do), L.ptr(l), L.ptr(m), L.ptr(dq),
                                     L.ptr(dk), L.ptr(dv), B, H, Lq, Lq, D, s3, s3, s3, block, scale, code, path, st)
    L.check(rc, f"backward ({entry})")
    torch.cuda.synchronize()
    return dq, dk, dv


@pytest.mark.parametrize("path,dtype,shape", [(P.PATH_TCGEN05, torch.bfloat16, (1, 2, 512, 128)),
                                              (P.PATH_GENERAL, torch.float32, (2, 2, 256, 64))])
def test_static_scratch_backward_matches_workspace_backward(path, dtype, shape):
    B, H, Lq, D = shape
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    # two different problems back to back: the second call finds the first call's leftovers in the shared scratch
    for seed, batch in ((1, B), (2, B + 1)):
        q, k, v, do = _problem(batch, H, Lq, D, dtype, seed)
        expected = _backward("workspace", q, k, v, do, path)
        got = _backward("static", q, k, v, do, path)
        for name, a, b in zip(("dq", "dk", "dv"), got, expected):
            assert torch.isfinite(a.float()).all(), name
            assert (a.float() - b.float()).abs().max().item() <= tol, name
    assert L.device_status() == 0


def test_static_scratch_rejects_oversized_problems_without_launching():
    lib = L.lib()
    limit = lib.lmk_attn_bwd_static_max_rows()
    assert limit == 1 << 20
    one = ctypes.c_void_p(256)          # never dereferenced: the size check comes first
    s = L.I64x3(1, 1, 1)
    rows_h = 64                          # B*H*Lq = 64 * 32768 = 2 * limit
    rc = lib.lmk_attn_bwd_static(one, one, one, one, one, one, one, one, one, one, 1, rows_h, 32768, 32768, 128, s, s, s,
                                 64, 0.1, L.LMK_BF16, P.PATH_GENERAL, None)
    assert rc == L.LMK_ERR_WORKSPACE
    assert b"exceed the built-in scratch" in lib.lmk_last_error()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
def test_static_scratch_on_a_second_device():
    # every GPU has its own copy of the built-in array; its address is looked up per device, with that device current
    q0, k0, v0, do0 = _problem(1, 2, 256, 128, torch.bfloat16, 5)
    first = _backward("static", q0, k0, v0, do0, P.PATH_TCGEN05)          # device 0 resolves its address first
    with torch.cuda.device(1):
        q, k, v, do = _problem(1, 2, 256, 128, torch.bfloat16, 5)
        assert q.device.index == 1
        expected = _backward("workspace", q, k, v, do, P.PATH_TCGEN05)
        got = _backward("static", q, k, v, do, P.PATH_TCGEN05)
        for a, b in zip(got, expected):
            assert torch.equal(a, b)
        assert L.device_status() == 0
    for a, b in zip(first, got):
        assert torch.equal(a, b.to(a.device))
