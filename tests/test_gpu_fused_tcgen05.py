"""Parity of the tcgen05/TMEM fused landmark attention kernels (through the C ABI) against the CPU oracle.
bf16/fp16 tolerances: 2e-2 max-abs and 1e-2 relative L2 for outputs and gradients."""
import pytest
import torch

import landmark_attention_b200 as P
from landmark_attention_b200 import _lib as L
from oracle import landmark_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_l2(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


def make(B, H, Lq, Lk, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, Lq, 128, generator=g) * 0.5).to(dtype)
    k = (torch.randn(B, H, Lk, 128, generator=g) * 0.5).to(dtype)
    v = (torch.randn(B, H, Lk, 128, generator=g) * 0.5).to(dtype)
    do = torch.randn(B, H, Lq, 128, generator=g).to(dtype)
    return q, k, v, do


FWD_SHAPES = [(1, 1, 128, 128), (1, 2, 256, 256), (2, 2, 512, 512), (1, 2, 128, 320), (1, 1, 256, 448),
              (1, 1, 1024, 1024)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", FWD_SHAPES)
def test_forward_against_oracle(shape, dtype):
    B, H, Lq, Lk = shape
    q, k, v, _ = make(B, H, Lq, Lk, dtype, 7)
    out, l, m = P.attn_forward_with_stats(q.to(DEV), k.to(DEV), v.to(DEV), 64, path=P.PATH_TCGEN05)
    assert L.device_status() == 0
    exp, em, el = O.landmark_attention(q.float(), k.float(), v.float(), 64, return_stats=True)
    got = out.float().cpu()
    assert (got - exp).abs().max().item() < 2e-2
    assert rel_l2(got, exp) < 1e-2
    assert (m.cpu().view_as(em) - em).abs().max().item() < 1e-3
    assert ((l.cpu().view_as(el) - el).abs() / el).max().item() < 2e-3


def test_forward_matches_general_path_and_known_answers():
    q, k, v, _ = make(1, 4, 512, 512, torch.bfloat16, 8)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    a = P.fused_landmark_attention(q, k, v, None, path=P.PATH_TCGEN05)
    b = P.fused_landmark_attention(q, k, v, None, path=P.PATH_GENERAL)
    assert (a.float() - b.float()).abs().max().item() < 1.5e-2
    ones = torch.ones_like(v)
    o = P.fused_landmark_attention(q, k, ones, None, path=P.PATH_TCGEN05)
    assert (o.float() - 1).abs().max().item() < 1e-2                       # rows of P sum to one
    assert torch.equal(a[:, :, 0], v[:, :, 0])                            # first row sees only the first key
    assert L.device_status() == 0


def test_forward_strided_views():
    g = torch.Generator().manual_seed(9)
    B, H, Lq = 2, 3, 256
    q, k, v = [(torch.randn(B, Lq, H, 128, generator=g) * 0.5).to(torch.bfloat16).to(DEV).transpose(1, 2)
               for _ in range(3)]
    out = P.fused_landmark_attention(q, k, v, None, path=P.PATH_TCGEN05)
    exp = O.landmark_attention(q.float().cpu().contiguous(), k.float().cpu().contiguous(),
                               v.float().cpu().contiguous(), 64)
    assert (out.float().cpu() - exp).abs().max().item() < 2e-2
    assert L.device_status() == 0


def run_bwd(q, k, v, do, path):
    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qc, kc, vc, None, path=path)
    grads = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    return [t.detach().float().cpu() for t in (out, *grads)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", FWD_SHAPES)
def test_backward_against_oracle(shape, dtype):
    B, H, Lq, Lk = shape
    q, k, v, do = make(B, H, Lq, Lk, dtype, 11)
    res = run_bwd(q, k, v, do, P.PATH_TCGEN05)
    assert L.device_status() == 0
    exp = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), 64)
    for name, got, e in zip(("out", "dq", "dk", "dv"), res, exp):
        assert (got - e).abs().max().item() < 2e-2, name
        assert rel_l2(got, e) < 1e-2, name


def test_backward_properties():
    q, k, v, do = make(1, 2, 512, 512, torch.bfloat16, 12)
    a = run_bwd(q, k, v, do, P.PATH_TCGEN05)
    b = run_bwd(q, k, v, do, P.PATH_TCGEN05)
    for x, y in zip(a, b):
        assert torch.equal(x, y)                                   # no atomics: bit-reproducible
    assert a[3][:, :, 63::64].abs().max().item() == 0.0            # landmark keys carry no value weight
    g = run_bwd(q, k, v, do, P.PATH_GENERAL)
    for x, y in zip(a, g):
        assert (x - y).abs().max().item() < 2e-2
    assert L.device_status() == 0


@pytest.mark.parametrize("std", [3.0, 8.0])
def test_extreme_logits_stay_finite_and_match(std):
    # Logits with a spread of tens to hundreds of nats: in-block scores far above AND far below the landmark level, so
    # both softmax levels saturate.  Every block is stabilised with its own maximum; nothing may overflow or turn NaN.
    g = torch.Generator().manual_seed(21)
    B, H, Lq = 1, 2, 512
    q = (torch.randn(B, H, Lq, 128, generator=g) * std).to(torch.bfloat16)
    k = (torch.randn(B, H, Lq, 128, generator=g) * std).to(torch.bfloat16)
    v = (torch.randn(B, H, Lq, 128, generator=g) * 0.5).to(torch.bfloat16)
    do = torch.randn(B, H, Lq, 128, generator=g).to(torch.bfloat16)
    res = run_bwd(q, k, v, do, P.PATH_TCGEN05)
    assert L.device_status() == 0
    exp = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), 64)
    for name, got, e in zip(("out", "dq", "dk", "dv"), res, exp):
        assert torch.isfinite(got).all(), name
        tol = 2e-2 * max(1.0, e.abs().max().item())         # gradients w.r.t. q, k scale with the other operand
        assert (got - e).abs().max().item() < tol, name
        assert rel_l2(got, e) < 2e-2, name


def test_persistent_kernels_with_several_units_per_cta():
    # cap the persistent grid so that every CTA walks through many work units (cross-unit pipelining, phase counters)
    q, k, v, do = make(1, 3, 512, 640, torch.bfloat16, 13)
    ref = run_bwd(q, k, v, do, P.PATH_TCGEN05)
    try:
        for cap in (1, 2, 5):
            L.lib().lmk_debug_set_max_ctas(cap)
            got = run_bwd(q, k, v, do, P.PATH_TCGEN05)
            for a, b in zip(got, ref):
                assert torch.equal(a, b)
            assert L.device_status() == 0
    finally:
        L.lib().lmk_debug_set_max_ctas(0)


def test_auto_path_falls_back_for_operands_tma_cannot_address():
    # Shapes the tcgen05 kernels take, but operands they cannot: a view that starts 8 bytes into its storage, and a key
    # tensor whose heads are an expanded (stride 0) view.  AUTO must run the general kernels and give the same
    # result; an explicit tcgen05 request must be refused.
    q, k, v, do = make(1, 2, 256, 256, torch.bfloat16, 21)
    exp = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), 64)

    def shifted(t):      # same values, storage offset of 4 elements = 8 bytes
        buf = torch.empty(t.numel() + 4, dtype=t.dtype, device=DEV)
        view = buf[4:].view(t.shape)
        view.copy_(t)
        return view

    qs = shifted(q).requires_grad_(True)
    kc, vc = [t.to(DEV).requires_grad_(True) for t in (k, v)]
    assert qs.data_ptr() % 16 == 8
    out = P.fused_landmark_attention(qs, kc, vc, None)
    grads = torch.autograd.grad(out, [qs, kc, vc], do.to(DEV))
    for got, e in zip((out, *grads), exp):
        assert (got.detach().float().cpu() - e).abs().max().item() < 2e-2
    with pytest.raises(NotImplementedError):
        P.fused_landmark_attention(qs, kc, vc, None, path=P.PATH_TCGEN05)

    k1 = k[:, :1].to(DEV)
    kexp = k1.expand(1, 2, 256, 128)
    assert kexp.stride(1) == 0
    qc = q.to(DEV)
    out2 = P.fused_landmark_attention(qc, kexp, v.to(DEV), None)
    ref2 = P.fused_landmark_attention(qc, kexp.contiguous(), v.to(DEV), None, path=P.PATH_GENERAL)
    assert (out2.float() - ref2.float()).abs().max().item() < 2e-2
    assert L.device_status() == 0


def test_auto_path_selection():
    lib = L.lib()
    assert lib.lmk_attn_tcgen05_supported(1, 32, 2048, 2048, 128, 64, L.LMK_BF16) == 1
    assert lib.lmk_attn_tcgen05_supported(1, 32, 2048, 2048, 64, 64, L.LMK_BF16) == 0      # head dim
    assert lib.lmk_attn_tcgen05_supported(1, 32, 2048, 2048, 128, 32, L.LMK_BF16) == 0     # block size
    assert lib.lmk_attn_tcgen05_supported(1, 32, 2048, 2048, 128, 64, L.LMK_F32) == 0      # fp32 needs the CUDA-core path
    assert lib.lmk_attn_tcgen05_supported(1, 32, 192, 192, 128, 64, L.LMK_BF16) == 0       # not whole 128-row tiles
    # a non-positive softmax scale is legal for the operator but not for the tcgen05 kernels: AUTO falls back
    q, k, v, do = make(1, 2, 256, 256, torch.bfloat16, 14)
    qc, kc, vc = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = P.fused_landmark_attention(qc, kc, vc, None, sm_scale=-0.05)
    grads = torch.autograd.grad(out, [qc, kc, vc], do.to(DEV))
    exp = O.landmark_attention_grads(q.float(), k.float(), v.float(), do.float(), 64, sm_scale=-0.05)
    for got, e in zip((out, *grads), exp):
        assert (got.detach().float().cpu() - e).abs().max().item() < 2e-2
    with pytest.raises(NotImplementedError):
        P.fused_landmark_attention(qc, kc, vc, None, sm_scale=-0.05, path=P.PATH_TCGEN05)
